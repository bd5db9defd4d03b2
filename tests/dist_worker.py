"""One rank of a CPU (gloo) multi-process test.  Launched by tests/test_dist_cpu.py.

Oracle: the same model trained in the same process with plain eager PyTorch on the
FULL global batch (every rank can compute it, inputs come from a shared seed)."""
import copy
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("RANNC_FORCE_CPU", "1")

import torch  # noqa: E402
import torch.nn as nn  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from tests import zoo  # noqa: E402


def main():
    import faulthandler
    if os.environ.get("RANNC_TEST_DUMP"):
        faulthandler.dump_traceback_later(int(os.environ["RANNC_TEST_DUMP"]), exit=True)
    case = json.loads(sys.argv[1])
    torch.manual_seed(case.get("seed", 0))
    rank, world = pyrannc.get_rank(), pyrannc.get_world_size()
    if case.get("dist_param"):
        # every rank declares the model but keeps 1/world of each parameter until deployment
        with pyrannc.DistributeModelParams():
            model = zoo.build(case["model"])
        torch.manual_seed(case.get("seed", 0))
        ref = zoo.build(case["model"])
    else:
        model = zoo.build(case["model"])
        ref = copy.deepcopy(model)
    lr = 0.05
    mk = (lambda ps: torch.optim.SGD(ps, lr=lr, momentum=0.9)) if case.get("opt", "sgd") == "sgd" else \
        (lambda ps: torch.optim.Adam(ps, lr=0.01))
    has_params = any(True for _ in model.parameters())
    if case.get("two_groups"):
        # biases first (no decay), then the matrices (decay): not the model's parameter order
        def groups(m):
            ps = list(m.named_parameters())
            return [{"params": [p for n, p in ps if p.dim() < 2], "weight_decay": 0.0},
                    {"params": [p for n, p in ps if p.dim() >= 2], "weight_decay": 0.01}]

        mk2 = lambda gs: torch.optim.Adam(gs, lr=0.01)  # noqa: E731
        opt, ropt = mk2(groups(model)), mk2(groups(ref))
    else:
        opt, ropt = (mk(model.parameters()), mk(ref.parameters())) if has_params else (None, None)
    wrapped = pyrannc.RaNNCModule(model, opt, enable_apex_amp=case.get("amp", False),
                                  enable_zero=case.get("zero", False), check_unused_values=False,
                                  allreduce_amp_master_params=case.get("ar_master", False),
                                  gather_inputs=case.get("gather_inputs", True))
    whole = not case.get("gather_inputs", True)    # every rank passes (rank 0's copy of) the whole batch
    B = case.get("batch", 8)
    lb = B // world
    g = torch.Generator().manual_seed(123)
    accum = case.get("accum", 1)
    tol = case.get("tol", 1e-4)
    ok = True
    msgs = []
    for it in range(case.get("iters", 3)):
        pyrannc.delay_grad_allreduce(accum > 1)
        for a in range(accum):
            inputs = zoo.inputs(case["model"], B, g)
            local = inputs if whole else tuple(t[rank * lb:(rank + 1) * lb] for t in inputs)
            if case.get("input_grad"):
                local = tuple(t.clone().requires_grad_(True) if t.is_floating_point() else t for t in local)
                inputs = tuple(t.clone().requires_grad_(True) if t.is_floating_point() else t for t in inputs)
            out = wrapped(*local)
            rout = ref(*inputs)
            if case.get("bad_upstream") and out.dim() == 0:
                # interleave_backward ran the backward passes assuming d(loss) = 1: anything else must be refused
                try:
                    (out * 2.0).backward()
                    ok = False
                    msgs.append("a scaled loss was accepted although the backward passes had already run")
                except RuntimeError as e:
                    if "interleave_backward" not in str(e):
                        ok = False
                        msgs.append(f"unexpected error: {e}")
                res = {"ok": ok, "msgs": msgs[:8], "stages": len(wrapped._dep.fwd_graph_order), "interleaved": 1,
                       "pipeline": wrapped._dep.pipeline_num}
                all_res = pyrannc._comm.allgather_obj(res)
                if rank == 0:
                    print("RESULT " + json.dumps({"ok": all(r["ok"] for r in all_res), "ranks": all_res}))
                pyrannc.barrier()
                pyrannc.clear()
                sys.exit(0 if all(r["ok"] for r in all_res) else 1)
            if out.dim() == 0:
                if abs(float(out) - float(rout)) > tol * max(1.0, abs(float(rout))):
                    ok = False
                    msgs.append(f"it {it}: loss {float(out)} vs {float(rout)}")
                out.backward()
                rout.backward()
            else:
                expect = rout if whole else rout[rank * lb:(rank + 1) * lb]
                if out.shape != expect.shape or not torch.allclose(out.float(), expect.float(), rtol=tol, atol=tol):
                    ok = False
                    msgs.append(f"it {it}: output mismatch {tuple(out.shape)} vs {tuple(expect.shape)}")
                go = torch.randn(rout.shape, generator=g)
                if not rout.requires_grad:
                    # a parameter-free model fed inputs that need no gradient: forward only
                    if out.requires_grad:
                        ok = False
                        msgs.append(f"it {it}: output requires grad although nothing it depends on does")
                    continue
                out.backward((go if whole else go[rank * lb:(rank + 1) * lb]).to(out.dtype))
                # DDP semantics: gradients are averaged over the ranks
                rout.backward(go / world)
                if case.get("input_grad"):
                    for tl, tf in zip(local, inputs):
                        if tl.is_floating_point():
                            want = tf.grad[rank * lb:(rank + 1) * lb] * world
                            if tl.grad is None or not torch.allclose(tl.grad, want, rtol=tol * 10, atol=tol * 10):
                                ok = False
                                msgs.append(f"it {it}: input gradient differs")
        if accum > 1:
            wrapped.allreduce_grads_zero() if case.get("zero") else wrapped.allreduce_grads()
        for n, p in ref.named_parameters():
            if p.grad is None:
                continue
            gr = wrapped.get_param_grad(n)
            if not torch.allclose(gr.float(), p.grad.float(), rtol=tol * 10, atol=tol * 10):
                ok = False
                msgs.append(f"it {it}: grad {n} differs by {(gr.float() - p.grad.float()).abs().max().item()}")
        if case.get("clip"):
            got = wrapped.clip_grad_norm(case["clip"])
            want = float(torch.nn.utils.clip_grad_norm_(ref.parameters(), case["clip"]))
            if abs(got - want) > tol * 10 * max(1.0, want):
                ok = False
                msgs.append(f"it {it}: grad norm {got} vs {want}")
        if opt is not None:
            opt.step()
            ropt.step()
            opt.zero_grad()
            ropt.zero_grad()
        for n, p in ref.named_parameters():
            v = wrapped.get_param(n)
            if not torch.allclose(v.float(), p.detach().float(), rtol=tol * 10, atol=tol * 10):
                ok = False
                msgs.append(f"it {it}: param {n} differs by {(v.float() - p.detach().float()).abs().max().item()}")
    if case.get("accessors") and has_params:
        # the reference's lower-level accessors: per-rank segments tile each parameter exactly once over its
        # owners, sync_param agrees with get_param, _sync_orig_params writes the trained values into the model
        for n, p in ref.named_parameters():
            full = wrapped.get_param(n, amp_master_param=True)
            a, b = wrapped.get_local_param_range(n)
            seg = wrapped.get_local_param_segment(n)
            cover = torch.zeros(full.numel())
            if b > a:
                if seg is None or seg.numel() != b - a or \
                        not torch.allclose(seg.detach().float().cpu().view(-1), full.view(-1)[a:b].float(),
                                           rtol=tol * 10, atol=tol * 10):
                    ok = False
                    msgs.append(f"local segment of {n} [{a}, {b}) does not match the parameter")
                cover[a:b] = 1.0
            tot = pyrannc._comm.allgather_obj(float(cover.sum()))
            owners = len(wrapped._storage.param_ranks[n])
            want_total = full.numel() * (1 if case.get("zero") else owners)
            if rank == 0 and abs(sum(tot) - want_total) > 0.5:
                ok = False
                msgs.append(f"segments of {n} cover {sum(tot)} elements, expected {want_total}")
            if not torch.equal(wrapped.sync_param(n), wrapped.get_param(n)):
                ok = False
                msgs.append(f"sync_param({n}) differs from get_param")
        wrapped._sync_orig_params(sync_all_ranks=True)
        for (n, p), (_, q) in zip(ref.named_parameters(), model.named_parameters()):
            if q.numel() != p.numel() or not torch.allclose(q.detach().float().cpu().view(-1),
                                                            p.detach().float().view(-1), rtol=tol * 10,
                                                            atol=tol * 10):
                ok = False
                msgs.append(f"_sync_orig_params left {n} different from the trained value")
    # checkpoint round trip
    sd = wrapped.state_dict()
    osd = opt.state_dict(from_global=True) if opt is not None else {"state": {}}
    if rank == 0:
        for n, p in ref.named_parameters():
            if not torch.allclose(sd[n].float(), p.detach().float(), rtol=tol * 10, atol=tol * 10):
                ok = False
                msgs.append(f"state_dict {n} differs")
        for n, b in ref.named_buffers():
            if n not in sd or not torch.allclose(sd[n].float(), b.float(), rtol=tol * 10, atol=tol * 10):
                ok = False
                msgs.append(f"state_dict buffer {n} differs or is missing")
        rsd = ropt.state_dict() if ropt is not None else {"state": {}}
        for k, st in rsd["state"].items():
            for item, v in st.items():
                if torch.is_tensor(v) and item != "step":
                    if k not in osd["state"] or item not in osd["state"][k]:
                        ok = False
                        msgs.append(f"optimizer state {k}/{item} missing")
                    elif not torch.allclose(osd["state"][k][item].float(), v.float(), rtol=tol * 10, atol=tol * 10):
                        ok = False
                        msgs.append(f"optimizer state {k}/{item} differs")
    if opt is not None and case.get("two_groups") and rank == 0:
        # the gathered dict must load into a plain optimizer over the eager copy and carry the same moments
        fresh = torch.optim.Adam(groups(ref), lr=0.01)
        fresh.load_state_dict(osd)
        for gi, g_ in enumerate(fresh.param_groups):
            for p in g_["params"]:
                a = fresh.state[p]["exp_avg"].float()
                b = ropt.state[p]["exp_avg"].float()
                if a.shape != b.shape or not torch.allclose(a, b, rtol=tol * 10, atol=tol * 10):
                    ok = False
                    msgs.append(f"two_groups: exp_avg of a parameter of group {gi} differs after loading into torch")
    if opt is not None:
        osd = pyrannc.comm_utils.bcast_obj(osd, 0)
        opt.load_state_dict(osd, from_global=True)
    if case.get("reload"):
        # load other values into the DEPLOYED module (every rank passes the same dict), then train one more step
        # in lockstep with the eager copy
        sd = pyrannc.comm_utils.bcast_obj(sd, 0)
        new_sd = {k: (v.float() * 0.5).to(v.dtype) if v.is_floating_point() else v for k, v in sd.items()}
        wrapped.load_state_dict(new_sd)
        ref.load_state_dict(new_sd)
        for n, p in ref.named_parameters():
            v = wrapped.get_param(n)
            if not torch.allclose(v.float(), p.detach().float(), rtol=tol * 10, atol=tol * 10):
                ok = False
                msgs.append(f"reload: param {n} differs")
        inputs = zoo.inputs(case["model"], B, g)
        local = inputs if whole else tuple(t[rank * lb:(rank + 1) * lb] for t in inputs)
        out, rout = wrapped(*local), ref(*inputs)
        if out.dim() == 0:
            out.backward()
            rout.backward()
        else:
            go = torch.randn(rout.shape, generator=g)
            out.backward((go if whole else go[rank * lb:(rank + 1) * lb]).to(out.dtype))
            rout.backward(go / world)
        opt.step()
        ropt.step()
        for n, p in ref.named_parameters():
            v = wrapped.get_param(n)
            if not torch.allclose(v.float(), p.detach().float(), rtol=tol * 10, atol=tol * 10):
                ok = False
                msgs.append(f"reload: param {n} differs after a step by "
                            f"{(v.float() - p.detach().float()).abs().max().item()}")
    stages = len(wrapped._dep.fwd_graph_order)
    res = {"ok": ok, "msgs": msgs[:8], "stages": stages,
           "interleaved": getattr(wrapped._runtime, "interleaved_steps", 0),
           "buckets": max([len(g_.buckets) for g_ in wrapped._storage.groups] or [0]), "pipeline": wrapped._dep.pipeline_num, "sliced": len(wrapped._storage.sliced),
           "alloc": {k: list(v) for k, v in wrapped._dep.allocation.items()}}
    all_res = pyrannc._comm.allgather_obj(res)
    if rank == 0:
        print("RESULT " + json.dumps({"ok": all(r["ok"] for r in all_res), "ranks": all_res}))
    pyrannc.barrier()
    pyrannc.clear()
    sys.exit(0 if all(r["ok"] for r in all_res) else 1)


if __name__ == "__main__":
    main()

"""One rank of a multi-GPU test (launched by tests/test_multi_gpu.py): tiny BERT, bf16 master-weight
training with ZeRO; writes the final parameters of rank 0 to a file so that two runs can be compared."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from rannc_b200.models.bert import BertConfig, BertForPreTraining, synthetic_batch  # noqa: E402
from rannc_b200.ops import _lib  # noqa: E402
from rannc_b200.ops import functional as RF  # noqa: E402


def main():
    case = json.loads(sys.argv[1])
    rank, world = pyrannc.get_rank(), pyrannc.get_world_size()
    torch.manual_seed(0)
    RF.manual_seed(5)
    resnet = case.get("model", "bert") == "resnet"
    if case.get("fp16"):
        pyrannc.amp.initialize(None, None, dtype=torch.float16)
    if resnet:
        from rannc_b200.models.resnet import ResNetWithLoss, tiny_resnet

        cfg = None
        model = ResNetWithLoss(tiny_resnet())
    else:
        cfg = BertConfig.tiny(hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                              num_hidden_layers=case.get("layers", 2))
        if case.get("dist_param"):
            # declared in shards: every rank keeps 1/world of each parameter until deployment
            full = BertForPreTraining(cfg)
            torch.manual_seed(0)
            with pyrannc.DistributeModelParams():
                model = BertForPreTraining(cfg, init_weights=False)
            with torch.no_grad():
                for (_, p), (_, q) in zip(model.named_parameters(), full.named_parameters()):
                    pyrannc.set_dist_param(id(p), q)
            del full
        else:
            model = BertForPreTraining(cfg)
    if case.get("opt", "adam") == "sgd":
        opt = torch.optim.SGD(model.parameters(), lr=0.02, momentum=0.9, weight_decay=1e-4)
    else:
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    wrapped = pyrannc.RaNNCModule(model, opt, enable_apex_amp=True, enable_zero=case.get("zero", True),
                                  offload_params=case.get("offload", False))
    if case.get("max_grad_norm"):
        wrapped.max_grad_norm = float(case["max_grad_norm"])
    B = case.get("batch", 16)
    lb = B // world
    dev = pyrannc._comm.device()
    losses, norms, skipped = [], [], []
    for it in range(case.get("iters", 3)):
        if resnet:
            g = torch.Generator().manual_seed(it)
            full = (torch.randn(B, 3, 64, 64, generator=g), torch.randint(0, 10, (B,), generator=g))
        else:
            full = synthetic_batch(cfg, B, 128, seed=it)
        local = tuple(t[rank * lb:(rank + 1) * lb].to(dev) for t in full)
        saved_scale = None
        if case.get("inject_inf") == it:
            # an overflow made on the host: an absurd loss scale for this one step turns the fp16 gradients
            # into inf; the step must be skipped on every rank
            sc = pyrannc.amp.get_scaler()
            saved_scale, sc._loss_scale = sc._loss_scale, 2.0 ** 60
        loss = wrapped(*local)
        if case.get("fp16"):
            with pyrannc.amp.scale_loss(loss) as scaled:
                scaled.backward()
        else:
            loss.backward()
        if case.get("clip"):
            norms.append(wrapped.clip_grad_norm(float(case["clip"])))
        opt.step()
        opt.zero_grad()
        if saved_scale is not None:
            skipped.append(pyrannc.amp.get_scaler().loss_scale() < 2.0 ** 60)
            pyrannc.amp.get_scaler()._loss_scale = saved_scale
        losses.append(float(loss))
    torch.cuda.synchronize()
    sd = wrapped.state_dict()
    osd = opt.state_dict(from_global=True)
    reload_ok = None
    if case.get("reload"):
        # other values written into the deployed module (symmetric 16-bit buffers, fp32 master shards), read back
        # through the same accessor a checkpoint uses, then one more training step on them
        sd_all = pyrannc.comm_utils.bcast_obj(sd, 0)
        new_sd = {k: (v.float() * 0.5).to(v.dtype) if v.is_floating_point() else v for k, v in sd_all.items()}
        wrapped.load_state_dict(new_sd)
        reload_ok = True
        for n, _ in list(model.named_parameters())[:12]:
            got = wrapped.get_param(n, amp_master_param=True).float().cpu()
            if not torch.allclose(got, new_sd[n].float(), rtol=1e-6, atol=1e-7):
                reload_ok = False
        full = (torch.randn(B, 3, 64, 64), torch.randint(0, 10, (B,))) if resnet else synthetic_batch(cfg, B, 128, seed=99)
        local = tuple(t[rank * lb:(rank + 1) * lb].to(dev) for t in full)
        loss = wrapped(*local)
        loss.backward()
        opt.step()
        opt.zero_grad()
        reload_ok = reload_ok and bool(torch.isfinite(loss))
        torch.cuda.synchronize()
    err = _lib.read_error()
    red = wrapped._fused_reducer
    info = {"reload_ok": reload_ok, "fused": red is not None, "norms": norms,
            "buckets": red.num_buckets() if red is not None else 0,
            "in_backward": red.launched_in_backward if red is not None else 0,
            "scale": pyrannc.amp.get_scaler().loss_scale(), "skipped": skipped, "stages": len(wrapped._dep.fwd_graph_order),
            "alloc": {k: list(v) for k, v in wrapped._dep.allocation.items()}, "losses": losses, "err": err,
            "sliced": len(wrapped._storage.sliced)}
    infos = pyrannc._comm.allgather_obj(info)
    if rank == 0:
        torch.save({"sd": sd, "opt": osd, "infos": infos}, case["out"])
    pyrannc.barrier()
    pyrannc.clear()


if __name__ == "__main__":
    main()

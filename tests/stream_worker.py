"""One rank of the CPU (gloo) test of parameters streamed from host memory.  Launched by tests/test_dist_cpu.py.

The same small BERT is trained twice in this process from the same seed: with every parameter resident and with
``offload_params`` + ``offload_param_window_mb``; losses and final parameters must agree (the two runs differ only
in where bf16 gradients of a weight used twice are summed)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("RANNC_FORCE_CPU", "1")

import torch  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from rannc_b200 import _core  # noqa: E402
from rannc_b200.models.bert import BertConfig, BertForPreTraining, synthetic_batch  # noqa: E402


def run(case, window_mb, segments=0):
    if window_mb:
        os.environ["RANNC_OFFLOAD_PARAM_WINDOW_MB"] = str(window_mb)
    else:
        os.environ.pop("RANNC_OFFLOAD_PARAM_WINDOW_MB", None)
    if segments:
        os.environ["RANNC_CHECKPOINT_SEGMENTS"] = str(segments)
    else:
        os.environ.pop("RANNC_CHECKPOINT_SEGMENTS", None)
    _core.config_reload()
    rank, world = pyrannc.get_rank(), pyrannc.get_world_size()
    torch.manual_seed(0)
    cfg = BertConfig(hidden_size=128, num_hidden_layers=4, num_attention_heads=4, intermediate_size=512,
                     vocab_size=1000, max_position_embeddings=32, hidden_dropout_prob=0.1,
                     attention_probs_dropout_prob=0.1)
    model = BertForPreTraining(cfg)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3) if case.get("opt", "adam") == "adam" else \
        torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    m = pyrannc.RaNNCModule(model, opt, enable_apex_amp=True, enable_zero=case.get("zero", False),
                            offload_params=bool(window_mb))
    B = case.get("batch", 8)
    lb = B // world
    losses = []
    for it in range(case.get("iters", 3)):
        batch = synthetic_batch(cfg, B, 16, seed=it)
        loss = m(*(t[rank * lb:(rank + 1) * lb] for t in batch))
        loss.backward()
        if case.get("clip"):
            m.clip_grad_norm(case["clip"])
        opt.step()
        opt.zero_grad()
        losses.append(float(loss.detach()))
    sd = m.state_dict()
    info = {}
    st = m._storage.streamer
    if segments:
        stages = list(m._stages.values())
        info = {"segments": sum(len(s.segments) for s in stages), "checkpointing": m.is_checkpointing_enabled(),
                "segmented_runs": sum(1 for s in stages if hasattr(s, "seg_saved"))}
    if window_mb:
        stages = list(m._stages.values())
        info = {"segments": sum(len(s.segments) for s in stages), "peak_resident": st.peak_resident,
                "resident_after": st.resident,
                "held": sum(p.data.numel() for g in m._storage.groups if g.streamed for p in g.params),
                "streamed_groups": sum(1 for g in m._storage.groups if g.streamed),
                "host_grads": all(not g.flat_grad.is_cuda for g in m._storage.groups if g.streamed)}
    pyrannc.barrier()
    return losses, sd, info


def main():
    case = json.loads(sys.argv[1])
    rank = pyrannc.get_rank()
    la, sda, _ = run(case, 0)
    if case.get("segments"):
        # recomputation segment by segment against recomputation of the whole stage (parameters resident)
        lb_, sdb, info = run(case, 0, case["segments"])
    else:
        lb_, sdb, info = run(case, case.get("window_mb", 1))
    ok, msgs = True, []
    for i, (x, y) in enumerate(zip(la, lb_)):
        if abs(x - y) > 2e-3 * max(1.0, abs(x)):
            ok = False
            msgs.append(f"loss {i}: {x} resident vs {y} streamed")
    if rank == 0:
        worst = max(float((sda[k].float() - sdb[k].float()).abs().max()) for k in sda)
        info["max_param_diff"] = worst
        if worst > 2e-2:
            ok = False
            msgs.append(f"parameters differ by {worst}")
    if case.get("segments"):
        if info.get("segments", 0) < 3 or not info.get("checkpointing"):
            ok = False
            msgs.append(f"segments: {info}")
    elif info.get("segments", 0) < 3 or info.get("held", 1) != 0 or info.get("resident_after", 1) != 0 or \
            not info.get("host_grads") or info.get("peak_resident", 1 << 40) > (case.get("window_mb", 1) << 20):
        ok = False
        msgs.append(f"residency: {info}")
    print("RESULT " + json.dumps({"rank": rank, "ok": ok, "msgs": msgs[:6], "info": info, "losses": [la, lb_]}),
          flush=True)
    pyrannc.barrier()


if __name__ == "__main__":
    main()

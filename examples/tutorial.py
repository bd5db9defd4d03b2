#!/usr/bin/env python
"""The tutorial: wrap a model and its optimizer, train a few steps, save and reload.

    python examples/tutorial.py                                  # one process (CPU or one GPU)
    torchrun --nproc-per-node 2 examples/tutorial.py             # one process per GPU
    RANNC_PARTITION_NUM=2 torchrun --nproc-per-node 2 examples/tutorial.py   # force two pipeline stages

Same steps as the reference's tutorial (examples/tutorial.py, documents/tutorial.rst): nothing in the model
is written for parallel execution; the partitioning is decided at the first call.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from rannc_b200.models.mlp import TutorialMLPWithLoss  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64, help="batch size per process")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--save", default="")
    args = ap.parse_args()

    torch.manual_seed(0)
    model = TutorialMLPWithLoss()                     # Linear 512 -> 1024 -> 1024 -> 10, cross-entropy
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    model = pyrannc.RaNNCModule(model, opt)

    dev = "cuda" if torch.cuda.is_available() and os.environ.get("RANNC_FORCE_CPU", "0") != "1" else "cpu"
    # one synthetic batch per process (inputs N(0, 1), labels uniform over the 10 classes), seen every step
    g = torch.Generator().manual_seed(pyrannc.get_rank())
    x = torch.randn(args.batch, 512, generator=g).to(dev)
    y = torch.randint(0, 10, (args.batch,), generator=g).to(dev)
    for step in range(args.steps):
        loss = model(x, y)                            # first call: trace, profile, partition, deploy
        loss.backward()
        opt.step()
        opt.zero_grad()
        if pyrannc.get_rank() == 0:
            print(f"step {step}: loss {float(loss):.4f}")

    sd = model.state_dict()                           # collective; full tensors on rank 0
    osd = opt.state_dict(from_global=True)
    if args.save and pyrannc.get_rank() == 0:
        torch.save({"model": sd, "optimizer": osd}, args.save)
    if pyrannc.get_rank() == 0:
        print(f"{len(sd)} tensors in the model state, {len(osd['state'])} in the optimizer state")
    pyrannc.barrier()
    pyrannc.clear()


if __name__ == "__main__":
    main()

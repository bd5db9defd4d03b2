#!/usr/bin/env python
"""BERT pre-training (masked language model + next sentence) on synthetic data: the large-model workflow.

    python examples/bert_pretrain.py --layers 2 --hidden 128 --heads 4 --seq 32 --batch 8   # a toy, CPU or one GPU
    torchrun --nproc-per-node 8 examples/bert_pretrain.py --layers 24 --hidden 1024 --heads 16 --batch 32
    torchrun --nproc-per-node 8 examples/bert_pretrain.py --layers 256 --hidden 2048 --heads 32 --batch 32 \\
        --dist-params --resume ckpt.pt --save ckpt.pt

What it shows, all of it with an unmodified ``nn.Module``:

* mixed precision with fp32 master weights and ZeRO sharding of the optimizer state (``enable_apex_amp``,
  ``enable_zero``); the stages, replicas and micro-batches are chosen at the first call;
* ``--dist-params``: the model is declared under ``DistributeModelParams`` so that no process ever holds all of
  it (each keeps 1/world of every parameter until the stages are placed);
* gradient clipping over all stages, evaluation under ``torch.no_grad()``;
* checkpoints a plain PyTorch job can read: ``state_dict()`` returns full tensors on rank 0 and
  ``optimizer.state_dict(from_global=True)`` the optimizer state in torch's own numbering; ``--resume`` loads both
  back, into whatever partitioning this run chose.

Switches worth knowing (environment, see docs/config.md and docs/tuning.md): ``RANNC_PARTITION_NUM``,
``RANNC_PIPELINE_NUM``, ``RANNC_CHECKPOINT_SEGMENTS``, ``RANNC_PARTITIONING_DRY_RUN_NP`` (plan only, no GPU needed).
"""
import argparse
import contextlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from rannc_b200.models.bert import BertConfig, BertForPreTraining, synthetic_batch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=1000)
    ap.add_argument("--batch", type=int, default=8, help="sequences per process and step")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--dist-params", action="store_true")
    ap.add_argument("--save", default="")
    ap.add_argument("--resume", default="")
    args = ap.parse_args()

    rank, world = pyrannc.get_rank(), pyrannc.get_world_size()
    cfg = BertConfig(hidden_size=args.hidden, num_hidden_layers=args.layers, num_attention_heads=args.heads,
                     intermediate_size=4 * args.hidden, vocab_size=args.vocab,
                     max_position_embeddings=max(32, args.seq))
    torch.manual_seed(0)
    with (pyrannc.DistributeModelParams() if args.dist_params else contextlib.nullcontext()):
        # under DistributeModelParams every layer is cut into shards the moment it has been constructed, so its
        # values must be final by then: the layers keep their own default initialisation instead of a pass over
        # the finished model
        model = BertForPreTraining(cfg, init_weights=not args.dist_params)
    decay = [p for n, p in model.named_parameters() if p.dim() >= 2]
    no_decay = [p for n, p in model.named_parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=1e-4)
    model = pyrannc.RaNNCModule(model, opt, enable_apex_amp=True, enable_zero=world > 1)

    dev = "cuda" if torch.cuda.is_available() and os.environ.get("RANNC_FORCE_CPU", "0") != "1" else "cpu"

    def batch_for(step):
        # every process draws its own rows of the step's global batch
        full = synthetic_batch(cfg, args.batch * world, args.seq, seed=step)
        return tuple(t[rank * args.batch:(rank + 1) * args.batch].to(dev) for t in full)

    def held_out_loss():
        # the same rows on every process, dropout off: comparable across runs and world sizes
        rows = tuple(t.to(dev) for t in synthetic_batch(cfg, args.batch, args.seq, seed=10 ** 6))
        model.eval()
        with torch.no_grad():
            val = float(model(*rows))
        model.train()
        return val

    first = 0
    for step in range(args.steps):
        loss = model(*batch_for(step))                # first call: trace, profile, partition, deploy
        if step == 0 and args.resume:
            # the checkpoint is loaded into the deployed module: every rank reads the file, each keeps its part
            ck = torch.load(args.resume, map_location="cpu")
            model.load_state_dict(ck["model"])
            opt.load_state_dict(ck["optimizer"], from_global=True)
            first = ck.get("step", 0)
            val = held_out_loss()
            if rank == 0:
                print(f"resumed at step {first}: held-out loss {val:.4f}")
            loss = model(*batch_for(step))
        loss.backward()
        norm = model.clip_grad_norm(args.clip)
        opt.step()
        opt.zero_grad()
        if rank == 0:
            print(f"step {first + step}: loss {float(loss):.4f} grad-norm {norm:.3f}")

    val = held_out_loss()
    if rank == 0:
        print(f"held-out loss {val:.4f}")

    sd = model.state_dict()                           # collective; full fp32 tensors on rank 0
    osd = opt.state_dict(from_global=True)            # collective; torch's own layout
    if args.save and rank == 0:
        torch.save({"model": sd, "optimizer": osd, "step": first + args.steps}, args.save)
        print(f"saved {len(sd)} tensors to {args.save}")
    pyrannc.barrier()
    pyrannc.clear()


if __name__ == "__main__":
    main()

"""One rank of the tensor-partitioned linear test over real peers (launched by tests/test_multi_gpu.py).
Every rank slices the same seeded nn.Linear, runs forward / backward on its own batch slice through the
all-gather -> GEMM and GEMM -> reduce-scatter kernels, and compares with the full-weight computation."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from rannc_b200.ops import _lib  # noqa: E402
from rannc_b200.parallel.distop import DistGroup, DistLinear  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


def main():
    case = json.loads(sys.argv[1])
    rank, world = pyrannc.get_rank(), pyrannc.get_world_size()
    dev = pyrannc._comm.device()
    M, N, K = case.get("M", 1024), case.get("N", 768), case.get("K", 2048)
    torch.manual_seed(0)
    lin = torch.nn.Linear(K, N).to(dev).bfloat16()
    with torch.no_grad():
        lin.weight.mul_(0.5)
    grp = DistGroup(list(range(world)), N * K, torch.bfloat16, dev)
    dl = DistLinear.from_linear(grp, lin)
    errs = {}
    for it in range(case.get("iters", 3)):
        g = torch.Generator(device="cpu").manual_seed(100 + it)
        xs = torch.randn(world, M, K, generator=g).bfloat16()
        dys = torch.randn(world, M, N, generator=g).bfloat16()
        x = xs[rank].to(dev).requires_grad_(True)
        dy = dys[rank].to(dev)
        dl.weight.main_grad.zero_()
        grp.barrier()                      # every shard and every zeroed gradient buffer is in place
        y = dl(x)
        y.backward(dy)
        grp.barrier()                      # every rank's contribution to this rank's gradient has landed
        torch.cuda.synchronize()
        ref_y = x.detach().float() @ lin.weight.float().t() + lin.bias.float()
        ref_dx = dy.float() @ lin.weight.float()
        dW = sum(dys[r].to(dev).float().t() @ xs[r].to(dev).float() for r in range(world)) / world
        ks = K // world
        errs[f"y{it}"] = rel(y, ref_y)
        errs[f"dx{it}"] = rel(x.grad, ref_dx)
        errs[f"dw{it}"] = rel(dl.weight.main_grad, dW[:, rank * ks:(rank + 1) * ks])
    info = {"errs": errs, "err_word": _lib.read_error()}
    infos = pyrannc._comm.allgather_obj(info)
    if rank == 0:
        with open(case["out"], "w") as f:
            json.dump(infos, f)
    pyrannc.barrier()
    pyrannc.clear()


if __name__ == "__main__":
    main()

"""Two CPU ranks.  After one clean training step every rank arms a host-side failure: the next guarded
collective raises before anything is issued (as a transport error would).  The communication layer must
re-create the communicators and retry, and training must go on with the same numbers as an undisturbed run."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ["RANNC_FORCE_CPU"] = "1"

import torch  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from rannc_b200.parallel import comm  # noqa: E402
from tests import zoo  # noqa: E402


def run(inject: bool):
    torch.manual_seed(0)
    model = zoo.build("deep")
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    wrapped = pyrannc.RaNNCModule(model, opt)
    rank = pyrannc.get_rank()
    g = torch.Generator().manual_seed(1)
    losses = []
    for it in range(3):
        inputs = zoo.inputs("deep", 8, g)
        local = tuple(t[rank * 4:(rank + 1) * 4] for t in inputs)
        out = wrapped(*local)
        if it == 1 and inject:
            comm.inject_collective_failures(1)     # the gradient all-reduce of this step fails once
        out.sum().backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(out.detach().sum()))
    sd = wrapped.state_dict()
    wrapped.undeploy()
    return losses, sd


def main():
    rank = pyrannc.get_rank()
    clean_losses, clean_sd = run(False)
    n0 = comm.retries_done()
    hurt_losses, hurt_sd = run(True)
    retried = comm.retries_done() - n0
    ok = retried == 1 and all(abs(a - b) < 1e-6 for a, b in zip(clean_losses, hurt_losses))
    if rank == 0:
        ok = ok and all(torch.allclose(clean_sd[k], hurt_sd[k]) for k in clean_sd)
    # exhausted retries surface as CommError
    comm.inject_collective_failures(5)
    try:
        t = torch.ones(1)
        comm.allreduce(t)
        ok = False
    except comm.CommError:
        pass
    comm.inject_collective_failures(0)
    print("RETRY_OK" if ok else f"RETRY_BAD retried={retried} {clean_losses} {hurt_losses}")
    pyrannc.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()

"""Two CPU ranks; rank 1 leaves between steps (no collective in flight) and removes its heartbeat file.
Rank 0 must learn of it on the host, before its next forward, and raise CommError."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ["RANNC_FORCE_CPU"] = "1"

import torch  # noqa: E402

import rannc_b200 as pyrannc  # noqa: E402
from rannc_b200.parallel import comm  # noqa: E402
from tests import zoo  # noqa: E402


def main():
    rank = pyrannc.get_rank()
    torch.manual_seed(0)
    model = zoo.build("loss")
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    wrapped = pyrannc.RaNNCModule(model, opt)
    g = torch.Generator().manual_seed(1)
    x, y = zoo.inputs("loss", 8, g)
    lo = rank * 4
    loss = wrapped(x[lo:lo + 4], y[lo:lo + 4])
    loss.backward()
    opt.step()
    opt.zero_grad()
    pyrannc.barrier()
    if rank == 1:
        comm.stop_watchdog(True)  # tells the peers, then leaves
        print("LEFT")
        os._exit(0)
    deadline = time.time() + 20
    try:
        while time.time() < deadline:
            comm.check_peers()
            time.sleep(0.05)
        wrapped(x[lo:lo + 4], y[lo:lo + 4])
        print("NOT DETECTED")
    except comm.CommError as e:
        print("DETECTED", e)
    os._exit(0)


if __name__ == "__main__":
    main()

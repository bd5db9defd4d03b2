"""Process bootstrap and host-issued communication.

One process per GPU, started by ``torchrun`` (or anything that sets RANK /
WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT).  ``torch.distributed``
takes the place of the reference's MPI + hand-rolled NCCL wrapper:

* control plane (ids, deployment, pickled objects): object collectives over the
  default group (reference: src/comm/ObjectComm.cpp, MPI + msgpack);
* one communicator per distinct rank set, created in a deterministic order --
  smaller sets first (reference: src/comm/NCCLWrapper.cpp:90-131,
  src/comp/ParamStorage.cpp:336-345);
* ``redist``: contiguous-row all-to-all-v between two rank sets with grouped
  send/recv (reference: NCCLWrapper.cpp:445-564), used by pipeline routes;
* all-reduce / broadcast / all-gather / reduce-scatter for the baseline gradient
  path, checkpoint gathering and ``tensor_coll``.

A world of one process needs no process group at all; every call degenerates to
a local operation.  Without CUDA the backend is gloo (CPU rank harness).
"""
from __future__ import annotations

import datetime
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import _core
from ..utils.config import conf
from ..utils.log import get_logger

logger = get_logger("Comm")


class CommError(RuntimeError):
    """A collective failed or a peer disappeared (reference: CommErrorException)."""


class _State:
    def __init__(self):
        self.initialized = False
        self.rank = 0
        self.world = 1
        self.local_rank = 0
        self.device = torch.device("cpu")
        self.backend = None
        self.groups: Dict[Tuple[int, ...], object] = {}
        self.owns_pg = False
        self.cpu_group = None
        self.watchdog = None
        self.failed_peer = -1
        self.p2p_stream = None
        self.inject_failures = 0     # test hook: the next N guarded collectives raise on the host
        self.retries_done = 0


_S = _State()


def start(device: Optional[torch.device] = None) -> None:
    """Counterpart of RaNNCProcess::start (src/bind/RaNNCProcess.cpp:20-104)."""
    if _S.initialized:
        return
    _S.rank = int(os.environ.get("RANK", "0"))
    _S.world = int(os.environ.get("WORLD_SIZE", "1"))
    _S.local_rank = int(os.environ.get("LOCAL_RANK", str(_S.rank)))
    use_cuda = torch.cuda.is_available() and os.environ.get("RANNC_FORCE_CPU", "0") != "1"
    if device is not None:
        _S.device = device
    elif use_cuda:
        _S.device = torch.device("cuda", _S.local_rank % torch.cuda.device_count())
        torch.cuda.set_device(_S.device)
    else:
        _S.device = torch.device("cpu")
    if _S.world > 1:
        if not dist.is_initialized():
            backend = "nccl" if _S.device.type == "cuda" else "gloo"
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            timeout = datetime.timedelta(seconds=float(conf("comm_timeout_s")))
            kwargs = {}
            if backend == "nccl":
                kwargs["device_id"] = _S.device
            dist.init_process_group(backend, rank=_S.rank, world_size=_S.world, timeout=timeout, **kwargs)
            _S.owns_pg = True
        _S.backend = dist.get_backend()
    _core.set_log_rank(_S.rank)
    _S.initialized = True
    if bool(conf("run_watchdog")) and _S.world > 1:
        start_watchdog()
    logger.debug("rank %d of %d on %s", _S.rank, _S.world, str(_S.device))


def start_watchdog(directory: Optional[str] = None) -> None:
    """Heartbeat files in a directory every rank can see; a missing or stale peer file marks the job as
    failed, and the next ``check_peers()`` -- called on the host before every forward / backward, i.e.
    before anything is launched -- raises ``CommError`` instead of entering a collective that would never
    complete (reference: SyncWatchDog, src/cuda/CudaSync.cpp:22-112)."""
    d = directory or os.environ.get("RANNC_WATCHDOG_LOCKFILE_DIR") or str(conf("watchdog_lockfile_dir"))
    if not d:
        raise RuntimeError("run_watchdog needs watchdog_lockfile_dir (or RANNC_WATCHDOG_LOCKFILE_DIR)")
    os.makedirs(d, exist_ok=True)

    def on_failure(peer: int):
        _S.failed_peer = int(peer)

    _S.watchdog = _core.Watchdog()
    _S.watchdog.start(d, _S.rank, _S.world, float(conf("watchdog_period_s")), float(conf("watchdog_stale_s")),
                      on_failure)


def stop_watchdog(remove_own_file: bool = True) -> None:
    """A rank that fails (or leaves between steps) removes its heartbeat file so the others notice."""
    if _S.watchdog is not None:
        _S.watchdog.stop(remove_own_file)
        _S.watchdog = None


def check_peers() -> None:
    if _S.failed_peer >= 0:
        peer = _S.failed_peer
        stop_watchdog(True)
        raise CommError(f"rank {peer} stopped responding (heartbeat file missing or stale)")


def clear() -> None:
    """Destroys communicators (reference: RaNNCProcess::clear)."""
    stop_watchdog(True)
    _S.failed_peer = -1
    _S.groups.clear()
    if _S.owns_pg and dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
    _S.owns_pg = False
    _S.initialized = False
    _S.cpu_group = None


def get_rank() -> int:
    start()
    return _S.rank


def get_world_size() -> int:
    start()
    return _S.world


def get_local_rank() -> int:
    start()
    return _S.local_rank


def device() -> torch.device:
    start()
    return _S.device


def is_cuda() -> bool:
    return device().type == "cuda"


def barrier() -> None:
    if get_world_size() > 1:
        if is_cuda():
            dist.barrier(device_ids=[_S.device.index])
        else:
            dist.barrier()


# ---------------------------------------------------------------- groups
def _key(ranks: Sequence[int]) -> Tuple[int, ...]:
    return tuple(sorted(set(int(r) for r in ranks)))


def create_groups(rank_sets: Sequence[Sequence[int]]) -> None:
    """Collective over the world: creates a communicator for every rank set not seen before,
    smaller sets first, ties broken by the ranks themselves."""
    start()
    if _S.world == 1:
        return
    keys = sorted({_key(r) for r in rank_sets}, key=lambda k: (len(k), k))
    for k in keys:
        if k in _S.groups or len(k) == 0:
            continue
        if len(k) == _S.world:
            _S.groups[k] = dist.group.WORLD
        else:
            _S.groups[k] = dist.new_group(list(k))


def group(ranks: Optional[Sequence[int]] = None):
    start()
    if _S.world == 1:
        return None
    if ranks is None:
        return dist.group.WORLD
    k = _key(ranks)
    if len(k) == _S.world:
        return dist.group.WORLD
    if k not in _S.groups:
        raise CommError(f"no communicator for ranks {k}; create_groups() must run on every rank first")
    return _S.groups[k]


def recreate_all_communicators() -> None:
    """Abort + re-create every communicator in creation order (reference: NCCLWrapper.cpp:667-703)."""
    if _S.world == 1:
        return
    keys = list(_S.groups.keys())
    for k in keys:
        g = _S.groups[k]
        if g is not dist.group.WORLD:
            try:
                dist.destroy_process_group(g)
            except Exception:  # noqa: BLE001
                pass
    _S.groups.clear()
    create_groups(keys)


# ---------------------------------------------------------------- objects
def bcast_obj(obj, root: int = 0, ranks: Optional[Sequence[int]] = None):
    if get_world_size() == 1:
        return obj
    box = [obj if get_rank() == root else None]
    dist.broadcast_object_list(box, src=root, group=group(ranks), device=_S.device if is_cuda() else None)
    return box[0]


def allgather_obj(obj, ranks: Optional[Sequence[int]] = None) -> list:
    if get_world_size() == 1:
        return [obj]
    g = group(ranks)
    n = dist.get_world_size(g)
    out = [None] * n
    dist.all_gather_object(out, obj, group=g)
    return out


def bcast_bytes(data: bytes, root: int = 0) -> bytes:
    return bcast_obj(data, root)


# ---------------------------------------------------------------- failure handling
def inject_collective_failures(n: int) -> None:
    """Test hook: the next ``n`` guarded collectives of this process raise before anything is issued (a failure
    made on the host, as a transport error would surface)."""
    _S.inject_failures = int(n)


def retries_done() -> int:
    return _S.retries_done


def _with_retry(what: str, fn):
    """Runs a collective; when it raises (a transport error, an aborted communicator, a process-group timeout)
    every communicator is re-created and the call is tried again, ``comm_retry`` times, before ``CommError`` is
    raised (reference: commWithRetry / recreateAllCommunicators, src/comm/NCCLWrapper.cpp:667-739).  All ranks
    of the collective see the failure (a failed rank makes the others' call fail or time out), so all of them
    take part in the re-creation."""
    attempts = max(0, int(conf("comm_retry")))
    for attempt in range(attempts + 1):
        try:
            if _S.inject_failures > 0:
                _S.inject_failures -= 1
                raise RuntimeError(f"injected failure in {what}")
            return fn()
        except CommError:
            raise
        except (RuntimeError, ValueError) as e:
            if attempt >= attempts:
                raise CommError(f"{what} failed after {attempt} retr{'y' if attempt == 1 else 'ies'}: {e}") from e
            logger.warning("%s failed (%s); re-creating the communicators and retrying", what, str(e)[:200])
            import time

            time.sleep(float(conf("comm_retry_wait_s")))
            recreate_all_communicators()
            _S.retries_done += 1


def sync_with_error_check(timeout_s: float = 0.0) -> None:
    """Waits for the work enqueued so far WITHOUT blocking inside the driver: polls an event and, while it is
    not complete, looks for a failed peer (heartbeat watchdog), so that a rank whose peer died raises instead
    of hanging in a synchronise (reference: syncWithErrorCheck, src/comm/NCCLWrapper.cpp:575-622, which polls
    cudaStreamQuery and ncclCommGetAsyncError; here torch's own NCCL watchdog turns an asynchronous NCCL error
    into an exception of the next call, which ``_with_retry`` handles)."""
    import time

    check_peers()
    if not is_cuda():
        return
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream())
    t0 = time.monotonic()
    limit = timeout_s if timeout_s > 0 else float(conf("comm_timeout_s"))
    while not ev.query():
        check_peers()
        if time.monotonic() - t0 > limit:
            raise CommError(f"work on the device did not finish within {limit:.0f} s")
        time.sleep(0.0005)


# ---------------------------------------------------------------- tensors
def _premul_sum(scale: float):
    """NCCL's PreMulSum reduction operator (every contribution is multiplied by ``scale`` on its way into the sum,
    inside the collective); None where the backend has none (reference: ncclRedOpCreatePreMulSum,
    src/comm/NCCLWrapper.cpp:340-372)."""
    if _S.backend != "nccl" or scale == 1.0:
        return None
    make = getattr(dist, "_make_nccl_premul_sum", None)
    if make is None:
        return None
    try:
        return make(float(scale))
    except Exception:  # noqa: BLE001 -- a build of torch without the operator
        return None


def allreduce(t: torch.Tensor, op: str = "sum", ranks: Optional[Sequence[int]] = None, async_op: bool = False,
              scale: float = 1.0):
    """``scale`` (with ``op="sum"``): every rank's contribution is multiplied by it first -- inside the
    collective where the backend can (PreMulSum), by one extra pass over ``t`` otherwise."""
    if get_world_size() == 1 or (ranks is not None and len(_key(ranks)) <= 1):
        if scale != 1.0:
            t.mul_(scale)
        return None
    if scale != 1.0 and op == "sum":
        rop = _premul_sum(scale)
        if rop is None:
            t.mul_(scale)
            rop = dist.ReduceOp.SUM
    else:
        rop = {"sum": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}[op]
    return _with_retry("all-reduce", lambda: dist.all_reduce(t, op=rop, group=group(ranks), async_op=async_op))


def bcast(t: torch.Tensor, root: int, ranks: Optional[Sequence[int]] = None) -> None:
    if get_world_size() == 1 or (ranks is not None and len(_key(ranks)) <= 1):
        return
    _with_retry("broadcast", lambda: dist.broadcast(t, src=root, group=group(ranks)))


def allgather_into(out: torch.Tensor, inp: torch.Tensor, ranks: Optional[Sequence[int]] = None) -> None:
    if get_world_size() == 1 or (ranks is not None and len(_key(ranks)) <= 1):
        out.view(-1)[: inp.numel()].copy_(inp.view(-1))
        return
    _with_retry("all-gather", lambda: dist.all_gather_into_tensor(out, inp, group=group(ranks)))


def reduce_scatter_into(out: torch.Tensor, inp: torch.Tensor, ranks: Optional[Sequence[int]] = None,
                        scale: float = 1.0) -> None:
    """``scale``: as for :func:`allreduce`; ``inp`` is left unscaled when the collective applies it."""
    if get_world_size() == 1 or (ranks is not None and len(_key(ranks)) <= 1):
        out.copy_(inp.view(-1)[: out.numel()].view_as(out))
        if scale != 1.0:
            out.mul_(scale)
        return
    if _S.backend == "gloo":
        # gloo has no reduce-scatter: all-reduce a copy and keep this rank's piece (CPU rank harness only)
        def via_allreduce():
            g = group(ranks)
            full = inp.clone()
            dist.all_reduce(full, op=dist.ReduceOp.SUM, group=g)
            n = out.numel()
            i = dist.get_rank(g)
            out.copy_(full.view(-1)[i * n:(i + 1) * n].view_as(out))
            if scale != 1.0:
                out.mul_(scale)

        _with_retry("reduce-scatter", via_allreduce)
        return
    rop = _premul_sum(scale) if scale != 1.0 else dist.ReduceOp.SUM
    post = 1.0
    if rop is None:
        rop, post = dist.ReduceOp.SUM, scale
    _with_retry("reduce-scatter", lambda: dist.reduce_scatter_tensor(out, inp, op=rop, group=group(ranks)))
    if post != 1.0:
        out.mul_(post)


def send_recv(t: Optional[torch.Tensor], src: int, dst: int) -> None:
    """One point-to-point copy of ``t`` from rank ``src`` to rank ``dst``; every other rank returns at once."""
    if get_world_size() == 1 or src == dst:
        return
    me = get_rank()
    if me == src:
        dist.send(t.contiguous(), dst)
    elif me == dst:
        dist.recv(t, src)


class PendingOps:
    """Handles of posted sends; buffers stay referenced until ``wait``."""

    def __init__(self):
        self.reqs = []
        self.keep = []
        self.events = []      # completion events of sends issued from the transfer stream

    def wait(self):
        for r in self.reqs:
            r.wait()
        if self.events:
            cur = torch.cuda.current_stream()
            for ev in self.events:
                cur.wait_event(ev)
            self.events.clear()
        self.reqs.clear()
        self.keep.clear()


def redist(src_rows: Optional[torch.Tensor], args, recv_rows: int, like: Optional[torch.Tensor],
           row_shape: Sequence[int], dtype: torch.dtype, pending: Optional[PendingOps] = None) -> Optional[torch.Tensor]:
    """Contiguous-row all-to-all-v.  ``args`` is a ``_core.RedistArgs`` for this rank: row counts and
    displacements per global rank.  Returns the received tensor ([recv_rows, *row_shape]) or None when
    this rank receives nothing.  Booleans travel as bytes (the reference widens them to int32)."""
    me = get_rank()
    out = None
    if recv_rows > 0:
        out = torch.empty((recv_rows, *row_shape), dtype=dtype, device=device())
    ops, is_send = [], []
    wire = lambda t: t.view(torch.uint8) if t.dtype == torch.bool else t  # noqa: E731
    world = get_world_size()
    # lower ranks first on both sides keeps the pairing order identical everywhere
    for r in range(world):
        sc = args.sendcounts[r]
        if sc > 0 and src_rows is not None:
            piece = src_rows[args.sdispls[r]: args.sdispls[r] + sc]
            if r == me:
                out[args.rdispls[r]: args.rdispls[r] + sc].copy_(piece)
            else:
                piece = piece.contiguous()
                ops.append(dist.P2POp(dist.isend, wire(piece), r))
                is_send.append(True)
                if pending is not None:
                    pending.keep.append(piece)
        rc = args.recvcounts[r]
        if rc > 0 and r != me:
            ops.append(dist.P2POp(dist.irecv, wire(out[args.rdispls[r]: args.rdispls[r] + rc]), r))
            is_send.append(False)
    if ops:
        if is_cuda():
            _redist_on_side_stream(ops, is_send, out, pending)
            return out
        reqs = dist.batch_isend_irecv(ops)
        if pending is not None and len(reqs) == len(ops):
            # one request per operation (gloo): receives are needed now, sends may finish later
            for q, s in zip(reqs, is_send):
                if s:
                    pending.reqs.append(q)
                else:
                    q.wait()
        else:
            for q in reqs:
                q.wait()
    return out


def p2p_stream() -> "torch.cuda.Stream":
    """The stream pipeline transfers are issued from (one per process)."""
    if getattr(_S, "p2p_stream", None) is None:
        _S.p2p_stream = torch.cuda.Stream(device=_S.device)
    return _S.p2p_stream


def _redist_on_side_stream(ops, is_send, out, pending) -> None:
    """NCCL send / recv of one route, issued from a dedicated stream: the transfer starts once the data is ready
    on the compute stream (an event), and the compute stream waits only when this rank RECEIVES something -- a
    stage that has sent its outputs goes straight on with the next micro-batch, whether or not the receiver has
    posted its receive yet.  (The reference orders sends behind a delay for the same purpose:
    src/comp/GraphConnector.cpp:53-96,363-374; its NCCL p2p runs on the compute stream,
    src/comm/NCCLWrapper.cpp:501-533.)"""
    cur = torch.cuda.current_stream()
    side = p2p_stream()
    ready = torch.cuda.Event()
    ready.record(cur)
    for op in ops:
        # the tensors were allocated on the compute stream and are used on the side stream
        op.tensor.record_stream(side)
    with torch.cuda.stream(side):
        side.wait_event(ready)
        reqs = dist.batch_isend_irecv(ops)
        for q in reqs:
            q.wait()          # orders the side stream behind NCCL's own stream; the host does not block
        done = torch.cuda.Event()
        done.record(side)
    if not all(is_send):
        cur.wait_event(done)
    elif pending is not None:
        pending.events.append(done)

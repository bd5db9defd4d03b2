"""Multi-GPU paths (need >= 2 devices): the fused reduce-scatter + Adam + all-gather kernel against the NCCL
collectives path, and a pipeline split across GPUs against pure data parallelism."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, case, extra_env=None, timeout=600, worker="gpu_worker.py"):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ)
        env.update({"RANK": str(r), "WORLD_SIZE": str(world), "LOCAL_RANK": str(r), "MASTER_ADDR": "127.0.0.1",
                    "MASTER_PORT": str(port), "RANNC_LOG_LEVEL": "warning"})
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", worker),
                                       json.dumps(case)], env=env, cwd=ROOT, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(o)
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-4000:]
    if worker != "gpu_worker.py":
        with open(case["out"]) as f:
            return json.load(f)
    return torch.load(case["out"], weights_only=False)


def _compare(a, b, tol):
    # Adam moves every weight by about lr per step whatever the gradient's size, so a rounding-level
    # difference in a near-zero gradient can shift a weight by lr x steps: bound the worst case by that
    # and the typical case tightly
    for k in a["sd"]:
        if k.endswith("key.bias"):
            continue  # exactly-zero gradient: Adam turns its rounding noise into +-lr steps
        x, y = a["sd"][k].float(), b["sd"][k].float()
        d = (x - y).abs()
        assert d.max().item() <= 4e-3 + tol * y.abs().max().item(), k
        assert d.mean().item() <= 4e-4 + tol * y.abs().mean().item(), k


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_reduce_matches_nccl_path(tmp_path):
    fused = _run(2, {"out": str(tmp_path / "fused.pt")})
    plain = _run(2, {"out": str(tmp_path / "plain.pt")}, {"RANNC_FUSED_GRAD_ALLREDUCE": "false"})
    assert all(i["fused"] for i in fused["infos"]) and not any(i["fused"] for i in plain["infos"])
    assert all(i["err"] == 0 for i in fused["infos"])
    for lf, lp in zip(fused["infos"][0]["losses"], plain["infos"][0]["losses"]):
        assert abs(lf - lp) < 2e-2 * abs(lp)
    _compare(fused, plain, 2e-2)
    # optimizer state gathered to the global layout in both
    assert set(fused["opt"]["state"].keys()) == set(plain["opt"]["state"].keys())
    k0 = sorted(fused["opt"]["state"].keys())[0]
    assert fused["opt"]["state"][k0]["exp_avg"].shape == plain["opt"]["state"][k0]["exp_avg"].shape


def _tight(a, b, rel, what=""):
    """Every weight of every tensor: |a - b| <= rel * max|b| of that tensor (no key is skipped)."""
    for k in a["sd"]:
        x, y = a["sd"][k].float(), b["sd"][k].float()
        assert torch.isfinite(x).all(), k
        assert (x - y).abs().max().item() <= rel * (y.abs().max().item() + 1e-3), (what, k)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("multimem", ["1", "0"])
def test_bucketed_reduce_overlapping_backward_matches_nccl(tmp_path, multimem):
    """Buckets of 256 KiB: the 4-layer model splits into many buckets, each rank owns a slice of each, and from
    the second step on every bucket is reduced and updated on the side stream while backward still runs.  SGD
    with momentum, so that a mis-reduced element shows up at its own size (Adam would hide it behind +-lr)."""
    case = {"opt": "sgd", "layers": 4, "iters": 5}
    env = {"RANNC_GRAD_BUCKET_MB": "0.25", "RANNC_USE_MULTIMEM": multimem}
    a = _run(2, dict(case, out=str(tmp_path / "a.pt")), env)
    b = _run(2, dict(case, out=str(tmp_path / "b.pt")), dict(env, RANNC_FUSED_GRAD_ALLREDUCE="false"))
    assert all(i["fused"] and i["err"] == 0 for i in a["infos"]), a["infos"]
    assert all(i["buckets"] >= 4 for i in a["infos"]), a["infos"]
    # 4 of the 5 steps ran with the launches inside backward
    assert all(i["in_backward"] >= 4 * (i["buckets"] - 1) for i in a["infos"]), a["infos"]
    for la, lb in zip(a["infos"][0]["losses"], b["infos"][0]["losses"]):
        assert abs(la - lb) < 2e-2 * abs(lb)
    _tight(a, b, 2e-2, "bucketed")


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_reduce_with_gradient_clipping(tmp_path):
    """clip_grad_norm between backward and the step (the reducer then keeps reduction and update apart and
    the norm comes from the reduction launches), and the same clipping done inside the step via max_grad_norm;
    both against the NCCL path."""
    case = {"opt": "sgd", "layers": 2, "iters": 4}
    env = {"RANNC_GRAD_BUCKET_MB": "0.25"}
    a = _run(2, dict(case, clip=0.5, out=str(tmp_path / "a.pt")), env)
    b = _run(2, dict(case, clip=0.5, out=str(tmp_path / "b.pt")), dict(env, RANNC_FUSED_GRAD_ALLREDUCE="false"))
    c = _run(2, dict(case, max_grad_norm=0.5, out=str(tmp_path / "c.pt")), env)
    assert all(i["fused"] and i["err"] == 0 for i in a["infos"] + c["infos"])
    for na, nb in zip(a["infos"][0]["norms"], b["infos"][0]["norms"]):
        assert nb > 0.5 and abs(na - nb) < 2e-2 * nb, (na, nb)   # the clip is active and the norms agree
    _tight(a, b, 2e-2, "clip_grad_norm")
    _tight(c, b, 2e-2, "max_grad_norm")


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_reduce_with_fp16_loss_scaling_and_an_overflow(tmp_path):
    """fp16 with the dynamic loss scale on the fused path; in step 1 an absurd loss scale set on the host makes
    the gradients overflow: every rank must skip that step and lower the scale, like the NCCL path does."""
    case = {"opt": "sgd", "layers": 2, "iters": 4, "fp16": True, "inject_inf": 1}
    a = _run(2, dict(case, out=str(tmp_path / "a.pt")))
    b = _run(2, dict(case, out=str(tmp_path / "b.pt")), {"RANNC_FUSED_GRAD_ALLREDUCE": "false"})
    assert all(i["fused"] and i["err"] == 0 for i in a["infos"])
    assert all(i["skipped"] == [True] for i in a["infos"] + b["infos"]), (a["infos"], b["infos"])
    assert a["infos"][0]["scale"] == b["infos"][0]["scale"] and a["infos"][1]["scale"] == b["infos"][0]["scale"]
    _tight(a, b, 3e-2, "fp16")


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_load_state_dict_into_a_deployed_module_on_the_fused_path(tmp_path):
    res = _run(2, {"out": str(tmp_path / "r.pt"), "reload": True})
    assert all(i["fused"] and i["reload_ok"] and i["err"] == 0 for i in res["infos"]), res["infos"]


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_reduce_without_multimem(tmp_path):
    a = _run(2, {"out": str(tmp_path / "a.pt")}, {"RANNC_USE_MULTIMEM": "0"})
    b = _run(2, {"out": str(tmp_path / "b.pt")}, {"RANNC_FUSED_GRAD_ALLREDUCE": "false"})
    assert all(i["err"] == 0 for i in a["infos"])
    _compare(a, b, 2e-2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_pipeline_over_two_gpus_matches_data_parallel(tmp_path):
    pp = _run(2, {"out": str(tmp_path / "pp.pt"), "zero": False}, {"RANNC_PARTITION_NUM": "2"})
    dp = _run(2, {"out": str(tmp_path / "dp.pt"), "zero": False})
    assert pp["infos"][0]["stages"] == 2 and dp["infos"][0]["stages"] == 1
    _compare(pp, dp, 3e-2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tensor_partitioned_linear_over_peers(tmp_path):
    n = 4 if _ngpu() >= 4 else 2
    infos = _run(n, {"out": str(tmp_path / "distop.json")}, {"NCCL_NVLS_ENABLE": "0"}, worker="distop_worker.py")
    for i in infos:
        assert i["err_word"] == 0
        for k, v in i["errs"].items():
            assert v < 2e-2, (k, v)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_force_dist_matmul_over_two_gpus(tmp_path):
    env = {"NCCL_NVLS_ENABLE": "0", "RANNC_USE_MULTIMEM": "0"}
    a = _run(2, {"out": str(tmp_path / "a.pt")}, dict(env, RANNC_FORCE_DIST_MATMUL="true"))
    b = _run(2, {"out": str(tmp_path / "b.pt")}, env)
    assert a["infos"][0]["sliced"] > 0 and b["infos"][0]["sliced"] == 0
    assert all(i["err"] == 0 for i in a["infos"])
    _compare(a, b, 3e-2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_dist_param_weights_stay_sliced_on_the_kernels(tmp_path):
    """A model declared under DistributeModelParams with keep_dist_params_sharded: its linear weights are never
    assembled whole -- each GPU keeps one column slice, the GEMM gathers the peers' slices in its prologue and
    scatters the weight gradient in its epilogue -- and training matches the run with whole weights."""
    env = {"NCCL_NVLS_ENABLE": "0", "RANNC_USE_MULTIMEM": "0"}
    case = {"opt": "sgd", "zero": False, "iters": 3}
    a = _run(2, dict(case, dist_param=True, out=str(tmp_path / "a.pt")),
             dict(env, RANNC_KEEP_DIST_PARAMS_SHARDED="true"))
    b = _run(2, dict(case, out=str(tmp_path / "b.pt")), env)
    assert a["infos"][0]["sliced"] > 0 and b["infos"][0]["sliced"] == 0
    assert all(i["err"] == 0 for i in a["infos"])
    for la, lb in zip(a["infos"][0]["losses"], b["infos"][0]["losses"]):
        assert abs(la - lb) < 3e-2 * abs(lb)
    _tight(a, b, 3e-2, "keep_dist_params_sharded")


@pytest.mark.skipif(_ngpu() < 1, reason="needs a GPU")
def test_offloaded_optimizer_state_matches_resident(tmp_path):
    # fp32 master weights and Adam moments in pinned host memory, streamed through the device in chunks
    env = {"RANNC_OFFLOAD_CHUNK_NUMEL": "1048576"}
    a = _run(1, {"out": str(tmp_path / "a.pt"), "zero": False, "offload": True}, env)
    b = _run(1, {"out": str(tmp_path / "b.pt"), "zero": False})
    assert all(i["err"] == 0 for i in a["infos"])
    for la, lb in zip(a["infos"][0]["losses"], b["infos"][0]["losses"]):
        assert abs(la - lb) < 1e-2 * abs(lb)
    _compare(a, b, 1e-2)
    k0 = sorted(a["opt"]["state"].keys())[0]
    assert torch.allclose(a["opt"]["state"][k0]["exp_avg"].float(), b["opt"]["state"][k0]["exp_avg"].float(),
                          rtol=1e-2, atol=1e-5)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("model", ["bert", "resnet"])
def test_fused_reduce_sgd_momentum(tmp_path, model):
    """The fused reduce-scatter + update + all-gather kernel in its SGD-momentum mode; with the ResNet the
    fp32 batch-norm parameters form a group of their own that takes the collective path beside it."""
    case = {"opt": "sgd", "model": model, "iters": 4}
    a = _run(2, dict(case, out=str(tmp_path / "a.pt")))
    b = _run(2, dict(case, out=str(tmp_path / "b.pt")), {"RANNC_FUSED_GRAD_ALLREDUCE": "false"})
    assert all(i["fused"] for i in a["infos"]) and not any(i["fused"] for i in b["infos"])
    assert all(i["err"] == 0 for i in a["infos"])
    # the two paths sum the gradients in a different order; batch norm amplifies that rounding noise a little
    # with every step, so the ResNet gets a wider band
    ltol, ptol = (3e-2, 2e-2) if model == "bert" else (1e-1, 0.0)
    la0, lb0 = a["infos"][0]["losses"][0], b["infos"][0]["losses"][0]
    assert abs(la0 - lb0) < 5e-3 * abs(lb0)            # same forward before any update
    for la, lb in zip(a["infos"][0]["losses"], b["infos"][0]["losses"]):
        assert abs(la - lb) < ltol * abs(lb)
    for k in a["sd"]:
        x, y = a["sd"][k].float(), b["sd"][k].float()
        assert torch.isfinite(x).all(), k
        if model == "bert":
            assert (x - y).abs().max().item() <= ptol * (y.abs().max().item() + 1e-3) + 2e-3, k
    # For the ResNet only the losses are compared: two runs of the SAME path already differ by about as much as
    # the two paths do (reductions with atomics in the split-K and batch-norm kernels, cuDNN's stem gradient),
    # and batch norm turns that into O(1) relative differences of its zero-initialised shifts within a few steps.

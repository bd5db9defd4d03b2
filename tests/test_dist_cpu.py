"""Full trace -> partition -> deploy -> train path on CPU ranks (gloo), checked against eager PyTorch on the
global batch: losses / outputs, gradients, parameters after the step, and the checkpoint round trip."""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_case(world, case, env_extra=None, timeout=240, worker="dist_worker.py", every_rank=False):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ)
        env.update({"RANK": str(r), "WORLD_SIZE": str(world), "LOCAL_RANK": str(r), "MASTER_ADDR": "127.0.0.1",
                    "MASTER_PORT": str(port), "RANNC_FORCE_CPU": "1", "OMP_NUM_THREADS": "1",
                    "RANNC_LOG_LEVEL": "warning"})
        env.update(env_extra or {})
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
    first = None
    for o in (outs if every_rank else outs[:1]):
        res = None
        for line in o.splitlines():
            if line.startswith("RESULT "):
                res = json.loads(line[7:])
        assert res is not None, "a rank gave no result:\n" + "\n----\n".join(o[-3000:] for o in outs)
        assert res["ok"], json.dumps(res, indent=1)[:4000]
        first = first or res
    return first


@pytest.mark.parametrize("model", ["basic", "forkjoin", "shared_input", "loss", "emb", "tied", "layernorm"])
def test_dp2(model):
    run_case(2, {"model": model, "batch": 8})


@pytest.mark.parametrize("model", ["deep", "loss", "forkjoin", "shared_input", "tied"])
def test_pp2(model):
    res = run_case(2, {"model": model, "batch": 8}, {"RANNC_PARTITION_NUM": "2"})
    assert res["ranks"][0]["stages"] == 2


@pytest.mark.parametrize("model", ["small_param", "const_mul", "func_loop", "buffer_ro"])
def test_zoo_corner_models_dp2_and_pp2(model):
    # 0-dim and 2-wide parameters, a lifted tensor constant, a layer reused by an unrolled loop, a read-only buffer
    run_case(2, {"model": model, "batch": 8})
    res = run_case(2, {"model": model, "batch": 8}, {"RANNC_PARTITION_NUM": "2"})
    assert res["ranks"][0]["stages"] == 2


def test_parameter_free_models():
    # nothing to place or reduce: forward only, and gradients of the inputs when they are asked for; an output
    # that is an input gets an alias node, and a forced stage count is clamped to the single block there is
    run_case(2, {"model": "one_op", "batch": 8})
    run_case(2, {"model": "one_op", "batch": 8, "input_grad": True}, {"RANNC_PARTITION_NUM": "2"})
    run_case(2, {"model": "identity", "batch": 8, "input_grad": True})
    res = run_case(2, {"model": "identity", "batch": 8}, {"RANNC_PARTITION_NUM": "2"})
    assert res["ranks"][0]["stages"] == 1


def test_overwritten_buffer_crosses_a_stage_boundary():
    # the buffer's new value is a statistic over the batch ([16], no batch dimension): it is computed in the
    # first stage and read in the second, so it must be moved whole instead of being split into rows
    run_case(1, {"model": "buffer_rw", "batch": 8})
    res = run_case(2, {"model": "buffer_rw", "batch": 8}, {"RANNC_PARTITION_NUM": "2"})
    assert res["ranks"][0]["stages"] == 2


def test_amp_gradients_reduced_in_master_precision_with_accumulation():
    # allreduce_amp_master_params: the fp32 master gradients are what the ranks exchange; four accumulation
    # steps with the reduction delayed to the last one (reference matrix: test/test_simple.py:37-46)
    run_case(2, {"model": "layernorm", "batch": 8, "amp": True, "ar_master": True, "accum": 4, "opt": "adam",
                 "tol": 1e-1})


def test_load_state_dict_into_a_deployed_module():
    # values written into the flat buffers (and fp32 masters / ZeRO shards / column slices) without re-partitioning
    run_case(2, {"model": "tied", "batch": 8, "reload": True}, {"RANNC_PARTITION_NUM": "2"})
    run_case(2, {"model": "layernorm", "batch": 8, "amp": True, "zero": True, "opt": "adam", "tol": 1e-1,
                 "reload": True})
    run_case(2, {"model": "deep", "batch": 8, "reload": True}, {"RANNC_FORCE_DIST_MATMUL": "true"})
    run_case(1, {"model": "bn", "batch": 8, "reload": True})


def test_pp2_dp2_pipeline2():
    res = run_case(4, {"model": "deep", "batch": 16}, {"RANNC_PARTITION_NUM": "2", "RANNC_PIPELINE_NUM": "2"})
    assert res["ranks"][0]["stages"] == 2 and res["ranks"][0]["pipeline"] == 2


def test_batchnorm_buffers_single_rank():
    # running statistics and num_batches_tracked follow eager exactly when one replica sees the whole batch
    run_case(1, {"model": "bn", "batch": 8})


def test_batchnorm_buffers_two_stages():
    res = run_case(2, {"model": "bn", "batch": 8}, {"RANNC_PARTITION_NUM": "2"})
    assert res["ranks"][0]["stages"] == 2


@pytest.mark.parametrize("opt", ["sgd", "adam"])
def test_force_dist_matmul_dp2(opt):
    # every linear weight is stored as column slices over the two replicas; forward, gradients, updates,
    # state_dict and the gathered optimizer state must still match eager on the full batch
    res = run_case(2, {"model": "deep", "batch": 8, "opt": opt}, {"RANNC_FORCE_DIST_MATMUL": "true"})
    assert res["ranks"][0]["sliced"] > 0


def test_force_dist_matmul_with_pipeline():
    res = run_case(4, {"model": "deep", "batch": 16}, {"RANNC_FORCE_DIST_MATMUL": "true",
                                                       "RANNC_PARTITION_NUM": "2"})
    assert res["ranks"][0]["stages"] == 2 and res["ranks"][0]["sliced"] > 0


def test_verify_partitioning_runs_with_two_stages():
    # the in-product self check: whole graph vs chained stage graphs on rank 0
    run_case(2, {"model": "bn", "batch": 8}, {"RANNC_PARTITION_NUM": "2", "RANNC_VERIFY_PARTITIONING": "true"})
    run_case(2, {"model": "forkjoin", "batch": 8}, {"RANNC_PARTITION_NUM": "2", "RANNC_VERIFY_PARTITIONING": "true"})


def test_gather_inputs_false_rank0_feeds_the_whole_batch():
    run_case(2, {"model": "basic", "batch": 8, "gather_inputs": False})
    run_case(2, {"model": "deep", "batch": 8, "gather_inputs": False}, {"RANNC_PARTITION_NUM": "2"})


def test_mixed_precision_master_weights_dp2():
    # bf16 compute with fp32 master weights and gradients on CPU ranks; compared loosely with fp32 eager
    run_case(2, {"model": "layernorm", "batch": 8, "amp": True, "opt": "adam", "tol": 1e-1})


def test_mixed_precision_with_zero_sharding_dp2():
    run_case(2, {"model": "layernorm", "batch": 8, "amp": True, "zero": True, "opt": "adam", "tol": 1e-1})
    run_case(2, {"model": "deep", "batch": 8, "amp": True, "zero": True, "accum": 2, "tol": 1e-1})


def test_zero_sharding_over_several_buckets():
    # a bucket of a few hundred bytes: every flat buffer splits into many buckets and each rank owns a slice of
    # each, so a rank's master / moment buffers are the concatenation of non-adjacent slices; gradients,
    # updates, state_dict, the gathered optimizer state and load_state_dict into the deployed module must agree
    env = {"RANNC_GRAD_BUCKET_MB": "0.0005"}
    res = run_case(2, {"model": "layernorm", "batch": 8, "amp": True, "zero": True, "opt": "adam", "tol": 1e-1,
                       "reload": True, "want_buckets": 2}, env)
    assert min(r["buckets"] for r in res["ranks"]) >= 2
    run_case(2, {"model": "deep", "batch": 8, "amp": True, "zero": True, "accum": 2, "tol": 1e-1}, env)
    run_case(3, {"model": "deep", "batch": 12, "amp": True, "zero": True, "opt": "adam", "tol": 1e-1},
             dict(env, RANNC_LIMIT_DEV_NUM_POT="false", RANNC_PARTITION_NUM="1", RANNC_REPLICA_NUM="3"))


def test_clip_grad_norm_matches_eager_under_zero():
    # the norm is taken over the reduced gradients (each element once across the ranks) and the clipped
    # update follows eager's clip_grad_norm_ on the full batch
    run_case(2, {"model": "deep", "batch": 8, "clip": 0.05})
    run_case(2, {"model": "deep", "batch": 8, "amp": True, "zero": True, "clip": 0.05, "tol": 1e-1},
             {"RANNC_GRAD_BUCKET_MB": "0.0005"})


def test_two_param_groups_checkpoint_loads_into_plain_torch():
    # decay / no-decay groups listed in an order that differs from the model's: the gathered state is keyed by
    # the optimizer's own numbering, so a fresh torch.optim.Adam built the same way accepts it as is
    run_case(2, {"model": "deep", "batch": 8, "opt": "adam", "two_groups": True})
    run_case(2, {"model": "deep", "batch": 8, "opt": "adam", "two_groups": True, "amp": True, "zero": True,
                 "tol": 1e-1})


@pytest.mark.parametrize("env", [{}, {"RANNC_PARTITION_NUM": "2"}])
def test_dist_param_model_declared_in_shards(env):
    run_case(2, {"model": "deep", "batch": 8, "dist_param": True}, env)


def test_dist_param_weights_stay_sliced_through_training():
    # keep_dist_params_sharded: the linear weights declared in shards are re-cut into column slices over the
    # replicas and never exist whole; everything else of the run must still match eager on the full batch
    res = run_case(2, {"model": "deep", "batch": 8, "dist_param": True}, {"RANNC_KEEP_DIST_PARAMS_SHARDED": "true"})
    assert res["ranks"][0]["sliced"] > 0
    res = run_case(4, {"model": "deep", "batch": 16, "dist_param": True, "opt": "adam"},
                   {"RANNC_KEEP_DIST_PARAMS_SHARDED": "true", "RANNC_PARTITION_NUM": "2"})
    assert res["ranks"][0]["sliced"] > 0 and res["ranks"][0]["stages"] == 2


def test_input_gradients_dp2_and_pp2():
    run_case(2, {"model": "deep", "batch": 8, "input_grad": True})
    run_case(2, {"model": "deep", "batch": 8, "input_grad": True}, {"RANNC_PARTITION_NUM": "2"})


def test_pp_checkpointing():
    run_case(2, {"model": "loss", "batch": 8}, {"RANNC_PARTITION_NUM": "2", "RANNC_PIPELINE_NUM": "2",
                                                "RANNC_CHECKPOINTING": "true"})


def test_pp_checkpointing_with_recompute_self_check():
    # verify_recomp: every recomputed stage output is compared with the forward pass's
    run_case(2, {"model": "loss", "batch": 8}, {"RANNC_PARTITION_NUM": "2", "RANNC_PIPELINE_NUM": "2",
                                                "RANNC_CHECKPOINTING": "true", "RANNC_VERIFY_RECOMP": "true"})


def test_grad_accumulation():
    run_case(2, {"model": "loss", "batch": 8, "accum": 2})


def test_adam_dp2():
    run_case(2, {"model": "layernorm", "batch": 8, "opt": "adam"})


def test_uneven_stage_replicas():
    # 3 ranks cannot be split evenly: stage counts / replica counts come from the search
    run_case(3, {"model": "deep", "batch": 12}, {"RANNC_LIMIT_DEV_NUM_POT": "false"})


def test_peer_failure_is_detected_on_the_host(tmp_path):
    """Failure detection without any device fault: a rank leaves between steps; the survivor's watchdog sees
    the missing heartbeat file and the next forward raises CommError before anything is launched."""
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ)
        env.update({"RANK": str(r), "WORLD_SIZE": "2", "LOCAL_RANK": str(r), "MASTER_ADDR": "127.0.0.1",
                    "MASTER_PORT": str(port), "RANNC_FORCE_CPU": "1", "OMP_NUM_THREADS": "1",
                    "RANNC_LOG_LEVEL": "warning", "RANNC_RUN_WATCHDOG": "true",
                    "RANNC_WATCHDOG_LOCKFILE_DIR": str(tmp_path), "RANNC_WATCHDOG_PERIOD_S": "0.1",
                    "RANNC_WATCHDOG_STALE_S": "5"})
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "failure_worker.py")], env=env,
                                      cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert "LEFT" in outs[1], outs[1][-2000:]
    assert "DETECTED" in outs[0] and "NOT DETECTED" not in outs[0], outs[0][-2000:]


def test_failed_collective_is_retried_after_recreating_the_communicators():
    """A collective that raises on the host (failure injected before anything is issued) is followed by
    re-creation of every communicator and one retry; training continues with unchanged numbers, and a failure
    that persists beyond the configured retries surfaces as CommError."""
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ)
        env.update({"RANK": str(r), "WORLD_SIZE": "2", "LOCAL_RANK": str(r), "MASTER_ADDR": "127.0.0.1",
                    "MASTER_PORT": str(port), "RANNC_FORCE_CPU": "1", "OMP_NUM_THREADS": "1",
                    "RANNC_LOG_LEVEL": "error", "RANNC_COMM_RETRY": "1", "RANNC_COMM_RETRY_WAIT_S": "0.05"})
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "retry_worker.py")], env=env,
                                      cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for o in outs:
        assert "RETRY_OK" in o, o[-3000:]


@pytest.mark.parametrize("world,case,env", [
    (1, {"batch": 4}, {}),
    (1, {"batch": 8, "clip": 0.5}, {"RANNC_PIPELINE_NUM": "2"}),          # micro-batches: gradients accumulate on the host
    (2, {"batch": 8}, {}),
    (2, {"batch": 8, "zero": True}, {"RANNC_GRAD_BUCKET_MB": "0.25"}),
    (2, {"batch": 8, "opt": "sgd"}, {"RANNC_PARTITION_NUM": "2"}),          # two pipeline stages, each streamed
])
def test_parameters_streamed_from_host_memory(world, case, env):
    """offload_params with offload_param_window_mb: 16-bit parameters and fp32 gradients live in host memory, a
    stage runs segment by segment with at most a window of parameters on the device, and training matches the
    run with everything resident (reference: per-operator offload hooks, src/torch/TorchDriver.cpp:318-374)."""
    res = run_case(world, case, env, timeout=600, worker="stream_worker.py", every_rank=True)
    assert res["info"]["segments"] >= 3 and res["info"]["streamed_groups"] >= 1


@pytest.mark.parametrize("world,case,env", [
    (1, {"batch": 8, "segments": 4}, {"RANNC_CHECKPOINTING": "true", "RANNC_PIPELINE_NUM": "2"}),
    (2, {"batch": 8, "segments": 3, "zero": True}, {"RANNC_CHECKPOINTING": "true", "RANNC_PARTITION_NUM": "2",
                                                     "RANNC_PIPELINE_NUM": "2"}),
])
def test_recomputation_segment_by_segment_matches_stage_recomputation(world, case, env):
    """checkpoint_segments: a checkpointed stage keeps the values at its segment boundaries and recomputes one
    segment at a time in backward; same dropout masks, same gradients as recomputing the whole stage."""
    res = run_case(world, case, env, timeout=600, worker="stream_worker.py", every_rank=True)
    assert res["info"]["segments"] >= 3


@pytest.mark.parametrize("world,case", [
    (1, {"model": "loss", "batch": 8}),
    (2, {"model": "loss", "batch": 16, "opt": "adam"}),
    (2, {"model": "loss", "batch": 16, "amp": True, "zero": True, "opt": "adam", "tol": 1e-1}),
    (2, {"model": "loss", "batch": 16, "accum": 2}),
])
def test_backward_interleaved_with_forward_per_micro_batch(world, case):
    """interleave_backward: a one-stage plan runs each micro-batch's backward right after its forward (one
    micro-batch's activations alive instead of all of them); losses, gradients, updates and checkpoints equal
    eager's on the full batch."""
    res = run_case(world, case, {"RANNC_INTERLEAVE_BACKWARD": "true", "RANNC_PIPELINE_NUM": "4",
                                 "RANNC_PARTITION_NUM": "1"})
    assert res["ranks"][0]["stages"] == 1 and res["ranks"][0]["pipeline"] == 4
    assert all(r["interleaved"] >= 3 for r in res["ranks"])


def test_interleaved_backward_refuses_another_upstream_gradient():
    run_case(1, {"model": "loss", "batch": 8, "bad_upstream": True},
             {"RANNC_INTERLEAVE_BACKWARD": "true", "RANNC_PIPELINE_NUM": "4", "RANNC_PARTITION_NUM": "1"})


@pytest.mark.parametrize("case,env", [
    ({"model": "deep", "batch": 8, "accessors": True}, {"RANNC_PARTITION_NUM": "2"}),
    ({"model": "layernorm", "batch": 8, "amp": True, "zero": True, "opt": "adam", "tol": 1e-1, "accessors": True},
     {"RANNC_GRAD_BUCKET_MB": "0.0005"}),
])
def test_low_level_parameter_accessors(case, env):
    """get_local_param_range / get_local_param_segment / sync_param / _sync_orig_params
    (reference: src/main.cpp:271-402, pyrannc/__init__.py:539-572)."""
    run_case(2, case, env)


def test_package_exports_the_reference_names():
    import rannc_b200 as pyrannc

    for name in ("RaNNCModule", "get_rank", "get_world_size", "barrier", "clear", "delay_grad_allreduce", "keep_graph",
                 "sync_params_on_init", "recreate_all_communicators", "show_deployment", "_run_dp_dry",
                 "_dump_events", "all_gather", "patch_optimizer", "abort_all_processes", "store_dist_param",
                 "load_dist_param", "set_dist_param", "get_dist_param_range", "set_dist_param_dtype"):
        assert hasattr(pyrannc, name), name
    for name in ("sync_param", "sync_param_grad", "sync_param_zero", "align_params", "get_local_param_range",
                 "get_local_param_segment", "_sync_orig_params", "clip_grad_norm", "_calc_grad_norm", "undeploy",
                 "enable_dropout", "save_deployment", "is_checkpointing_enabled"):
        assert hasattr(pyrannc.RaNNCModule, name), name
    assert hasattr(pyrannc.tensor_coll, "bcast_tensor") and hasattr(pyrannc.tensor_coll, "allreduce_tensor")


def test_bert_pretraining_example_saves_and_resumes_across_world_sizes(tmp_path):
    """examples/bert_pretrain.py: two ranks, two pipeline stages, the model declared in shards, two optimizer
    groups, clipping; the checkpoint it writes is resumed by a single process (another partitioning)."""
    ck = tmp_path / "bert.pt"
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), RANNC_FORCE_CPU="1", OMP_NUM_THREADS="1", RANNC_LOG_LEVEL="warning",
                   RANNC_PARTITION_NUM="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "examples", "bert_pretrain.py"), "--steps",
                                       "3", "--dist-params", "--save", str(ck)], env=env, cwd=ROOT,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n----\n".join(o[-2000:] for o in outs)
    first = [float(ln.split("loss ")[1].split()[0]) for ln in outs[0].splitlines() if ln.startswith("step ")]
    assert len(first) == 3 and ck.exists()
    saved_val = [float(ln.split()[-1]) for ln in outs[0].splitlines() if ln.startswith("held-out loss")][0]
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", RANNC_FORCE_CPU="1", RANNC_LOG_LEVEL="warning",
               MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "bert_pretrain.py"), "--steps", "2", "--resume",
                        str(ck)], env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    resumed = [ln for ln in r.stdout.splitlines() if ln.startswith("step ")]
    assert resumed and resumed[0].startswith("step 3:")
    # the weights the single process starts from are the ones the two ranks trained: same held-out loss
    got_val = [float(ln.split()[-1]) for ln in r.stdout.splitlines() if ln.startswith("resumed at step 3")][0]
    assert abs(got_val - saved_val) < 2e-2 * abs(saved_val), (got_val, saved_val)

"""trace -> profile -> partition -> deployment (the body of the reference's RaNNCModule::init,
src/comp/RaNNCModule.cpp:160-501, steps 4-7).

Planning is deterministic given the graph, the profiles and the configuration, so
every rank can run it; the runtime lets rank 0 plan and broadcasts the msgpack
deployment so that measured profiles (which differ slightly per rank) cannot make
ranks disagree.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Optional

from .. import _core
from ..utils.config import conf
from ..utils.log import get_logger

logger = get_logger("Decomposer")


@dataclass
class Plan:
    deployment: "_core.Deployment"
    estimates: list
    ml_nodes: int
    dev_mem: int


def device_memory_budget(total_bytes: int) -> int:
    """min(total, mem_limit_gb) x (1 - mem_margin) (reference: MLPartDecomposer.cpp:15-24)."""
    limit_gb = int(conf("mem_limit_gb"))
    mem = total_bytes
    if limit_gb > 0:
        mem = min(mem, limit_gb * (1 << 30)) if mem > 0 else limit_gb * (1 << 30)
    return int(mem * (1.0 - float(conf("mem_margin"))))


def make_partitioning_conf(world_size: int, batch_size: int, dev_mem: int, use_amp: bool, enable_zero: bool,
                           offload_params: bool) -> "_core.PartitioningConf":
    c = _core.PartitioningConf()
    dry = int(conf("partitioning_dry_run_np"))
    c.dev_num = dry if dry > 0 else world_size
    c.batch_size = batch_size
    c.dev_mem = dev_mem
    c.use_amp_master_params = use_amp
    c.enable_zero = enable_zero
    c.offload_params = offload_params
    c.force_dist_matmul = bool(conf("force_dist_matmul")) or bool(conf("keep_dist_params_sharded"))
    c.opt_param_factor = int(conf("opt_param_factor"))
    c.min_pipeline = int(conf("min_pipeline"))
    c.max_pipeline = int(conf("max_pipeline"))
    c.min_pipeline_bs = int(conf("min_pipeline_bs"))
    c.min_partition_num = int(conf("min_partition_num"))
    c.max_partition_num = int(conf("max_partition_num"))
    c.cfg_partition_num = int(conf("partition_num"))
    c.cfg_replica_num = int(conf("replica_num"))
    c.cfg_pipeline_num = int(conf("pipeline_num"))
    c.limit_dev_num_pot = bool(conf("limit_dev_num_pot"))
    c.limit_dev_num_more_than_bs = bool(conf("limit_dev_num_more_than_bs"))
    c.dp_search_all = bool(conf("dp_search_all"))
    c.do_coarsening = bool(conf("do_coarsening"))
    c.do_uncoarsening = bool(conf("do_uncoarsening"))
    c.coarsen_by_time = bool(conf("coarsen_by_time"))
    c.checkpointing = bool(conf("checkpointing"))
    c.checkpointing_no_last = bool(conf("checkpointing_no_last"))
    c.prefer_no_checkpointing = bool(conf("prefer_no_checkpointing"))
    link = _core.LinkModel()
    link.p2p_bytes_per_us = float(conf("p2p_gbs")) * 1e3
    link.allreduce_bytes_per_us = float(conf("allreduce_gbs")) * 1e3
    c.link = link
    return c


def _fmt_table(estimates) -> str:
    rows = ["Estimated profiles of subgraphs (times in us, sizes in bytes)"]
    for e in estimates:
        p = e.profile
        rows.append(
            f"  {e.name}: repl={e.repl} micro_batch={e.micro_batch} fwd={p.fwd_time} bwd={p.bwd_time} "
            f"allreduce={e.allreduce_us:.0f} in={p.input_size} out={p.output_size} params={p.param_size} "
            f"mem={e.total_mem} (fwd+bwd={p.param_size + p.activation_size + p.working_mem} opt={e.opt_mem} "
            f"comm={e.comm_mem})")
    return "\n".join(rows)


def _calibrate(pm, ml, ir_graph, node_profiles, pconf, sp):
    """One measurement per block of the coarsened graph (forward + backward on the device at the micro-batch
    size a pure data-parallel plan would use); the operator profiles of the block are scaled to it.  With
    ``measure_subgraphs`` the stage search additionally measures the stages it considers, up to
    ``max_measured_subgraphs`` of them (reference: every candidate is profiled, GraphProfiler.cpp:245-415)."""
    owned = {n.id for n in ir_graph.nodes if n.is_batch or n.is_criterion}
    bs = max(1, int(pconf.batch_size) // max(1, int(pconf.dev_num)))
    blocks = [(n.id, [i for i in n.sub_nodes if i in owned], n.graph) for n in ml.nodes]
    graphs = {n.id: n.graph for n in ml.nodes}

    def additive(name):
        p = pm.profile(graphs[name], bs, False)
        return float(p.fwd_time), float(p.bwd_time), float(p.activation_size)

    new_profiles, report = sp.calibrate(node_profiles, blocks, bs, additive)
    if report:
        logger.info("Measured %d block(s) at micro-batch %d: measured / estimated (fwd, bwd, kept bytes) %s", len(report),
                    bs, ", ".join(f"{n}: {rf:.2f} {rb:.2f} {ra:.2f}" for n, _, rf, rb, ra in report))
    pm2 = _core.ProfileModel(ir_graph, new_profiles, pconf.link)
    if bool(conf("measure_subgraphs")):
        pm2.set_subgraph_measure(lambda ids, b, ckpt: sp.measure(list(ids), int(b), bool(ckpt)),
                                 int(conf("max_measured_subgraphs")))
    return pm2, new_profiles


def _load_alloc_solution(pconf):
    """``load_alloc_solutions``: reuse a stage assignment written by ``save_alloc_solutions`` instead of
    searching again (files ``<alloc_solutions_file_prefix>_s<stages>_p<micro-batches>.bin``).  A forced
    ``partition_num`` / ``pipeline_num`` selects among several files; otherwise the one with the fewest stages
    is taken.  Returns None when there is no matching file."""
    import glob
    import re

    prefix = str(conf("alloc_solutions_file_prefix"))
    found = []
    for path in glob.glob(glob.escape(prefix) + "_s*_p*.bin"):
        m = re.search(r"_s(\d+)_p(\d+)\.bin$", path)
        if not m:
            continue
        stages, pipe = int(m.group(1)), int(m.group(2))
        if pconf.cfg_partition_num > 0 and stages != pconf.cfg_partition_num:
            continue
        if pconf.cfg_pipeline_num > 0 and pipe != pconf.cfg_pipeline_num:
            continue
        found.append((stages, pipe, path))
    if not found:
        logger.warning("load_alloc_solutions: no file matches %s_s*_p*.bin; searching instead", prefix)
        return None
    found.sort()
    with open(found[0][2], "rb") as f:
        sol = _core.AllocSolution.loads(f.read())
    logger.info("Loaded the stage assignment from %s", found[0][2])
    return sol


def plan(ir_graph, node_profiles: Dict[str, "_core.NodeProfile"], world_size: int, global_batch: int,
         dev_total_mem: int, use_amp: bool, enable_zero: bool, offload_params: bool, dep_id: str,
         load_deployment: Optional[str] = None, subgraph_profiler=None, interleave: bool = False) -> Plan:
    """``ir_graph`` must already be scaled to the global batch size.  ``subgraph_profiler``
    (``profiler.SubgraphProfiler``): when given, every block of the coarsened graph is measured once and the
    operator profiles are calibrated to it; with ``measure_subgraphs`` the stage search measures its candidate
    stages themselves."""
    if dev_total_mem == 0 and int(conf("partitioning_dry_run_np")) > 0 and int(conf("mem_limit_gb")) <= 0:
        # a dry run on a machine without the target device plans for a B200's 180 GB unless told otherwise
        dev_total_mem = 180 * 10 ** 9
    dev_mem = device_memory_budget(dev_total_mem)
    pconf = make_partitioning_conf(world_size, global_batch, dev_mem, use_amp, enable_zero, offload_params)
    pconf.interleave_single_stage = bool(interleave)

    load_path = load_deployment or (str(conf("deployment_file")) if bool(conf("load_deployment")) else None)
    if load_path:
        with open(load_path, "rb") as f:
            dep, ws, dm = _core.load_deployment(f.read())
        # a deployment is only valid for the world size and device memory it was planned for
        # (reference: src/graph/DeploymentSerializer.cpp:34-46)
        if ws != pconf.dev_num:
            raise RuntimeError(f"deployment file was made for {ws} ranks, this job has {pconf.dev_num}")
        if dm != dev_mem:
            raise RuntimeError(f"deployment file was made for {dm} bytes of device memory, this device has {dev_mem}")
        logger.info("Loaded deployment from %s", load_path)
        return Plan(dep, [], len(dep.fwd_graph_order), dev_mem)

    # more stages than devices can be forced for testing: search with one virtual device per stage,
    # the allocation then wraps around the real ranks
    real_dev = pconf.dev_num
    if pconf.cfg_partition_num > pconf.dev_num:
        pconf.dev_num = pconf.cfg_partition_num
        pconf.cfg_replica_num = 1
        pconf.limit_dev_num_more_than_bs = False

    pm = _core.ProfileModel(ir_graph, node_profiles, pconf.link)
    decomposer = str(conf("decomposer"))
    estimates = []
    if decomposer == "fair_weight":
        sol = _core.fair_weight_decompose(pm, pconf)
        ml_nodes = len(sol.graphs)
    else:
        ml_file = str(conf("mlpart_results_file"))
        if bool(conf("load_mlpart_results")) and os.path.exists(ml_file):
            with open(ml_file, "rb") as f:
                ml = _core.MLGraph.loads(f.read())
        else:
            ml = _core.ml_partition(pm, pconf)
            if bool(conf("save_mlpart_results")):
                with open(ml_file, "wb") as f:
                    f.write(ml.dumps())
        ml_nodes = len(ml.nodes)
        logger.info("Coarsened the graph to %d blocks", ml_nodes)
        if subgraph_profiler is not None:
            pm, node_profiles = _calibrate(pm, ml, ir_graph, node_profiles, pconf, subgraph_profiler)
        if 0 < ml_nodes < pconf.cfg_partition_num:
            # a forced stage count cannot exceed the number of blocks there are to distribute
            logger.warning("partition_num=%d is more than the %d block(s) of this model; using %d",
                           pconf.cfg_partition_num, ml_nodes, ml_nodes)
            pconf.cfg_partition_num = ml_nodes
            pconf.dev_num = max(real_dev, ml_nodes)
        if str(conf("dump_dp_cache")):
            with open(str(conf("dump_dp_cache")), "wb") as f:
                f.write(_core.dump_dp_cache(ml, ir_graph, node_profiles, pconf))
        loaded = _load_alloc_solution(pconf) if bool(conf("load_alloc_solutions")) else None
        if loaded is not None:
            sol, estimates, node_json = loaded, [], ""
        else:
            sol, estimates, node_json = _core.dp_staging(pm, ml, pconf)
        if str(conf("dump_dp_node_profiles")) and node_json:
            with open(str(conf("dump_dp_node_profiles")), "w") as f:
                f.write(node_json)
        if bool(conf("save_alloc_solutions")):
            path = f"{conf('alloc_solutions_file_prefix')}_s{len(sol.graphs)}_p{sol.pipeline_num}.bin"
            with open(path, "wb") as f:
                f.write(sol.dumps())
        logger.info(_fmt_table(estimates))
    dep = _core.create_deployment(ir_graph, sol, real_dev, bool(conf("alloc_repl_flat")), dep_id)
    dep.offload_params = offload_params
    dep.force_dist_matmul = bool(conf("force_dist_matmul"))
    err = _core.verify_deployment(dep)
    if err:
        raise RuntimeError("inconsistent deployment: " + err)
    for name in dep.fwd_graph_order:
        logger.info("Assigned subgraph %s to rank(s) %s", name, dep.allocation[name])
    if bool(conf("dump_graph")):
        prefix = str(conf("dump_graph_prefix"))
        for name, sg in dep.subgraphs.items():
            with open(f"{prefix}_{name}.dot", "w") as f:
                f.write(sg.to_dot())
    if bool(conf("save_deployment")):
        with open(str(conf("deployment_file")), "wb") as f:
            f.write(_core.save_deployment(dep, real_dev, dev_mem))
    return Plan(dep, list(estimates), ml_nodes, dev_mem)


def planned_step_ms(estimates, pipeline_num: int) -> float:
    """Step time the stage search expects for its own solution, in ms: the synchronous pipeline runs
    stages + micro-batches - 1 slots each bounded by the slowest stage (forward and backward), then the
    slowest gradient reduction (reference: DPStaging::estimateTime, src/graph/DPStaging.cpp:240-276)."""
    if not estimates:
        return 0.0
    fwd = max(float(e.profile.fwd_time) + e.in_comm_us + e.out_comm_us for e in estimates)
    bwd = max(float(e.profile.bwd_time) + e.in_comm_us + e.out_comm_us for e in estimates)
    slots = len(estimates) + max(1, int(pipeline_num)) - 1
    return (slots * (fwd + bwd) + max(e.allreduce_us for e in estimates)) / 1e3

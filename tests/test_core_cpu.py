"""Unit tests of the native core: msgpack codec, IR, value classification, batch arithmetic, redistribution
plans, segment math, coarsening + stage search on synthetic profiles, deployment files, configuration, event
trace, time counters and the watchdog.  CPU only."""
import json
import os
import time

import pytest

from rannc_b200 import _core


# ----------------------------------------------------------------------------- msgpack
def test_msgpack_roundtrip_and_wire_format():
    obj = {"a": [1, -2, 3.5, None, True, "x" * 40, b"\x00\x01"], "n": {"k": [2 ** 40, -2 ** 40, 2 ** 64 - 1]}}
    data = _core.msgpack_pack(obj)
    assert _core.msgpack_unpack(data) == obj
    # fixed points of the wire format
    assert _core.msgpack_pack(None) == b"\xc0"
    assert _core.msgpack_pack(True) == b"\xc3"
    assert _core.msgpack_pack(5) == b"\x05"
    assert _core.msgpack_pack(-1) == b"\xff"
    assert _core.msgpack_pack(300) == b"\xcd\x01\x2c"
    assert _core.msgpack_pack("ab") == b"\xa2ab"
    assert _core.msgpack_pack([1, 2]) == b"\x92\x01\x02"
    assert _core.msgpack_pack({"a": 1}) == b"\x81\xa1a\x01"
    assert _core.msgpack_pack(2 ** 64 - 1) == b"\xcf" + b"\xff" * 8  # size_t(-1): default list_size


# ----------------------------------------------------------------------------- IR
def _t(dims, elem=None, rg=False):
    return _core.IRType.tensor(elem or _core.IRTensorElemType.FLOAT, dims, rg)


def make_mlp_graph(layers=4, hidden=16, batch=8, with_loss=True):
    g = _core.IRGraph()
    g.name = "mlp"
    g.batch_size = batch
    g.add_input(_core.IRValue("x", _t([batch, hidden])))
    if with_loss:
        g.add_input(_core.IRValue("y", _t([batch], _core.IRTensorElemType.LONG)))
    for i in range(layers):
        g.add_input(_core.IRValue(f"w{i}", _t([hidden, hidden], rg=True), True))
        g.add_input(_core.IRValue(f"b{i}", _t([hidden], rg=True), True))
    prev = "x"
    for i in range(layers):
        g.add_value(_core.IRValue(f"h{i}", _t([batch, hidden])))
        g.add_node(_core.IRNode("aten::linear", [prev, f"w{i}", f"b{i}"], [f"h{i}"], f"lin{i}"))
        g.add_value(_core.IRValue(f"a{i}", _t([batch, hidden])))
        g.add_node(_core.IRNode("aten::relu", [f"h{i}"], [f"a{i}"], f"relu{i}"))
        prev = f"a{i}"
    if with_loss:
        g.add_value(_core.IRValue("loss", _t([])))
        g.add_node(_core.IRNode("aten::cross_entropy_loss", [prev, "y"], ["loss"], "ce"))
        g.add_output("loss")
    else:
        g.add_output(prev)
    g.check()
    return _core.guess_value_types(g)


def test_ir_classification_and_serialisation():
    g = make_mlp_graph()
    vals = g.values
    assert vals["x"].is_batch and not vals["x"].is_param
    assert vals["w0"].is_param and not vals["w0"].is_batch
    assert vals["h2"].is_batch and vals["h2"].batch_size == 8
    assert vals["loss"].is_loss and not vals["loss"].is_batch
    nodes = {n.id: n for n in g.nodes}
    assert nodes["lin0"].is_batch and not nodes["lin0"].is_criterion
    assert nodes["ce"].is_criterion
    g2 = _core.IRGraph.loads(g.dumps())
    assert str(g2) == str(g)
    # positional layout: name, nodes, values, input_names, output_names, is_replicable, batch_size
    raw = _core.msgpack_unpack(g.dumps())
    assert raw[0] == "mlp" and raw[5] is True and raw[6] == 8
    node0 = raw[1][0]
    assert node0[0] == "aten::linear" and node0[1] == ["x", "w0", "b0"] and node0[3] == "lin0"
    v = raw[2]["w0"]
    assert v[0] == "w0" and v[2] is True  # name, type, is_param
    assert v[1][0] == 1 and v[1][2] == [16, 16] and v[1][3] == 3 and v[1][7] == 2 ** 64 - 1  # TENSOR, dims, FLOAT
    assert g.param_size_in_byte() == 4 * (16 * 16 + 16) * 4


def test_batch_reduced_value_is_owned_but_moved_whole():
    # mean over the batch: the node stays in the batch flow (one stage owns it), the value is not split in rows
    g = _core.IRGraph()
    g.batch_size = 8
    g.add_input(_core.IRValue("x", _t([8, 16])))
    stat = _core.IRValue("stat", _t([16]))
    stat.batch_hint = -1
    g.add_value(stat)
    g.add_node(_core.IRNode("aten::mean", ["x"], ["stat"], "mean"))
    y = _core.IRValue("y", _t([8, 16]))
    y.batch_hint = 1
    g.add_value(y)
    g.add_node(_core.IRNode("aten::div", ["x", "stat"], ["y"], "div"))
    g.add_output("y")
    g = _core.guess_value_types(g)
    nodes = {n.id: n for n in g.nodes}
    assert nodes["mean"].is_batch and nodes["div"].is_batch
    assert not g.values["stat"].is_batch and g.values["stat"].batch_size == 0
    assert g.values["y"].is_batch and g.values["y"].batch_size == 8
    # without a hint the propagation rule applies, as in the reference (src/graph/ir.cpp, guessValueTypes)
    h = _core.IRGraph()
    h.batch_size = 8
    h.add_input(_core.IRValue("x", _t([8, 16])))
    h.add_value(_core.IRValue("stat", _t([16])))
    h.add_node(_core.IRNode("aten::mean", ["x"], ["stat"], "mean"))
    h.add_output("stat")
    assert _core.guess_value_types(h).values["stat"].is_batch


def test_traced_batch_statistic_carries_no_batch_dimension():
    import torch

    from rannc_b200.graph import tracer
    from tests import zoo

    tm = tracer.trace(zoo.build("buffer_rw").train(), (torch.randn(8, 16),))
    whole = [v for v in tm.ir.values.values() if not v.is_batch and not v.is_param and not v.is_loss and
             list(v.type.tensor_dim) == [16]]
    assert whole, "the batch statistic should be classified as a value that is moved whole"
    assert all(v.is_batch for v in tm.ir.values.values() if len(v.type.tensor_dim) == 2 and not v.is_param)


def test_scale_graph_unused_and_shared():
    g = make_mlp_graph(batch=8)
    s = _core.scale_graph(g, 2)
    assert s.batch_size == 2 and s.value("h1").type.tensor_dim == [2, 16] and s.value("w1").type.tensor_dim == [16, 16]
    g.add_input(_core.IRValue("dangling", _t([3]), True))
    assert "dangling" in _core.find_unused_values(g)
    r = _core.remove_unused_nodes(g)
    assert "dangling" not in r.input_names and len(r.nodes) == len(g.nodes)
    g3 = _core.IRGraph()
    g3.batch_size = 4
    g3.add_input(_core.IRValue("x", _t([4, 2])))
    g3.add_value(_core.IRValue("a", _t([4, 2])))
    g3.add_value(_core.IRValue("b", _t([4, 2])))
    g3.add_node(_core.IRNode("aten::relu", ["x"], ["a"], "n0"))
    g3.add_node(_core.IRNode("aten::add", ["x", "a"], ["b"], "n1"))
    g3.add_output("b")
    assert _core.shared_inputs(g3) == ["x"]
    # inputs + outputs + input grads + 2 x shared clones
    assert g3.comm_buf_size() == 32 + 32 + 32 + 64


# ----------------------------------------------------------------------------- batch arithmetic
def test_batch_size_calculator_rotation():
    c = _core.BatchSizeCalculator(3, 10)  # micro-batches of 4, 3, 3
    assert [c.split_size(i) for i in range(3)] == [4, 3, 3]
    # 4 rows over 3 ranks: the extra row goes to rank 0 for split 0
    assert [c.local_split_size(r, 3, 0) for r in range(3)] == [2, 1, 1]
    # split 1 (3 rows, previous total 4 -> offset 1): equal
    assert [c.local_split_size(r, 3, 1) for r in range(3)] == [1, 1, 1]
    c2 = _core.BatchSizeCalculator(2, 10)  # 5 + 5 over 2 ranks: the extra row alternates
    assert [c2.local_split_size(r, 2, 0) for r in range(2)] == [3, 2]
    assert [c2.local_split_size(r, 2, 1) for r in range(2)] == [2, 3]
    assert sum(c2.local_batch_size(r, 2) for r in range(2)) == 10
    assert c2.local_dims(10, 2, 0) == [6, 4]  # first dim is 2 x the split size


@pytest.mark.parametrize("src,dst,rows", [([0, 1], [2, 3], 8), ([0, 1, 2, 3], [1, 2], 12), ([0], [0, 1, 2], 7),
                                          ([0, 1, 2], [3], 9)])
def test_redist_args_conserve_rows(src, dst, rows):
    world = 4
    args = [_core.get_redist_args(r, world, rows, src, dst, 0, 1, rows) for r in range(world)]
    for a in range(world):
        for b in range(world):
            assert args[a].sendcounts[b] == args[b].recvcounts[a]
    assert sum(sum(a.sendcounts) for a in args) == rows
    # every destination rank receives one contiguous, gap-free range
    for r in dst:
        got = sorted((args[r].rdispls[s], args[r].recvcounts[s]) for s in range(world) if args[r].recvcounts[s])
        pos = 0
        for d, c in got:
            assert d == pos
            pos += c


def test_segment_math():
    # padded to 16 B x ranks: fp16 -> 8 elements x 4 ranks
    assert _core.aligned_numel(100, 2, 4) == 128
    assert [_core.segment_range(100, 2, 4, i) for i in range(4)] == [(0, 32), (32, 64), (64, 96), (96, 100)]
    # short / empty trailing segments
    assert [_core.segment_range(10, 4, 4, i) for i in range(4)] == [(0, 4), (4, 8), (8, 10), (10, 10)]


# ----------------------------------------------------------------------------- partitioner
def _profiles(g, fwd=100.0, bwd=200.0, act=1 << 20):
    return {n.id: _core.NodeProfile(fwd, bwd, act, 0, True) for n in g.nodes}


def _conf(dev, batch, mem=0):
    c = _core.PartitioningConf()
    c.dev_num, c.batch_size, c.dev_mem = dev, batch, mem
    return c


def test_small_model_is_pure_data_parallel():
    g = make_mlp_graph(layers=10, hidden=512, batch=128, with_loss=False)
    np_ = _profiles(g, act=128 * 512 * 4)
    conf = _conf(2, 128, 38 * 1024 ** 3)
    pm = _core.ProfileModel(g, np_, conf.link)
    ml = _core.ml_partition(pm, conf)
    assert 1 <= len(ml.nodes) <= 32
    sol, est, _ = _core.dp_staging(pm, ml, conf)
    assert len(sol.graphs) == 1 and sol.dev_nums == [2] and sol.pipeline_num == 1


def test_large_model_is_split_into_stages():
    # 100 x Linear(5000): 2.5 G parameters, 10 GB in fp32 -> does not fit one 40 GB device with its optimizer
    # state and gradients (10 + 10 + 20 GB), so the search needs at least two stages
    g = make_mlp_graph(layers=100, hidden=5000, batch=512, with_loss=False)
    np_ = _profiles(g, fwd=300, bwd=600, act=512 * 5000 * 4)
    conf = _conf(8, 512, 38255689728)
    pm = _core.ProfileModel(g, np_, conf.link)
    ml = _core.ml_partition(pm, conf)
    sol, est, _ = _core.dp_staging(pm, ml, conf)
    assert len(sol.graphs) >= 2
    assert sum(sol.dev_nums) == 8
    assert all(e.total_mem < conf.dev_mem for e in est)
    # stages cover the whole model exactly once
    owned = [n.id for sg in sol.graphs for n in sg.nodes if n.is_batch]
    assert sorted(owned) == sorted(n.id for n in g.nodes if n.is_batch)
    dep = _core.create_deployment(g, sol, 8, True, "d")
    assert _core.verify_deployment(dep) == ""
    # ranks are used exactly once
    used = sorted(r for v in dep.allocation.values() for r in v)
    assert used == list(range(8))


def test_nothing_fits_raises():
    g = make_mlp_graph(layers=4, hidden=4096, batch=8, with_loss=False)
    conf = _conf(1, 8, 1 << 20)
    pm = _core.ProfileModel(g, _profiles(g), conf.link)
    ml = _core.ml_partition(pm, conf)
    with pytest.raises(RuntimeError):
        _core.dp_staging(pm, ml, conf)


def test_forced_stage_and_pipeline_counts_and_dry_run():
    g = make_mlp_graph(layers=8, batch=16)
    conf = _conf(4, 16)
    conf.cfg_partition_num, conf.cfg_pipeline_num = 2, 4
    np_ = _profiles(g)
    pm = _core.ProfileModel(g, np_, conf.link)
    ml = _core.ml_partition(pm, conf)
    sol, est, node_json = _core.dp_staging(pm, ml, conf)
    assert len(sol.graphs) == 2 and sol.pipeline_num == 4 and sum(sol.dev_nums) == 4
    assert "nodes" in json.loads(node_json)
    # the dumped cache replays the search without profiles from a device
    cache = _core.dump_dp_cache(ml, g, np_, conf)
    sol2 = _core.run_dp_dry(cache)
    assert [sg.name for sg in sol2.graphs] == [sg.name for sg in sol.graphs] and sol2.dev_nums == sol.dev_nums
    s3 = _core.AllocSolution.loads(sol.dumps())
    assert s3.pipeline_num == 4 and s3.boundaries == sol.boundaries


def _residual_ffn_graph(layers=24, h=64, batch=8):
    """x -> [linear(h -> 4h) -> gelu -> linear(4h -> h) -> add(x)] x layers: wide values inside a block, narrow
    ones (two of them: the sum and the skip) between blocks."""
    g = _core.IRGraph()
    g.name = "res"
    g.batch_size = batch
    g.add_input(_core.IRValue("x", _t([batch, h])))
    for i in range(layers):
        g.add_input(_core.IRValue(f"w{i}a", _t([4 * h, h], rg=True), True))
        g.add_input(_core.IRValue(f"w{i}b", _t([h, 4 * h], rg=True), True))
    prev = "x"
    for i in range(layers):
        g.add_value(_core.IRValue(f"u{i}", _t([batch, 4 * h])))
        g.add_node(_core.IRNode("aten::linear", [prev, f"w{i}a"], [f"u{i}"], f"up{i}"))
        g.add_value(_core.IRValue(f"g{i}", _t([batch, 4 * h])))
        g.add_node(_core.IRNode("aten::gelu", [f"u{i}"], [f"g{i}"], f"act{i}"))
        g.add_value(_core.IRValue(f"d{i}", _t([batch, h])))
        g.add_node(_core.IRNode("aten::linear", [f"g{i}", f"w{i}b"], [f"d{i}"], f"down{i}"))
        g.add_value(_core.IRValue(f"r{i}", _t([batch, h])))
        g.add_node(_core.IRNode("aten::add", [f"d{i}", prev], [f"r{i}"], f"add{i}"))
        prev = f"r{i}"
    g.add_output(prev)
    g.check()
    return _core.guess_value_types(g)


def test_uncoarsening_moves_boundaries_to_a_smaller_cut():
    """Multi-level partitioning: coarsening records which blocks a block was merged from; uncoarsening walks the
    levels back down and lets boundary blocks change sides when that shrinks the cut.  The result must still be
    a partition of all operators into a DAG of convex blocks that the stage search accepts."""
    import random

    g = _residual_ffn_graph()
    random.seed(0)
    np_ = {n.id: _core.NodeProfile(50.0 + random.random() * 100, 100.0 + random.random() * 200, 1 << 16, 0, True)
           for n in g.nodes}
    conf = _conf(4, 8)
    conf.min_partition_num = 8
    pm = _core.ProfileModel(g, np_, conf.link)
    conf.do_uncoarsening = False
    coarse, levels, moves, cut0, cut1 = _core.ml_partition_stats(pm, conf)
    assert levels >= 2 and moves == 0 and cut0 == cut1 and 2 <= coarse.level() <= levels
    conf.do_uncoarsening = True
    fine, levels2, moves2, before, after = _core.ml_partition_stats(pm, conf)
    assert levels2 == levels and moves2 > 0 and after < before == cut0
    assert _core.ml_cut_bytes(g, fine) < _core.ml_cut_bytes(g, coarse)
    assert len(fine.nodes) == len(coarse.nodes)
    # still a partition of the operators ...
    ops = sorted(o for n in fine.nodes for o in n.sub_nodes)
    assert ops == sorted(n.id for n in g.nodes)
    # ... whose blocks, in the emitted order, only feed later blocks
    pos = {n.id: k for k, n in enumerate(fine.nodes)}
    assert all(pos[e.src_id] < pos[e.tgt_id] for e in fine.edges)
    sol, est, _ = _core.dp_staging(pm, fine, conf)
    owned = sorted(n.id for sg in sol.graphs for n in sg.nodes if n.is_batch)
    assert owned == sorted(n.id for n in g.nodes if n.is_batch)
    # hierarchy: one level down there are more, smaller nodes covering the same operators; lifting them back
    # up in pairs restores a coarser graph; the file format keeps the nesting
    low = _core.ml_to_lower_level(g, coarse)
    assert len(low.nodes) > len(coarse.nodes) and low.level() == coarse.level() - 1
    assert sorted(o for n in low.nodes for o in n.sub_nodes) == ops
    groups = [[i, i + 1] if i + 1 < len(low.nodes) else [i] for i in range(0, len(low.nodes), 2)]
    up = _core.ml_lift_up(g, low, groups)
    assert len(up.nodes) == len(groups) and up.level() == low.level() + 1
    back = _core.MLGraph.loads(coarse.dumps())
    assert back.level() == coarse.level() and [len(n.children) for n in back.nodes] == \
        [len(n.children) for n in coarse.nodes]
    raw = _core.msgpack_unpack(coarse.dumps())
    node0 = raw[0][0]                      # MLNode: id, graph, sub_nodes, sub_edges
    assert node0[0] == "ML_0" and isinstance(node0[2][0], list) and node0[2][0][0].startswith("ML_0_")


def test_coarsening_by_memory_and_checkpointing_no_last():
    g = make_mlp_graph(layers=16, hidden=256, batch=32, with_loss=False)
    # one operator is heavy in memory but cheap in time
    np_ = {n.id: _core.NodeProfile(100.0, 200.0, (64 << 20) if n.id == "lin8" else (1 << 20), 0, True)
           for n in g.nodes}
    conf = _conf(2, 32)
    conf.min_partition_num = 6
    pm = _core.ProfileModel(g, np_, conf.link)
    by_time = _core.ml_partition(pm, conf)
    conf.coarsen_by_time = False
    by_mem = _core.ml_partition(pm, conf)
    size_of = lambda ml: [len(n.sub_nodes) for n in ml.nodes if "lin8" in n.sub_nodes][0]  # noqa: E731
    # weighed by memory, the heavy operator's block stays small (it is the outlier nothing merges with)
    assert size_of(by_mem) < size_of(by_time)
    # checkpointing_no_last: with recomputation forced, the last stage is planned without it
    conf = _conf(2, 32)
    conf.cfg_partition_num, conf.cfg_pipeline_num, conf.checkpointing = 2, 2, True
    pm = _core.ProfileModel(g, np_, conf.link)
    ml = _core.ml_partition(pm, conf)
    _, est, _ = _core.dp_staging(pm, ml, conf)
    assert est[0].profile.checkpointing and est[1].profile.checkpointing
    conf.checkpointing_no_last = True
    _, est2, _ = _core.dp_staging(pm, ml, conf)
    assert est2[0].profile.checkpointing and not est2[1].profile.checkpointing
    assert est2[1].profile.bwd_time < est[1].profile.bwd_time


def test_measured_subgraph_profiles_replace_the_additive_estimate():
    """The profile model asks a callback to measure whole candidate subgraphs (time and allocator peak); what it
    returns is what the stage search plans with, each subgraph is measured once, and a callback that declines
    leaves the additive estimate in place."""
    g = make_mlp_graph(layers=8, hidden=64, batch=16, with_loss=False)
    np_ = _profiles(g)
    conf = _conf(2, 16)
    pm = _core.ProfileModel(g, np_, conf.link)
    calls = []

    def measure(ids, bs, ckpt):
        calls.append((tuple(ids), bs, ckpt))
        if len(ids) > 12:
            return None
        p = _core.GraphProfile()
        p.fwd_time, p.bwd_time = 7 * len(ids), 11 * len(ids)
        p.max_allocated_mem, p.activation_size, p.working_mem = 12345 * len(ids), 1000 * len(ids), 10
        return p

    pm.set_subgraph_measure(measure, 1000)
    ml = _core.ml_partition(pm, conf)
    sol, est, _ = _core.dp_staging(pm, ml, conf)
    assert calls and pm.measured_count() == len(set(calls)) == len(calls)
    for e in est:
        n_ops = sum(1 for n in sol.graphs[0].nodes if n.is_batch)
        if n_ops <= 12:
            assert e.profile.fwd_time == 7 * n_ops and e.profile.bwd_time == 11 * n_ops
            assert e.profile.activation_size == 1000 * n_ops
        else:
            assert e.profile.fwd_time > 7 * n_ops      # the additive estimate (100 us per operator)


def test_subgraph_profiler_measures_blocks_and_files_them_in_the_profile_db(tmp_path):
    """The measuring profiler cuts operator sets out of the traced graph, runs them forward + backward at a
    given micro-batch size (here on the host clock), calibrates the operator profiles block by block, and its
    measurements travel in the reference's ProfileDB layout together with the operator profiles."""
    import torch

    from rannc_b200.graph import planner, profiler, tracer
    from tests import zoo

    torch.manual_seed(0)
    m = zoo.build("deep")
    x = zoo.inputs("deep", 8, torch.Generator().manual_seed(1))
    tm = tracer.trace(m, x, use_kernels=False, name="t")
    sp = profiler.SubgraphProfiler(tm, torch.device("cpu"), iters=1)
    ids = [n.id for n in tm.ir.nodes if n.is_batch or n.is_criterion]
    gp = sp.measure(ids[:4], 4, False)
    assert gp.fwd_time > 0 and gp.bwd_time > 0 and gp.activation_size == 4 * 16 * 4 and not gp.checkpointing
    gp2 = sp.measure(ids, 8, True)
    assert gp2.checkpointing and gp2.bwd_time > gp2.fwd_time
    assert sp.measure(["no_such_operator"], 4, False) is None
    np_ = profiler.analytic_profiles(tm.gm)
    ir = _core.scale_graph(tm.ir, 8)
    n0 = sp.count
    plan = planner.plan(ir, np_, 2, 8, 0, False, False, False, "x", None, subgraph_profiler=sp)
    assert sp.count - n0 == plan.ml_nodes and len(sp.db) == plan.ml_nodes
    path = str(tmp_path / "profiles.bin")
    profiler.save_profiles(path, np_, tm.trace_batch, tm.ir, db=sp.db)
    back = profiler.load_profiles(path, [n.id for n in tm.ir.nodes], tm.trace_batch, tm.ir)
    assert set(back) == set(np_)
    db = _core.ProfileDB()
    db.loads(open(path, "rb").read())
    assert len(db) == plan.ml_nodes + 1
    raw = _core.msgpack_unpack(open(path, "rb").read())        # map: hash -> ProfileItem(key, profile)
    item = next(iter(raw.values()))
    assert len(item) == 2 and len(item[0]) == 5 and len(item[1]) == 2
    with pytest.raises(RuntimeError):
        profiler.load_profiles(path, ["other"], tm.trace_batch, tm.ir)


def test_subgraph_cut_replicates_non_batch_nodes():
    g = _core.IRGraph()
    g.batch_size = 4
    g.add_input(_core.IRValue("x", _t([4, 8])))
    g.add_input(_core.IRValue("w", _t([8, 8], rg=True), True))
    for name, dims in [("wt", [8, 8]), ("h", [4, 8]), ("o", [4, 8])]:
        g.add_value(_core.IRValue(name, _t(dims)))
    g.add_node(_core.IRNode("aten::t", ["w"], ["wt"], "t"))           # parameter-only computation
    g.add_node(_core.IRNode("aten::matmul", ["x", "wt"], ["h"], "m1"))
    g.add_node(_core.IRNode("aten::matmul", ["h", "wt"], ["o"], "m2"))
    g.add_output("o")
    g = _core.guess_value_types(g)
    assert not {n.id: n for n in g.nodes}["t"].is_batch
    parts = _core.create_subgraphs(g, [-1, 0, 1], 2, "P_")
    for p in parts:
        assert "t" in [n.id for n in p.nodes] and "w" in p.input_names  # copied into both parts
    assert parts[0].output_names == ["h"] and "h" in parts[1].input_names and parts[1].output_names == ["o"]
    merged = _core.merge_subgraphs(g, parts, 0, 1, "M")
    assert merged.output_names == ["o"] and [n.id for n in merged.nodes] == ["t", "m1", "m2"]


def test_deployment_file_roundtrip_and_routes():
    g = make_mlp_graph(layers=6, batch=8)
    conf = _conf(2, 8)
    conf.cfg_partition_num = 2
    pm = _core.ProfileModel(g, _profiles(g), conf.link)
    sol, _, _ = _core.dp_staging(pm, _core.ml_partition(pm, conf), conf)
    dep = _core.create_deployment(g, sol, 2, True, "dep1")
    assert _core.verify_deployment(dep) == ""
    data = _core.save_deployment(dep, 2, 12345)
    dep2, world, mem = _core.load_deployment(data)
    assert (world, mem) == (2, 12345) and dep2.fwd_graph_order == dep.fwd_graph_order
    assert dep2.allocation == dep.allocation and dep2.pipeline_num == dep.pipeline_num
    # DeploymentState = [deployment, world_size, dev_mem]; Deployment has 17 positional fields
    raw = _core.msgpack_unpack(data)
    assert len(raw) == 3 and len(raw[0]) == 17 and raw[0][0] == "dep1"
    # labels enter at the last stage from the caller, activations cross between the stages, the loss leaves
    assert {r.value_name for r in dep.fwd_in_routes} == {"x", "y"}
    assert len(dep.fwd_routes) == 1 and dep.fwd_routes[0].type == _core.RouteType.REDIST
    assert dep.fwd_out_routes[0].type == _core.RouteType.WEIGHTED_REDUCE
    assert len(dep.bwd_routes) == 1 and dep.bwd_in_routes[0].type == _core.RouteType.BROADCAST
    # a broken deployment is reported
    dep.fwd_routes = []
    assert "no forward route" in _core.verify_deployment(dep)


def test_allocation_strategies():
    order = ["a", "b"]
    flat = _core.search_allocation_flat(order, {"a": 2, "b": 2}, 4)
    assert flat == {"a": [0, 2], "b": [1, 3]}  # each pipeline replica on neighbouring devices
    simple = _core.search_allocation_simple(order, {"a": 1, "b": 3}, 4)
    assert simple == {"b": [0, 1, 2], "a": [3]}
    assert _core.tag_of_ranks([3, 1]) == _core.tag_of_ranks([1, 3, 3]) and _core.tag_of_ranks([0]) < 30000


def test_cost_model():
    link = _core.LinkModel()
    assert _core.calc_comm_time(link, 0) == 0
    assert abs(_core.calc_comm_time(link, 770_000_000) - (link.latency_us + 1000.0)) < 1e-6
    # bus-bandwidth convention: 2 (n-1)/n x bytes / busbw
    assert abs(_core.calc_allreduce_time(link, 725_000_000, 8) - (link.latency_us + 1750.0)) < 1e-6
    assert _core.calc_allreduce_time(link, 1 << 20, 1) == 0
    g = make_mlp_graph(layers=2, hidden=64, batch=8, with_loss=False)
    conf = _conf(1, 8)
    params = g.param_size_in_byte()
    assert _core.get_opt_mem_size(g, conf, 1) == params + 2 * params  # gradient + 2 x state
    conf.enable_zero = True
    assert _core.get_opt_mem_size(g, conf, 4) == params + 2 * params // 4


def test_profile_db_roundtrip():
    db = _core.ProfileDB()
    g = make_mlp_graph(layers=2)
    p = _core.GraphProfile()
    p.name, p.fwd_time, p.bwd_time, p.max_allocated_mem = "g", 11, 22, 33
    db.add({"g": g}, 8, 1, False, {"g": p})
    db2 = _core.ProfileDB()
    db2.loads(db.dumps())
    got = db2.get({"g": g}, 8, 1, False)
    assert got["g"].fwd_time == 11 and got["g"].bwd_time == 22
    assert db2.get({"g": g}, 4, 1, False) is None
    # GraphProfile has 14 positional fields, working_mem / activation_size before checkpointing
    raw = _core.msgpack_unpack(p.dumps())
    assert len(raw) == 14 and raw[0] == "g" and raw[1] == 11 and raw[4] == 22 and raw[13] is False


# ----------------------------------------------------------------------------- config / logging / trace
def test_config_defaults_env_and_toml(tmp_path, monkeypatch):
    monkeypatch.delenv("RANNC_CONF_DIR", raising=False)
    _core.config_reload()
    assert _core.config_get("max_pipeline") == 32 and _core.config_get("min_partition_num") == 5
    assert _core.config_get("decomposer") == "ml_part" and abs(_core.config_get("mem_margin") - 0.1) < 1e-9
    assert _core.config_get("deployment_file") == "/tmp/rannc_deployment.bin"
    assert _core.config_get("save_deployment") is False
    (tmp_path / "rannc_conf.toml").write_text('max_pipeline = 8  # comment\ndecomposer = "fair_weight"\nbogus = 1\n')
    monkeypatch.setenv("RANNC_CONF_DIR", str(tmp_path))
    monkeypatch.setenv("RANNC_MAX_PIPELINE", "4")  # the environment wins over the file
    _core.config_reload()
    assert _core.config_get("max_pipeline") == 4 and _core.config_get("decomposer") == "fair_weight"
    assert any("bogus" in w for w in _core.config_warnings())
    monkeypatch.delenv("RANNC_CONF_DIR")
    monkeypatch.delenv("RANNC_MAX_PIPELINE")
    _core.config_reload()
    assert len(_core.config_items()) >= 62
    with pytest.raises(RuntimeError):
        _core.config_get("no_such_item")


def test_event_trace_and_time_counter():
    _core.trace_clear()
    _core.trace_enable(True)
    _core.trace_begin(_core.func_key("forward", "g0", 1, False))
    _core.trace_end(_core.func_key("forward", "g0", 1, False))
    _core.trace_enable(False)
    _core.trace_begin("ignored")
    assert _core.trace_size() == 2
    doc = json.loads(_core.trace_merge([_core.trace_dump_local(0), _core.trace_dump_local(1)]))
    ev = doc["traceEvents"]
    assert len(ev) == 4 and {e["ph"] for e in ev} == {"B", "E"} and {e["pid"] for e in ev} == {0, 1}
    assert "graph=g0" in ev[0]["name"] and "split=1" in ev[0]["name"]
    _core.trace_clear()
    tc = _core.TimeCounter(True)
    tc.start("a")
    time.sleep(0.01)
    tc.stop("a")
    assert tc.count("a") == 1 and tc.total_us("a") >= 9000 and "a:" in tc.summary()


def test_watchdog_detects_missing_peer(tmp_path):
    """Failure detection on the host: the peer's heartbeat file disappears; no GPU is involved."""
    d = str(tmp_path)
    failed = []
    peer = _core.Watchdog()
    peer.start(d, 1, 2, 0.05, 5.0, None)
    wd = _core.Watchdog()
    wd.start(d, 0, 2, 0.05, 5.0, lambda r: failed.append(r))
    time.sleep(0.3)
    assert wd.running() and not failed and os.path.exists(_core.Watchdog.lock_path(d, 1))
    peer.stop(True)  # a failing rank removes its own file so that the others notice
    deadline = time.time() + 5
    while not failed and time.time() < deadline:
        time.sleep(0.05)
    assert failed == [1] and wd.failed_peer() == 1 and not wd.running()
    wd.stop(True)


def test_reference_package_name_is_an_alias():
    import pyrannc
    import pyrannc.amp  # noqa: F401
    from pyrannc.opt import patch_optimizer  # noqa: F401

    import rannc_b200

    assert pyrannc.RaNNCModule is rannc_b200.RaNNCModule
    assert pyrannc.dist_param is rannc_b200.dist_param
    assert pyrannc.get_world_size() >= 1


def test_tutorial_script_runs_on_cpu(tmp_path):
    """BASELINE config 1: the tutorial MLP through trace, profile, plan and a few training steps, world size 1."""
    import os
    import subprocess
    import sys

    import torch

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "ckpt.pt"
    env = dict(os.environ, RANNC_FORCE_CPU="1", RANK="0", WORLD_SIZE="1", RANNC_LOG_LEVEL="warning")
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "tutorial.py"), "--steps", "4", "--save",
                        str(out)], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("step ")]
    assert len(lines) == 4
    first, last = float(lines[0].split()[-1]), float(lines[-1].split()[-1])
    assert last < first
    ck = torch.load(out, weights_only=False)
    assert set(ck["model"].keys()) == {"net.fc1.weight", "net.fc1.bias", "net.fc2.weight", "net.fc2.bias",
                                       "net.fc3.weight", "net.fc3.bias"}
    assert len(ck["optimizer"]["state"]) == 6


def test_dry_run_plans_a_large_model_from_meta_tensors():
    """partitioning_dry_run_np: plan for 8 devices of 180 GB in one CPU process; the model exists only as
    meta tensors, so nothing of its size is allocated (reference: RaNNCModule.cpp:416-421, run_dp_dry)."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r'''
import os, sys
sys.path.insert(0, os.getcwd())
import torch
import rannc_b200 as pyrannc
from rannc_b200.models.bert import BertConfig, BertForPreTraining, synthetic_batch
cfg = BertConfig(hidden_size=2048, num_hidden_layers=24, num_attention_heads=32, intermediate_size=8192)
with torch.device("meta"):
    model = BertForPreTraining(cfg)
opt = torch.optim.Adam(model.parameters(), lr=1e-4)
m = pyrannc.RaNNCModule(model, opt, enable_apex_amp=True, enable_zero=True, check_unused_values=False)
batch = tuple(t.to("meta") for t in synthetic_batch(cfg, 256, 512, seed=0))
try:
    m(*batch)
except SystemExit:
    print("PLANNED")
'''
    env = dict(os.environ, RANNC_FORCE_CPU="1", RANK="0", WORLD_SIZE="1", RANNC_LOG_LEVEL="info",
               RANNC_PARTITIONING_DRY_RUN_NP="8")
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=900)
    out = r.stdout + r.stderr
    assert "PLANNED" in out, out[-3000:]
    assert "Assigned subgraph" in out and "repl=" in out


def test_conv_bn_rewrite_keeps_the_function_on_cpu():
    """The convolution / batch-norm fusion pass (with the batch-norm counters anchored after it) leaves the
    traced ResNet numerically identical; on the CPU the fused operators fall back to ATen."""
    import torch

    from rannc_b200.graph import rewrite, tracer
    from rannc_b200.models.resnet import tiny_resnet

    torch.manual_seed(0)
    m = tiny_resnet().train()
    ref = tiny_resnet().train()
    ref.load_state_dict(m.state_dict())
    x = torch.randn(4, 3, 64, 64)
    ep, _ = tracer.export_model(m, (x,))
    gm = ep.graph_module
    stats = rewrite.fuse(gm, training=True)
    assert stats["conv2d"] == 17 and stats["batch_norm_act"] == 17
    targets = [getattr(n.target, "__name__", str(n.target)) for n in gm.graph.nodes if n.op == "call_function"]
    assert not any("relu" in t for t in targets)          # every ReLU went into a fused batch norm
    assert targets.count("after_effects") == 17           # one anchored counter update per batch norm
    state = dict(m.named_parameters())
    state.update(dict(m.named_buffers()))
    vals = [state[s.target].detach().clone() if s.kind.name in ("PARAMETER", "BUFFER") else x
            for s in ep.graph_signature.input_specs]
    out = gm(*vals)
    out = out[0] if isinstance(out, (tuple, list)) else out
    assert torch.allclose(out, ref(x), atol=1e-5)


def test_smaller_last_batch_is_padded_and_trimmed():
    import torch

    import rannc_b200 as pyrannc
    from rannc_b200.models.mlp import TutorialMLP

    torch.manual_seed(0)
    net = TutorialMLP(d_in=32, hidden=64, classes=8)
    ref = TutorialMLP(d_in=32, hidden=64, classes=8)
    ref.load_state_dict(net.state_dict())
    model = pyrannc.RaNNCModule(net, torch.optim.SGD(net.parameters(), lr=0.1))
    x = torch.randn(8, 32)
    assert torch.allclose(model(x), ref(x), atol=1e-5)
    out = model(x[:5])                       # the last, smaller batch of an epoch
    assert out.shape == (5, 8)
    assert torch.allclose(out, ref(x[:5]), atol=1e-5)
    out.sum().backward()
    import pytest
    with pytest.raises(RuntimeError):
        model(torch.randn(9, 32))
    pyrannc.clear()


def test_checkpoint_reload_into_a_fresh_module():
    """state_dict() and the global optimizer state go into a newly wrapped copy of the model, which then
    continues exactly like the original (reference: test/common.py:254-310)."""
    import copy

    import torch

    import rannc_b200 as pyrannc
    from rannc_b200.models.mlp import TutorialMLPWithLoss

    torch.manual_seed(0)
    x, y = torch.randn(16, 512), torch.randint(0, 10, (16,))

    def train(model, opt, steps):
        out = []
        for _ in range(steps):
            loss = model(x, y)
            loss.backward()
            opt.step()
            opt.zero_grad()
            out.append(float(loss))
        return out

    net = TutorialMLPWithLoss()
    fresh = copy.deepcopy(net)
    opt = torch.optim.Adam(net.parameters(), lr=1e-2)
    m1 = pyrannc.RaNNCModule(net, opt)
    train(m1, opt, 3)
    sd, osd = m1.state_dict(), opt.state_dict(from_global=True)
    after = train(m1, opt, 2)

    opt2 = torch.optim.Adam(fresh.parameters(), lr=1e-2)
    m2 = pyrannc.RaNNCModule(fresh, opt2)
    m2.load_state_dict(sd)                       # before the first call
    loss = m2(x, y)                              # deploys
    opt2.load_state_dict(osd, from_global=True)
    loss.backward()
    opt2.step()
    opt2.zero_grad()
    assert abs(float(loss) - after[0]) < 1e-5
    assert abs(float(m2(x, y)) - after[1]) < 1e-4
    pyrannc.clear()


def test_gradients_of_model_inputs_reach_the_caller():
    import torch

    import rannc_b200 as pyrannc
    from rannc_b200.models.mlp import TutorialMLP

    torch.manual_seed(0)
    net = TutorialMLP(d_in=32, hidden=64, classes=8)
    ref = TutorialMLP(d_in=32, hidden=64, classes=8)
    ref.load_state_dict(net.state_dict())
    model = pyrannc.RaNNCModule(net, torch.optim.SGD(net.parameters(), lr=0.1))
    x = torch.randn(8, 32, requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    go = torch.randn(8, 8)
    model(x).backward(go)
    ref(xr).backward(go)
    assert x.grad is not None and torch.allclose(x.grad, xr.grad, atol=1e-5)
    pyrannc.clear()


def test_operator_profiles_round_trip_and_debug_switches(tmp_path):
    """save / load of operator profiles and of the stage assignment, display_act_value, profiling and
    sync_allreduce on one rank."""
    import subprocess
    import sys

    prof = tmp_path / "profiles.bin"
    code = (
        "import torch, rannc_b200 as pyrannc\n"
        "from tests import zoo\n"
        "torch.manual_seed(0)\n"
        "m = zoo.build('deep'); o = torch.optim.SGD(m.parameters(), lr=0.1)\n"
        "w = pyrannc.RaNNCModule(m, o)\n"
        "out = w(torch.randn(8, 16)); out.sum().backward(); o.step()\n"
        "print('OUT', float(out.sum()))\n"
        "pyrannc.clear()\n")
    base = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", RANNC_FORCE_CPU="1",
                RANNC_GRAPH_PROFILE_FILE=str(prof), RANNC_LOG_LEVEL="info",
                RANNC_ALLOC_SOLUTIONS_FILE_PREFIX=str(tmp_path / "sols"))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(extra, port):
        r = subprocess.run([sys.executable, "-c", code], env=dict(base, MASTER_PORT=str(port), **extra), cwd=root,
                           capture_output=True, text=True, timeout=240)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        return r.stdout + r.stderr

    first = run({"RANNC_SAVE_GRAPH_PROFILE": "true", "RANNC_DISPLAY_ACT_VALUE": "true", "RANNC_PROFILING": "true",
                 "RANNC_SYNC_ALLREDUCE": "true", "RANNC_SAVE_ALLOC_SOLUTIONS": "true"}, 29731)
    assert (tmp_path / "sols_s1_p1.bin").exists()
    assert prof.exists() and "Saved operator profiles" in first
    assert "absmean=" in first and "time per stage" in first
    # the reference's ProfileDB layout: {hash: [key, result]}; key = [ir_graphs, batch_size, repl_nums,
    # iteration, checkpointing], result = [node_profiles, value_types]
    raw = _core.msgpack_unpack(prof.read_bytes())
    (key, result), = raw.values()
    assert key[1] == 8 and len(result[0]) >= 16
    second = run({"RANNC_LOAD_GRAPH_PROFILE": "true", "RANNC_LOAD_ALLOC_SOLUTIONS": "true"}, 29732)
    assert "Loaded operator profiles" in second and "Loaded the stage assignment" in second
    out = lambda t: [l for l in t.splitlines() if l.startswith("OUT")]
    assert out(first) == out(second)
    # a file taken for another graph is refused
    h, = raw.keys()
    result[0].pop(next(iter(result[0])))
    prof.write_bytes(_core.msgpack_pack({h: [key, result]}))
    r = subprocess.run([sys.executable, "-c", code], env=dict(base, MASTER_PORT="29733", RANNC_LOAD_GRAPH_PROFILE="true"),
                       cwd=root, capture_output=True, text=True, timeout=240)
    assert r.returncode != 0 and "does not match the traced graph" in r.stdout + r.stderr


def test_keyword_arguments_are_bound_by_the_forward_signature():
    import subprocess
    import sys

    code = (
        "import torch, torch.nn as nn, rannc_b200 as pyrannc\n"
        "class M(nn.Module):\n"
        "    def __init__(self):\n"
        "        super().__init__(); self.l = nn.Linear(16, 16)\n"
        "    def forward(self, x, scale=None, shift=None):\n"
        "        h = self.l(x)\n"
        "        if scale is not None: h = h * scale\n"
        "        if shift is not None: h = h + shift\n"
        "        return h\n"
        "torch.manual_seed(0)\n"
        "m = M(); ref = M(); ref.load_state_dict(m.state_dict())\n"
        "w = pyrannc.RaNNCModule(m, torch.optim.SGD(m.parameters(), lr=0.1))\n"
        "x, sh = torch.randn(8, 16), torch.randn(8, 16)\n"
        "out = w(x, shift=sh)\n"
        "assert torch.allclose(out, ref(x, shift=sh), atol=1e-5), 'mismatch'\n"
        "out2 = w(x, shift=sh * 2)\n"
        "assert torch.allclose(out2, ref(x, shift=sh * 2), atol=1e-5), 'mismatch 2'\n"
        "try:\n"
        "    w(x, nonsense=1)\n"
        "    raise SystemExit('no error for an unknown keyword')\n"
        "except RuntimeError as e:\n"
        "    assert 'do not fit' in str(e)\n"
        "print('KW OK'); pyrannc.clear()\n")
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29741",
               RANNC_FORCE_CPU="1", RANNC_LOG_LEVEL="warning")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0 and "KW OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


# ----------------------------------------------------------------------------- byte-level goldens
def test_serialised_bytes_match_an_independent_msgpack_encoder():
    """The files this library writes are meant to be readable by the reference's loaders, whose classes are
    serialised positionally by msgpack-c (src/graph/ir.h:225-227,381,458-459,603-604;
    src/comp/GraphProfiler.h:54-57).  The positional structures below are written out by hand from those field
    lists and encoded with the ``msgpack`` Python package; the native encoder must produce the same bytes, and
    bytes frozen in this file must still load."""
    import msgpack

    SIZE_MAX = 2 ** 64 - 1
    g = _core.IRGraph()
    g.name, g.batch_size = "g", 4
    g.add_input(_core.IRValue("x", _t([4, 3])))
    g.add_value(_core.IRValue("y", _t([4, 3], _core.IRTensorElemType.HALF, True)))
    g.add_node(_core.IRNode("aten::relu", ["x"], ["y"], "relu_1"))
    g.add_output("y")

    def ir_type(elem, dims, rg):
        # base_type (TENSOR = 1), scalar_type (NONE = 0), tensor_dim, tensor_elem_type, requires_grad,
        # list_type (not meaningful for a tensor; this library writes GENERIC = 4), compound_types, list_size,
        # func_name
        return [1, 0, dims, elem, rg, 4, [], SIZE_MAX, ""]

    def ir_value(name, ty):
        return [name, ty, False, False, False, 0]      # name, type, is_param, is_batch, is_loss, batch_size

    want = ["g",
            [["aten::relu", ["x"], ["y"], "relu_1", False, False, 0]],   # name, inputs, outputs, id, flags, batch
            {"x": ir_value("x", ir_type(3, [4, 3], False)), "y": ir_value("y", ir_type(4, [4, 3], True))},
            ["x"], ["y"], True, 4]
    assert g.dumps() == msgpack.packb(want)
    frozen = bytes.fromhex(
        "97a1679197aa6174656e3a3a72656c7591a17891a179a672656c755f31c2c20082a17896a17899010092040303c20490cfffff"
        "ffffffffffffa0c2c2c200a17996a17999010092040304c30490cfffffffffffffffffa0c2c2c20091a17891a179c304")
    assert g.dumps() == frozen
    g2 = _core.IRGraph.loads(frozen)
    assert str(g2) == str(g) and g2.dumps() == frozen
    assert g2.values["y"].type.requires_grad and g2.values["y"].type.tensor_dim == [4, 3]

    p = _core.GraphProfile()
    p.name, p.fwd_time, p.bwd_time, p.max_allocated_mem = "g", 11, 22, 33
    # name, fwd_time, fwd_cpu_time, fwd_cuda_time, bwd_time, bwd_cpu_time, bwd_cuda_time, max_allocated_mem,
    # param_size, input_size, output_size, working_mem, activation_size, checkpointing
    assert p.dumps() == msgpack.packb(["g", 11, 0, 0, 22, 0, 0, 33, 0, 0, 0, 0, 0, False])
    assert p.dumps() == bytes.fromhex("9ea1670b0000160000210000000000c2")


def test_dimension_names_follow_the_batch_through_the_trace(monkeypatch):
    """``use_named_tensors``: the batch dimension is named "N" wherever it ends up, other dimensions after the
    value (reference: src/comp/GraphProfiler.cpp:149-170)."""
    import torch

    from rannc_b200.graph import tracer

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(8, 4)

        def forward(self, x):
            return self.lin(x).transpose(0, 1).sum(1)

    monkeypatch.setenv("RANNC_USE_NAMED_TENSORS", "true")
    _core.config_reload()
    try:
        tm = tracer.trace(M(), (torch.randn(4, 8),), use_kernels=False, name="m")
    finally:
        monkeypatch.delenv("RANNC_USE_NAMED_TENSORS")
        _core.config_reload()
    assert tm.dim_names["x"] == ["N", "x_D1"]
    assert tm.dim_names["linear"] == ["N", "linear_D1"]
    assert tm.dim_names["transpose"] == ["transpose_D0", "N"]
    assert "N" not in tm.dim_names["sum_1"] and "N" not in tm.dim_names["p_lin_weight"]
    tm2 = tracer.trace(M(), (torch.randn(4, 8),), use_kernels=False, name="m")
    assert tm2.dim_names == {}


def test_single_stage_plan_with_interleaved_backward_needs_one_micro_batch_of_memory():
    """interleave_single_stage: the stage search counts ONE micro-batch's activations for a one-stage plan, so a
    model that the synchronous schedule can only fit with recomputation runs without it in several micro-batches."""
    g = make_mlp_graph(layers=8, hidden=256, batch=64, with_loss=True)
    act = 64 * 256 * 4 * 40                                  # activations per operator at the full batch
    np_ = _profiles(g, act=act)
    total_act = act * len(g.nodes)
    conf = _conf(1, 64, int(total_act * 0.4) + g.param_size_in_byte() * 4)
    pm = _core.ProfileModel(g, np_, conf.link)
    ml = _core.ml_partition(pm, conf)
    sol, est, _ = _core.dp_staging(pm, ml, conf)
    assert sol.checkpointing or len(sol.graphs) > 1, \
        "the synchronous schedule should not fit this model without recomputation"
    conf.interleave_single_stage = True
    sol2, est2, _ = _core.dp_staging(pm, _core.ml_partition(pm, conf), conf)
    assert len(sol2.graphs) == 1 and not sol2.checkpointing and sol2.pipeline_num >= 4


def test_bench_reference_arm_reports_unavailable_and_cpu_run_is_refused():
    """bench.py: the reference arm prints one JSON line saying why the reference cannot run here and exits 0; the
    library's own arm refuses to produce a number without a CUDA device."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps",
                        "2", "--warmup", "3"], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and len(line["unavailable"]) > 10
    env = dict(os.environ, RANNC_FORCE_CPU="1", RANK="0", WORLD_SIZE="1", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--no-baseline", "--layers", "1", "--hidden", "64",
                        "--heads", "2", "--seq", "16", "--global-batch", "4"], cwd=root, env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 2 and "CUDA" in r.stderr

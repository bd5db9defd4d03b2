"""Pieces of the parameter streamer that need no process group: run grouping and segment cutting."""
import torch
import torch.fx as fx

from rannc_b200.parallel.param_storage import FlatGroup
from rannc_b200.parallel.param_stream import _runs, split_into_segments


def _streamed_group(shapes):
    import rannc_b200.parallel.comm as comm

    g = FlatGroup((0,), torch.bfloat16, torch.device("cpu"))
    params = [torch.nn.Parameter(torch.randn(*s).bfloat16()) for s in shapes]
    for i, p in enumerate(params):
        g.add(f"p{i}", p, 0)
    orig = comm.get_rank
    comm.get_rank = lambda: 0
    try:
        g.finalize(True, False, streamed=True)
    finally:
        comm.get_rank = orig
    return g, params


def test_streamed_parameters_leave_no_device_copy_and_group_into_runs():
    g, ps = _streamed_group([(8, 16), (8, 16), (8, 16), (3,), (64, 64)])
    assert g.streamed and all(p.data.numel() == 0 and p._rannc_shape for p in ps)
    assert all(torch.equal(p._rannc_host.view(-1), g.flat_param[o:o + n]) for p, o, n in
               zip(ps, g.offsets, g.numels))
    # neighbours in the flat layout form one run (one allocation, one copy); a gap starts a new one
    runs = _runs(ps)
    assert len(runs) == 1 and runs[0][1] == 0 and runs[0][2] == g.offsets[-1] + g.numels[-1]
    runs = _runs([ps[0], ps[1], ps[4]])
    assert [(lo, hi) for _, lo, hi, _ in runs] == [(0, 256), (g.offsets[4], g.offsets[4] + 4096)]
    assert [len(items) for _, _, _, items in runs] == [2, 1]


def test_stage_graph_is_cut_by_parameter_bytes_with_values_handed_across():
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(64, 64)
            self.b = torch.nn.Linear(64, 64)
            self.c = torch.nn.Linear(64, 64)

        def forward(self, x):
            h = torch.relu(self.a(x))
            return self.c(torch.relu(self.b(h)) + h)        # h crosses the second cut as well

    m = M()
    gm = fx.symbolic_trace(m)
    # stage graphs take their parameters as placeholders: rebuild the trace in that form
    g2 = fx.Graph()
    env, params = {}, {}
    for n in gm.graph.nodes:
        if n.op == "placeholder":
            env[n.name] = g2.placeholder(n.name)
    for name, p in m.named_parameters():
        ph = g2.placeholder(name.replace(".", "_"))
        env[name] = ph
        params[ph.name] = p
    x = env["x"]
    h = g2.call_function(torch.relu, (g2.call_function(torch.nn.functional.linear, (x, env["a.weight"], env["a.bias"])),))
    t = g2.call_function(torch.relu, (g2.call_function(torch.nn.functional.linear, (h, env["b.weight"], env["b.bias"])),))
    s = g2.call_function(torch.add, (t, h))
    out = g2.call_function(torch.nn.functional.linear, (s, env["c.weight"], env["c.bias"]))
    g2.output((out,))
    stage = fx.GraphModule(m, g2)
    one_layer = 64 * 64 * 4 + 64 * 4
    segs = split_into_segments(stage, params, one_layer, resident=True)
    assert len(segs) == 3
    assert [sorted(k for k in sg.params) for sg in segs] == [["a_bias", "a_weight"], ["b_bias", "b_weight"],
                                                             ["c_bias", "c_weight"]]
    # chained execution reproduces the module
    xin = torch.randn(5, 64)
    vals = {"x": xin}
    for sg in segs:
        outs = sg.gm(*[sg.params[nm] if nm in sg.params else vals[nm] for nm in sg.inputs])
        vals.update(zip(sg.outputs, outs))
    assert torch.allclose(vals[segs[-1].outputs[-1]], m(xin), atol=1e-6)
    assert h.name in segs[0].outputs and h.name in segs[1].inputs and h.name in segs[1].inputs

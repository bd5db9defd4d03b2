"""Parameters streamed from pinned host memory through a device window (offload_param_window_mb), on the kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _train(window_mb: int, micro_batches: int, segments: int = 0, checkpointing: bool = False):
    import rannc_b200 as pyrannc
    from rannc_b200.models.bert import BertConfig, BertForPreTraining, synthetic_batch
    from rannc_b200.ops import functional as RF
    from rannc_b200.utils.config import set_conf

    set_conf("offload_param_window_mb", window_mb)
    set_conf("pipeline_num", micro_batches)
    set_conf("checkpoint_segments", segments)
    set_conf("checkpointing", checkpointing)
    try:
        torch.manual_seed(0)
        RF.manual_seed(7)
        cfg = BertConfig.tiny(num_hidden_layers=4)
        model = BertForPreTraining(cfg)
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
        wrapped = pyrannc.RaNNCModule(model, opt, enable_apex_amp=True, offload_params=window_mb > 0)
        losses = []
        for it in range(3):
            batch = tuple(t.cuda() for t in synthetic_batch(cfg, 8, 128, seed=it))
            loss = wrapped(*batch)
            loss.backward()
            opt.step()
            opt.zero_grad()
            losses.append(float(loss.detach()))
        torch.cuda.synchronize()
        sd = {k: v.float().cpu() for k, v in wrapped.state_dict().items()}
        return losses, sd, wrapped
    finally:
        set_conf("offload_param_window_mb", 0)
        set_conf("pipeline_num", 0)
        set_conf("checkpoint_segments", 0)
        set_conf("checkpointing", False)


@pytest.mark.parametrize("micro_batches", [0, 2])
def test_streamed_parameters_match_resident_ones(micro_batches):
    from rannc_b200.ops import _lib

    la, sda, _ = _train(0, micro_batches)
    lb, sdb, w = _train(4, micro_batches)
    st = w._storage.streamer
    stages = list(w._stages.values())
    assert sum(len(s.segments) for s in stages) >= 3
    assert st.resident == 0 and st.peak_resident <= (4 << 20)
    for g in w._storage.groups:
        if g.streamed:
            assert not g.flat_param.is_cuda and not g.flat_grad.is_cuda and g.flat_param.is_pinned()
            assert all(p.data.numel() == 0 for p in g.params)
    # same dropout masks (the recomputation replays the counters); the runs differ in summation order only
    for x, y in zip(la, lb):
        assert abs(x - y) < 5e-3 * max(1.0, abs(x)), (la, lb)
    worst = max(float((sda[k] - sdb[k]).abs().max()) for k in sda)
    assert worst < 2e-2, worst
    assert _lib.read_error() == 0


def test_recomputation_segment_by_segment_matches_stage_recomputation():
    """checkpoint_segments: same dropout masks and gradients as recomputing the whole stage, with the activations
    of one segment instead of one stage alive in backward."""
    from rannc_b200.ops import _lib

    la, sda, wa = _train(0, 2, segments=0, checkpointing=True)
    lb, sdb, wb = _train(0, 2, segments=4, checkpointing=True)
    assert wa.is_checkpointing_enabled() and wb.is_checkpointing_enabled()
    stages = list(wb._stages.values())
    assert sum(len(s.segments) for s in stages) >= 3
    for x, y in zip(la, lb):
        assert abs(x - y) < 5e-3 * max(1.0, abs(x)), (la, lb)
    worst = max(float((sda[k] - sdb[k]).abs().max()) for k in sda)
    assert worst < 2e-2, worst
    assert _lib.read_error() == 0

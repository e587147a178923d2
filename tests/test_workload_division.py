"""Tile-row balancer: cuts, border snapping, per-camera strategies, heuristic feedback (CPU only)."""
from types import SimpleNamespace

import pytest
import torch

from cgx import workload_division as WD


def cams(n):
    return [SimpleNamespace(uid=100 + i) for i in range(n)]


def ctx(ws, rank=0, H=1200, W=1600, bsz=8, **kw):
    return WD.DivisionContext(image_height=H, image_width=W, rank=rank, world_size=ws, bsz=bsz, device="cpu", **kw)


def test_division_pos_heuristic_uniform_and_skewed():
    h = torch.ones(12)
    assert WD.division_pos_heuristic(h, 12, 3, right=True) == [0, 4, 8, 12]
    assert WD.division_pos_heuristic(h, 12, 3, right=False) == [0, 3, 7, 12]
    h = torch.tensor([10.0, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1])
    pos = WD.division_pos_heuristic(h, 11, 2, right=True)
    assert pos == [0, 1, 11]                    # the first row alone is half of the work
    with pytest.raises(AssertionError):
        WD.division_pos_heuristic(torch.ones(5), 6, 2)


def test_cfg2_every_gpu_gets_exactly_one_camera():
    c = ctx(8)
    hist = WD.DivisionStrategyHistoryFinal(cams(8), 8, 0, ctx=c)
    strategies, tasks = WD.start_strategy_final(cams(8), hist, ctx=c)
    assert c.tile_y == 75 and c.tile_x == 100
    for k, s in enumerate(strategies):
        assert s.gpu_ids == [k] and s.division_pos == [0, 75] and s.world_size == 1
    assert tasks == [[(k, 0, 75)] for k in range(8)]
    assert strategies[0].rank == 0 and strategies[1].rank == -1
    loc = strategies[0].get_compute_locally()
    assert loc.shape == (75, 100) and bool(loc.all())
    assert strategies[1].get_compute_locally() is None


def test_split_inside_a_camera_and_tile_bounds():
    c = ctx(3, rank=1, bsz=2)
    cs = cams(2)
    hist = WD.DivisionStrategyHistoryFinal(cs, 3, 1, ctx=c)
    strategies, tasks = WD.start_strategy_final(cs, hist, ctx=c)
    # 150 rows over 3 GPUs: cuts at 50 and 100
    assert strategies[0].gpu_ids == [0, 1] and strategies[0].division_pos == [0, 50, 75]
    assert strategies[1].gpu_ids == [1, 2] and strategies[1].division_pos == [0, 25, 75]
    assert tasks[1] == [(0, 50, 75), (1, 0, 25)]
    assert strategies[0].rank == 1 and strategies[1].rank == 0
    assert strategies[0].tile_bounds().tolist() == [0, 5000, 7500]
    loc = strategies[0].get_compute_locally()
    assert not loc[:50].any() and loc[50:].all()
    assert strategies[0].get_extended_compute_locally() is None


def test_cuts_near_an_image_border_snap_to_it():
    c = ctx(2, bsz=2, border_divpos_coeff=3.0)
    cs = cams(2)
    hist = WD.DivisionStrategyHistoryFinal(cs, 2, 0, ctx=c)
    hist.accum_heuristic[cs[0].uid] = torch.ones(75) * 1.04      # balanced cut would fall at row 73 of camera 0
    strategies, tasks = WD.start_strategy_final(cs, hist, ctx=c)
    assert strategies[0].gpu_ids == [0] and strategies[1].gpu_ids == [1]
    hist.accum_heuristic[cs[0].uid] = torch.ones(75) * 0.96      # ... at row 1 of camera 1 -> snaps back
    strategies, tasks = WD.start_strategy_final(cs, hist, ctx=c)
    assert strategies[0].gpu_ids == [0] and strategies[1].gpu_ids == [1]


def test_finish_updates_heuristics_only_when_the_reference_would(monkeypatch):
    cs = cams(1)
    # small image with bsz >= ws: the reference never updates the heuristics there
    c = ctx(2, H=1080, W=1920, bsz=2)
    hist = WD.DivisionStrategyHistoryFinal(cs, 2, 0, ctx=c)
    s, _ = WD.start_strategy_final(cs, hist, ctx=c)
    before = hist.accum_heuristic[cs[0].uid].clone()
    stats = [{"forward_render_time": 1.0, "backward_render_time": 2.0, "forward_loss_time": 0.5}]
    seen = {}

    def fake_gather(values, ctx):
        seen["local"] = list(values)
        return [list(values), [7.0]]

    monkeypatch.setattr(WD, "allgather_float_list", fake_gather)
    WD.finish_strategy_final(cs, hist, s, stats, ctx=c)
    assert seen["local"] == [4.0]                       # fwd + bwd + 2 * loss time
    assert torch.equal(hist.accum_heuristic[cs[0].uid], before)
    assert hist.history[-1]["all_camera_running_time"] == [11.0]
    assert hist.history[-1]["all_gpu_running_time"] == [4.0, 7.0]


def test_heuristic_feedback_moves_the_cut(monkeypatch):
    cs = cams(1)
    c = ctx(2, rank=0, H=2160, W=3840, bsz=1)
    hist = WD.DivisionStrategyHistoryFinal(cs, 2, 0, ctx=c)
    s, _ = WD.start_strategy_final(cs, hist, ctx=c)
    assert s[0].division_pos == [0, 68, 135] or s[0].division_pos == [0, 67, 135]
    # pretend GPU 0 needed 3x the time of GPU 1
    monkeypatch.setattr(WD, "allgather_float_list", lambda values, ctx: [[3.0], [1.0]])
    stats = [{"forward_render_time": 1.0, "backward_render_time": 2.0, "forward_loss_time": 0.0}]
    WD.finish_strategy_final(cs, hist, s, stats, ctx=c)
    h = hist.accum_heuristic[cs[0].uid]
    cut = s[0].division_pos[1]
    assert torch.allclose(h[:cut], torch.full((cut,), 3.0 / cut))
    assert torch.allclose(h[cut:], torch.full((135 - cut,), 1.0 / (135 - cut)))
    s2, _ = WD.start_strategy_final(cs, hist, ctx=c)
    assert s2[0].division_pos[1] < cut                      # the slow GPU gets fewer rows next time
    # decay blends old and new
    c.heuristic_decay = 0.5
    WD.finish_strategy_final(cs, hist, s, stats, ctx=c)
    assert torch.allclose(hist.accum_heuristic[cs[0].uid], h)   # same measurement -> same value after blending


def test_strategy_validation():
    c = ctx(2)
    with pytest.raises(AssertionError):
        WD.DivisionStrategyFinal(cams(1)[0], 2, [0, 1], [0, 40, 74], [(0, 40), (40, 74)], ctx=c)   # must end at TILE_Y
    with pytest.raises(AssertionError):
        WD.DivisionStrategyFinal(cams(1)[0], 2, [0], [0, 40, 75], [(0, 40), (40, 75)], ctx=c)


def test_distribution_config_table():
    from cgx.distribution_config import init_image_distribution_config

    a = SimpleNamespace(image_distribution_mode="3")
    cfg = init_image_distribution_config(a)
    assert cfg.avoid_pixels_all2all and cfg.workloads_division_mode == "DivisionStrategyDynamicAdjustment"
    assert len(cfg.local_running_time_mode) == 4
    with pytest.raises(ValueError):
        init_image_distribution_config(SimpleNamespace(image_distribution_mode="final"))


def test_balancer_follows_the_reference_step_by_step():
    """tests/golden/division_golden.json holds what the reference's own start_strategy_final / finish_strategy_final
    did over a few steps of four scenarios (cuts moving with measured times, decay, images too small to update,
    local sampling), made by tests/golden/make_division_golden.py.  The same time tables through this module must
    give the same ranks, cuts and task lists at every step, the same log, and the same heuristics to float rounding."""
    import json
    from pathlib import Path
    from types import SimpleNamespace as NS

    golden = json.loads((Path(__file__).resolve().parent / "golden" / "division_golden.json").read_text())
    assert len(golden) == 4
    moved = False
    for g in golden:
        sc = g["scenario"]
        ctx = WD.DivisionContext(image_height=sc["H"], image_width=sc["W"], rank=0, world_size=sc["ws"],
                                 bsz=sc["bsz"], local_sampling=sc["local_sampling"],
                                 border_divpos_coeff=sc["border"], heuristic_decay=sc["decay"],
                                 adjust_strategy_warmp_iterations=sc["warm"])
        cams = [NS(uid=100 + k) for k in range(sc["n_cams"])]
        history = WD.DivisionStrategyHistoryFinal(cams, sc["ws"], 0, ctx=ctx)
        for step in g["steps"]:
            ctx.iteration = step["iteration"]
            strategies, tasks = WD.start_strategy_final(cams, history, ctx=ctx)
            assert [list(s.gpu_ids) for s in strategies] == step["gpu_ids"], (sc["name"], step["iteration"])
            assert [list(map(int, s.division_pos)) for s in strategies] == step["division_pos"], (sc["name"], step["iteration"])
            assert [[list(map(int, t)) for t in ts] for ts in tasks] == step["tasks"]
            WD.finish_strategy_final(cams, history, strategies, None, ctx=ctx, gathered_times=step["table"])
            for cam, want in zip(cams, step["heuristic"]):
                got = history.accum_heuristic[cam.uid]
                assert torch.allclose(got, torch.tensor(want), rtol=1e-6, atol=1e-9), (sc["name"], step["iteration"])
            assert history.history[-1]["all_gpu_running_time"] == pytest.approx(step["log"], rel=1e-12)
            assert history.history[-1]["iteration"] == step["iteration"]
        if g["steps"][0]["division_pos"] != g["steps"][-1]["division_pos"]:
            moved = True
    assert moved, "no scenario of the golden file ever moved a cut"

"""Generate golden vectors for the tile-row balancer by running the reference's OWN functions
(gaussian_renderer/workload_division.py: division_pos_heuristic :75-94, DivisionStrategyFinal :684-778,
DivisionStrategyHistoryFinal :781-824, start_strategy_final :827-916, finish_strategy_final :919-973):

    python tests/golden/make_division_golden.py /path/to/reference [out_dir]

The module itself cannot be imported here (it pulls in the scene, the trainer's utilities and the CUDA extension), so
the five definitions are cut out of its source with `ast` and executed in a namespace whose `utils` is a stand-in
holding what they read: tile grid, rank, group size, the argument flags, the iteration counter, and the all-gather of
the ranks' render times, which returns the scenario's table.  The only change to the source text is the device of
the few heuristic tensors ("cuda" -> "cpu").  Every scenario is a few training steps of one rank: divide the batch,
"render" with a fixed per-row cost profile per camera (so the time of a band is the sum of its rows' costs), feed
the times back.  Stored per step: the time table, every camera's ranks and cuts, the task lists, and the heuristic
vectors after the update.  tests/test_workload_division.py replays the same tables through cgx.workload_division.
"""
import ast
import json
import sys
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
WANTED = ("division_pos_heuristic", "DivisionStrategyFinal", "DivisionStrategyHistoryFinal", "start_strategy_final",
          "finish_strategy_final")

SCENARIOS = [
    dict(name="four_ranks_4k", ws=4, n_cams=4, H=2160, W=3840, bsz=4, decay=0.0, warm=-1, border=1.0,
         local_sampling=False, steps=6, seed=1),
    dict(name="three_ranks_decay", ws=3, n_cams=5, H=2160, W=3840, bsz=2, decay=0.5, warm=1, border=2.0,
         local_sampling=False, steps=6, seed=2),
    dict(name="small_images_never_update", ws=2, n_cams=3, H=1080, W=1920, bsz=3, decay=0.0, warm=-1, border=1.0,
         local_sampling=False, steps=3, seed=3),
    dict(name="local_sampling", ws=2, n_cams=4, H=2160, W=3840, bsz=4, decay=0.0, warm=-1, border=1.0,
         local_sampling=True, steps=2, seed=4),
]


def load_reference(ref):
    src = (ref / "gaussian_renderer" / "workload_division.py").read_text()
    tree = ast.parse(src)
    parts = [ast.get_source_segment(src, node) for node in tree.body
             if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name in WANTED]
    assert len(parts) == len(WANTED)
    return "\n\n".join(parts).replace('device="cuda"', 'device="cpu"')


def cost_profile(n_cams, tile_y, seed):
    """Per camera a positive cost per tile row: a ramp plus a bump whose place depends on the camera."""
    gen = torch.Generator().manual_seed(seed)
    rows = torch.arange(tile_y, dtype=torch.float64)
    out = []
    for k in range(n_cams):
        centre = float(torch.rand(1, generator=gen)) * tile_y
        width = 10.0 + 20.0 * float(torch.rand(1, generator=gen))
        out.append(0.02 + 0.01 * rows / tile_y + 0.08 * torch.exp(-0.5 * ((rows - centre) / width) ** 2))
    return out


def run_scenario(code, sc):
    tile_y, tile_x = (sc["H"] + 15) // 16, (sc["W"] + 15) // 16
    state = {"iteration": 0, "table": None}
    args = types.SimpleNamespace(local_sampling=sc["local_sampling"], bsz=sc["bsz"], border_divpos_coeff=sc["border"],
                                 adjust_strategy_warmp_iterations=sc["warm"], no_heuristics_update=False,
                                 heuristic_decay=sc["decay"])
    utils = types.SimpleNamespace(
        BLOCK_X=16, BLOCK_Y=16, TILE_X=tile_x, TILE_Y=tile_y, GLOBAL_RANK=0, WORLD_SIZE=sc["ws"],
        DEFAULT_GROUP=types.SimpleNamespace(size=lambda: sc["ws"]), get_args=lambda: args,
        get_cur_iter=lambda: state["iteration"], get_img_height=lambda: sc["H"], get_img_width=lambda: sc["W"],
        our_allgather_among_cpu_processes_float_list=lambda values, group: state["table"])
    ns = {"torch": torch, "utils": utils, "diff_gaussian_rasterization": None, "dist": None, "time": None}
    exec(code, ns)
    cams = [types.SimpleNamespace(uid=100 + k) for k in range(sc["n_cams"])]
    history = ns["DivisionStrategyHistoryFinal"](types.SimpleNamespace(cameras=cams), sc["ws"], 0)
    cost = cost_profile(sc["n_cams"], tile_y, sc["seed"])
    steps = []
    for it in range(1, sc["steps"] + 1):
        state["iteration"] = it
        strategies, tasks = ns["start_strategy_final"](cams, history)
        table = [[-1.0] * sc["n_cams"] for _ in range(sc["ws"])]
        for k, s in enumerate(strategies):
            for rank, lo, hi in zip(s.gpu_ids, s.division_pos[:-1], s.division_pos[1:]):
                table[rank][k] = float(cost[k][lo:hi].sum())
        state["table"] = table
        collectors = [dict(forward_render_time=0.0, backward_render_time=0.0, forward_loss_time=0.0) for _ in cams]
        ns["finish_strategy_final"](cams, history, strategies, collectors)
        steps.append(dict(iteration=it, table=table, gpu_ids=[list(s.gpu_ids) for s in strategies],
                          division_pos=[list(map(int, s.division_pos)) for s in strategies],
                          tasks=[[list(map(int, t)) for t in ts] for ts in tasks],
                          heuristic=[history.accum_heuristic[c.uid].tolist() for c in cams],
                          log=history.history[-1]["all_gpu_running_time"]))
    return dict(scenario=sc, steps=steps)


def main():
    ref = Path(sys.argv[1])
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else HERE
    code = load_reference(ref)
    out = [run_scenario(code, sc) for sc in SCENARIOS]
    for o in out:
        last = o["steps"][-1]
        print(o["scenario"]["name"], "cuts of the last step:", last["division_pos"], "per-rank ms:",
              [round(x, 3) for x in last["log"]])
    path = out_dir / "division_golden.json"
    path.write_text(json.dumps(out))
    print(path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()

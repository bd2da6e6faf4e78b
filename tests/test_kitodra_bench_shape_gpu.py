"""Kitodra at the layer sizes bench.py times (width 1024, 8 heads on 2 key heads, heads of 128 in the lightning and window
layers and two maps of 64 over values of 128 in the difference layer, 32 experts of width 512 chosen four a token among
the best 4 of 8 groups, a shared expert, a window and chunks of 1,024), four layers deep with a small vocabulary: a
2,560-token prompt in one step (the tcgen05 window attention with the extra term and values that are keys, the tensor-core
flexible kernel with two maps and the cap, the tcgen05 products, the grouped experts with the clamped gate in their
epilogue, the recurrence) and tokens decoded one by one after it (experts pair by pair, attention with key splits), against
the plain implementation on the experts the engine chose."""
import os
import sys

import pytest

import helpers
import kitodra_helpers as kh

pytestmark = pytest.mark.gpu


def test_bench_shape_prompt_and_decode(tmp_path):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    cfg = bench.kitodra_config("s")
    cfg["vocab"], cfg["layers"] = 2048, cfg["layers"][:4]
    cfg_d, weights = kh.make_folder(str(tmp_path), cfg, seed=5, init_std=0.03)
    reqs = {"p": helpers.random_tokens(2566, cfg["vocab"], 3)}
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": reqs["p"][:2560], "want": [100, 1023, 1024, 1500, 2559]}], "end": []}]
    for i in range(6):
        steps.append({"step": 1 + i, "entries": [{"id": "p", "tokens": [reqs["p"][2560 + i]], "want": [0]}], "end": ["p"] if i == 5 else []})
    places = [100, 1023, 1024, 1500, 2559] + [2560 + i for i in range(6)]
    import torch
    for dtype in ("bfloat16", "float32"):
        outputs, runner = helpers.run_replay(str(tmp_path), dtype, steps, 2624, page_size=16, max_requests=2, tap=True)
        got = torch.cat([outputs[s["step"]] for s in steps])
        plain = kh.plain(cfg_d, weights, reqs["p"], runner.routing["p"]["experts"])[places]
        worst = kh.assert_close(got, plain, dtype, f"bench shape {dtype}")
        print(f"bench shape {dtype}: worst error {worst:.3e}")
    from quench6k_b200 import ops
    assert ops.tc_status() == 0

"""Helpers of the Kitodra tests: model folders with random weights and the comparison with the plain implementation."""
import json
import os

import torch

import helpers
import plain_kitodra
from kipedra_helpers import TOL          # noqa: F401  (the same tolerances)


def assert_close(got, want, dtype, what, tol=None):
    """Per position, the largest difference of the logits over the largest logit of the request.  A head's result of the
    difference attention is divided by its root mean square after a subtraction, so where the two maps nearly cancel the
    rounding is magnified: a few positions in hundreds stand well above the rest.  At most 2 % of the positions may pass the
    limit (5 % in bfloat16), none threefold.  (What the tests look for, a key, a sink or a state lost, is asserted to be
    many times the limit.)"""
    want = want.to(torch.float64)
    got = got.to(device=want.device, dtype=torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: the engine produced non-finite logits"
    scale = float(want.abs().max())
    per_pos = (got - want).abs().reshape(want.shape[0], -1).max(dim=-1).values / scale
    worst = int(per_pos.argmax())
    limit = tol if tol is not None else TOL[dtype]
    share = 0.05 if dtype == "bfloat16" else 0.02
    over = int((per_pos > limit).sum())
    assert over <= share * len(per_pos) + (0 if dtype == "bfloat16" else 1) and float(per_pos[worst]) <= 3.0 * limit, (
        f"{what}: {over} of {len(per_pos)} positions beyond {limit:.1e}, the worst {float(per_pos[worst]):.3e} of scale {scale:.3f} at position {worst}")
    return float(per_pos[worst])


def make_folder(folder, cfg_d, seed=0, init_std=0.15, doctor=None):
    """config.json + model.safetensors with random weights, the experts stored one by one; returns (config dict,
    {stored name: tensor}).  doctor(weights) may change tensors in place before they are written."""
    from quench6k_b200.config.kitodra import KitodraConfig
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.kitodra import build_spec
    from quench6k_b200.weights.random_init import make_tensor
    from quench6k_b200.weights.safetensors_io import write_safetensors

    cfg = KitodraConfig.from_dict(cfg_d)
    model = DecoderModel(build_spec(cfg, norm_init="random"))
    weights = {}
    for t in model.tensors():
        w = make_tensor(t, seed, init_std)
        w = w.to(torch.bfloat16) if w.dtype == torch.float32 else w                  # the files hold bfloat16 throughout
        if ".mlp.experts." in t.name:                                               # l<i>.mlp.experts.up -> l<i>.mlp.e<j>.up
            head, kind = t.name.split(".experts.")
            for j in range(w.shape[0]):
                weights[f"{head}.e{j}.{kind}"] = w[j].contiguous()
        else:
            weights[t.name] = w
    if doctor is not None:
        doctor(weights)
    os.makedirs(folder, exist_ok=True)
    cfg.save(folder)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights.items())
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f), weights


def plain(cfg_d, weights, tokens, forced=None):
    return plain_kitodra.forward(cfg_d, weights, tokens, forced=forced)


def replay_and_compare(folder, cfg, weights, requests, steps, max_tokens, dtype, what, page=None, max_requests=4, tol=None):
    """Replays the steps through the engine and compares every request with the plain implementation.  A mixture of experts
    is discontinuous (a rounding that flips a near-tie of two choice values moves a position by far more than rounding), so
    the engine reports the experts it chose and the plain implementation is run on those; how often its own choice would
    have differed is counted and must stay rare."""
    routed = any(L.get("mlp") for L in cfg["layers"])
    outputs, runner = helpers.run_replay(folder, dtype, steps, max_tokens, page_size=page, max_requests=max_requests, tap=routed)
    got = helpers.collect(requests, steps, outputs)
    worst, flips, positions = 0.0, 0, 0
    for rid, toks in requests.items():
        forced = runner.routing[rid]["experts"] if routed else None
        want = plain(cfg, weights, toks, forced)
        if routed:
            plain_kitodra.forward(cfg, weights, toks)
            for p, chosen in plain_kitodra.forward.chosen.items():
                flips += int((chosen.sort(-1).values != forced[p].sort(-1).values).any(-1).sum())
                positions += len(toks)
        worst = max(worst, assert_close(got[rid], want, dtype, f"{what} {dtype} {rid}", tol=tol))
    assert flips <= (0.002 if dtype == "float32" else 0.05) * positions + 1, f"{what} {dtype}: {flips} of {positions} choices of experts differ"
    print(f"{what} {dtype}: worst error {worst:.3e}, {flips} of {positions} choices of experts differ")
    return got


def plain_layers(cfg_d, weights, tokens, out):
    """Fills `out` with the plain implementation's stream after every layer."""
    plain_kitodra.forward(cfg_d, weights, tokens, layers_out=out)


def streams_of(runner, tokens):
    """The engine's stream after every executed layer for one prompt run in one step: every block's closing add, which the
    engine leaves to the block after it, is made at once and the stream copied."""
    from quench6k_b200.engine import StepEntry
    seen = []
    for b in runner.model.blocks:
        def forward(h, ctx, cache, state, pending=None, inner=b.forward, **kw):
            left = inner(h, ctx, cache, state, pending, **kw)
            if left is not None:
                left.apply(h)
            seen.append(h.clone())
            return None
        b.forward = forward
    runner.cuda_graphs = False
    runner.add_request("s")
    runner.step([StepEntry("s", list(tokens), [len(tokens) - 1])])
    runner.end_request("s")
    return seen

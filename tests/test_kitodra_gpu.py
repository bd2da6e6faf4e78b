"""The Kitodra decoder in the engine against the plain implementation (tests/plain_kitodra.py): the new kernels alone,
each mechanism alone (models of one layer), whole prompts against token-by-token decoding, portions down to two tokens,
mixed batches with so few pages and slots that both are used again, long decoding, and greedy generation through the
engine's entry point.

Where random weights would hide a fault the inputs are made so that it shows: the score scale of an attention layer is
raised so that the softmax of every (position, head) rests on few keys (a key wrongly seen or hidden, one position off at
a window's or a chunk's edge or a page's border, then moves that position's logits by far more than rounding), a model
is built whose every query looks for ONE token (at a window's edge, a chunk's edge, or hundreds of positions back),
scores are kept low where the extra term of the softmax denominator is to weigh, and lightning decays are close to (or
equal to) one so that the first tokens of a long prompt still weigh in its last positions (a state that is lost, or
started from another request's, shows)."""
import copy

import pytest
import torch

import helpers
import kitodra_configs as kc
import kitodra_helpers as kh
import plain_kitodra as pk

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


# ------------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("D, buckets, mp, mc, dt", [(24, 11, 3, 5, torch.float32), (130, 1, 7, 0, torch.bfloat16), (64, 521, 2_000_003, 1_000_000_007, torch.bfloat16)])
def test_token_pair_embedding_in_portions(D, buckets, mp, mc, dt):
    """h += table[hash(token before, token)]: the token before a portion's first row comes from the request's slot, a
    request's first token takes the table's last row, a sampled token that is still on the device is looked up there, and a
    slot nobody owns stays as it is."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(D)
    table = torch.randn(buckets + 1, D, generator=g).to(dt)
    seqs = [torch.randint(0, 2 ** 31 - 1, (n,), generator=g).tolist() for n in (40, 9)]
    bg = {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}
    want = [table.double()[pk.pair_rows(s, bg)] for s in seqs]
    for cuts in ([[40], [9]], [[1, 2, 30, 1, 6], [7, 2]], [[20, 3, 17], [1, 1, 7]]):
        prev = torch.full((4,), 123, dtype=torch.int32).cuda()
        got, at = [[], []], [0, 0]
        for step in range(max(len(c) for c in cuts)):
            live = [i for i in (0, 1) if step < len(cuts[i])]
            ctx = helpers.make_context([cuts[i][step] for i in live], [at[i] for i in live], [[[0]] * len(live)])
            ctx.slot_ids = torch.tensor([[3, 0][i] for i in live], dtype=torch.int32).cuda()
            toks = sum((seqs[i][at[i]:at[i] + cuts[i][step]] for i in live), [])
            fed = torch.tensor([toks[-1]], dtype=torch.int32).cuda()
            toks[-1] = -1                                   # the step's last token stands on the device
            h = torch.zeros(len(toks), D).cuda()
            ops.embed_pair(h, torch.tensor(toks, dtype=torch.int32).cuda(), table.cuda(), mp, mc, ctx.positions, ctx.req_of_token, ctx.q_start,
                           ctx.slot_ids, prev, fed=fed)
            row = 0
            for i in live:
                got[i].append(h[row:row + cuts[i][step]].double().cpu())
                row += cuts[i][step]
                at[i] += cuts[i][step]
        for i in (0, 1):
            assert torch.equal(torch.cat(got[i]), want[i]), f"cuts {cuts}, request {i}"
        assert prev.tolist() == [seqs[1][-1], 123, 123, seqs[0][-1]]


@pytest.mark.parametrize("E, k, groups, slices", [(6, 2, (3, 1), 1), (8, 4, (2, 1), 2), (12, 3, (4, 2), 1), (5, 5, None, 1), (64, 6, (8, 3), 3),
                                                  (9, 2, (9, 4), 1), (300, 8, (10, 10), 1), (16, 1, (16, 1), 1)])
def test_choice_of_experts_by_groups(E, k, groups, slices):
    """sigmoid scores, a correction that steers the choice, the choice limited to the groups of most worth, the plain scores
    as weights: against the plain implementation, token by token."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(E * k)
    T = 70
    z = torch.randn(slices, T, E, generator=g) * 2
    corr = torch.randn(E, generator=g)                     # of the scores' size and of both signs: choice values go negative
    router = {"experts": E, "top": k}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    sel_e, sel_w = ops.route_biased((z if slices > 1 else z[0]).contiguous().cuda(), k, corr.cuda(), 1.0, renorm=False, groups=groups)
    total = z[0].clone()
    for s in range(1, slices):
        total += z[s]
    for t in range(T):
        chosen, wt = pk.choose_experts(total[t].double(), corr.double(), router)
        assert sorted(sel_e[t].tolist()) == sorted(chosen.tolist()), f"token {t}"
        for e, w in zip(sel_e[t].tolist(), sel_w[t].tolist()):
            assert abs(w - float(torch.sigmoid(total[t, e].double()))) < 1e-6
    # renormalised weights still work, with and without groups
    sel_e2, sel_w2 = ops.route_biased(total.contiguous().cuda(), k, corr.cuda(), 2.5, renorm=True, groups=groups)
    assert torch.equal(sel_e2, sel_e) and torch.allclose(sel_w2.sum(-1), torch.full((T,), 2.5).cuda(), atol=1e-5)


@pytest.mark.parametrize("H, dv, dt", [(3, 12, torch.float32), (4, 96, torch.bfloat16), (1, 7, torch.float32), (2, 300, torch.bfloat16)])
def test_difference_of_two_maps(H, dv, dt):
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(H + dv)
    a = torch.randn(9, H, 2, dv, generator=g)
    want = pk.rms_norm(a[:, :, 0].double() - 0.37 * a[:, :, 1].double(), None, 1e-5) * 0.8
    got = ops.map_difference(a.view(9, -1).contiguous().cuda(), H, dv, 0.37, 1e-5, 0.8, dt)
    assert (got.double().cpu().view(9, H, dv) - want).abs().max() < (1e-5 if dt == torch.float32 else 0.03)


@pytest.mark.parametrize("H, dk, dv", [(3, 16, 24), (2, 100, 20), (5, 7, 9), (1, 136, 33), (4, 32, 80), (3, 8, 1400)])
def test_lightning_kernels_in_portions(H, dk, dv):
    """silu on the projections, the recurrence and the norm of all heads together with the sigmoid gate, over two requests
    whole and cut into portions, against loops in double precision."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(H * dk + dv)
    lens = [60, 17]
    N = 2 * H * dk + 2 * H * dv + 5
    g_col = 2 * H * dk + H * dv
    decay = torch.tensor([1.0, 0.99, 0.9, 0.5, 0.999][:H])
    w = torch.randn(H * dv, generator=g)
    seqs = [torch.randn(n, N, generator=g) for n in lens]
    want = []
    for x in seqs:
        n, xd = x.shape[0], x.double()
        q, k = pk.silu(xd[:, :H * dk]).view(n, H, dk), pk.silu(xd[:, H * dk:2 * H * dk]).view(n, H, dk)
        v = pk.silu(xd[:, 2 * H * dk:g_col]).view(n, H, dv)
        o = torch.zeros(n, H, dv, dtype=torch.float64)
        for h in range(H):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            for t in range(n):
                S = float(decay[h]) * S + torch.outer(k[t, h], v[t, h])
                o[t, h] = S.T @ q[t, h]
        want.append(pk.rms_norm(o.view(n, H * dv), w.double(), 1e-5) * torch.sigmoid(xd[:, g_col:g_col + H * dv]))
    for cuts in ([[60], [17]], [[1, 2, 30, 1, 26], [15, 2]], [[40, 3, 17], [1, 1, 15]]):
        state = torch.zeros(4, H, dk, dv).cuda()
        state[1] = 7.0
        got, at = [[], []], [0, 0]
        for step in range(max(len(c) for c in cuts)):
            live = [i for i in (0, 1) if step < len(cuts[i])]
            ctx = helpers.make_context([cuts[i][step] for i in live], [at[i] for i in live], [[[0]] * len(live)])
            ctx.slot_ids = torch.tensor([[3, 0][i] for i in live], dtype=torch.int32).cuda()
            p = torch.cat([seqs[i][at[i]:at[i] + cuts[i][step]] for i in live]).contiguous().cuda()
            ops.retention_prep(p, H, dk, 0, H * dk, None, 1.0, ctx.positions, act_cols=g_col)
            o = ops.retention(p, 0, H * dk, 2 * H * dk, decay.cuda(), state, ctx.q_start, ctx.slot_ids, ctx.R, H, dk, dv)
            y = ops.delta_out(o, p, g_col, w.cuda(), 1e-5, 1, H * dv, torch.float32, gate="sigmoid")
            row = 0
            for i in live:
                got[i].append(y[row:row + cuts[i][step]].double().cpu())
                row += cuts[i][step]
                at[i] += cuts[i][step]
        for i in (0, 1):
            err = (torch.cat(got[i]) - want[i]).abs().max() / want[i].abs().max()
            assert err < 2e-5, f"cuts {cuts}, request {i}: {float(err):.3e}"
        assert bool((state[1] == 7.0).all()) and bool((state[2] == 0).all())


# ------------------------------------------------------------------------------------------------- one mechanism alone
ONE = {
    "lightning": kc.lightning(3, 16, 24, [0.999, 0.99, 1.0]),
    "lightning_wide_keys": kc.lightning(2, 136, 33, [0.995, 0.9]),
    "lightning_and_experts": kc.lightning(2, 8, 8, [0.98, 1.0], kc.ff(6, 2, 20, 0.8, groups=(3, 1), shared=(12, 1.4))),
    "window": kc.sink(4, 2, 16, 0.5, 5, 8, 100.0),
    "window_of_pages": kc.sink(3, 3, 16, 0.6, 64, 16, 10000.0),
    "window_of_one": kc.sink(2, 1, 24, 0.4, 1, 6, 50.0),
    "window_never_reached": kc.sink(2, 2, 40, 0.3, 1000, 0, 10000.0),
    "window_tensor_cores": kc.sink(4, 2, 64, 0.12, 70, 32, 10000.0),
    "window_and_all_experts": kc.sink(2, 1, 8, 0.5, 6, 8, 20.0, kc.ff(3, 3, 20, 1.0)),
    "window_low_scores": kc.sink(4, 2, 16, 0.5, 9, 8, 100.0),
    "difference": kc.difference(4, 2, 8, 12, 0.8, 19, 4.0, 0.3),
    "difference_of_pages": kc.difference(2, 1, 16, 8, 0.6, 64, 30.0, 0.7),
    "difference_chunk_of_one": kc.difference(3, 3, 6, 10, 0.5, 1, 2.0, 0.2),
    "difference_tensor_cores": kc.difference(4, 2, 32, 64, 0.3, 48, 10.0, 0.5),
    "difference_and_one_expert": kc.difference(2, 2, 8, 16, 0.5, 23, 8.0, 0.4, kc.ff(4, 1, 12, 0.6, groups=(2, 1), shared=(8, 0.9))),
}


def _loud_maps(weights):
    """The four vectors behind the weight of the second map made large enough to move it well away from `diff`."""
    for name, w in weights.items():
        if name.endswith((".lq1", ".lk1")):
            w.fill_(0.25)
        if name.endswith((".lq2", ".lk2")):
            w.fill_(-0.2)


def _low_scores(weights):
    """Biases that point q and k of a window layer in opposite directions along the entries that do not turn: most scores
    lie below zero, so the denominator's extra term of score zero takes a good and changing part of every softmax."""
    for name, w in weights.items():
        if name.endswith(".mix.q.b") or name.endswith(".mix.k.b"):
            w.view(-1, 16)[:, 8:] += 4.0 if name.endswith("q.b") else -4.0


@pytest.fixture(scope="module", params=sorted(ONE))
def single(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    width = 128 if name.endswith("tensor_cores") else 48
    cfg, weights = kh.make_folder(folder, kc.one_layer(ONE[name], width=width, page=16 if width == 128 else 4), seed=3, init_std=0.3,
                                  doctor=_low_scores if name == "window_low_scores" else _loud_maps)
    reqs = {"long": helpers.random_tokens(330, cfg["vocab"], 1), "short": helpers.random_tokens(9, cfg["vocab"], 2),
            "one": helpers.random_tokens(1, cfg["vocab"], 3)}
    return name, folder, cfg, weights, reqs


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_whole_prompt(single, dtype):
    name, folder, cfg, weights, reqs = single
    steps, mt = helpers.schedule_whole(reqs)
    kh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_token_by_token(single, dtype):
    """Every token decoded alone from the first one on: each key is found through the cache, each state through its slot,
    each token's predecessor in the slot as well."""
    name, folder, cfg, weights, reqs = single
    reqs = {"long": reqs["long"][:150], "short": reqs["short"]}
    steps, mt = helpers.schedule_tail(reqs, tail=10 ** 6)
    kh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_portions(single, dtype):
    name, folder, cfg, weights, reqs = single
    for seed in (0, 1):
        steps, mt = helpers.schedule_portions(reqs, seed=seed)
        kh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} portions")


def test_a_fault_would_show(single):
    """The premise of the tests above: a key more or less in a window or a chunk, the extra term of the denominator left
    out, the second map forgotten, a token's predecessor mistaken or a state that forgot its first tokens, is far beyond
    the tolerance: the plain implementation, broken on purpose, differs from itself."""
    name, folder, cfg, weights, reqs = single
    if cfg["layers"][0]["mlp"] is not None:
        pytest.skip("written for the mixers alone")
    toks = reqs["long"]
    a = kh.plain(cfg, weights, toks)
    far = lambda b, rows=slice(None): ((a[rows] - b).abs().max(-1).values / a.abs().max()) > 3 * kh.TOL["bfloat16"]
    size = cfg["layers"][0]["mixer"].get("mask", {}).get("size", 0)
    if name.startswith(("window", "difference")) and 1 < size < 32 and name != "window_low_scores":
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["mask"]["size"] += 1
        assert far(kh.plain(other, weights, toks)).float().mean() > 0.15, "a key more does not show"
    if name in ("window_low_scores", "window_of_one"):
        b = pk.forward(cfg, weights, toks, mixers={"attention_2": lambda *x: pk.sink_attention(*x, sink=False)})
        assert far(b).float().mean() > 0.15, "the extra term of the denominator left out does not show"
    if name.startswith("difference") and size > 1:           # alone in its chunk a position's two maps are equal, and the norm hides their weight
        quiet = dict(weights)
        for n in ("lq1", "lk1", "lq2", "lk2"):
            quiet[f"l0.mix.{n}"] = torch.zeros_like(weights[f"l0.mix.{n}"])
        assert far(kh.plain(cfg, quiet, toks)).float().mean() > 0.15, "the weight of the second map does not show"
    if name.startswith("lightning"):
        b = kh.plain(cfg, weights, toks[150:])
        moved = (a[150:] - b).abs().max(-1).values / a.abs().max()
        assert (moved[1:40] > 3 * kh.TOL["bfloat16"]).float().mean() > 0.5, "a lost state does not show in the next tokens"
        assert float(moved[100:].median()) > 100 * kh.TOL["float32"], "the state of the first 150 tokens no longer shows 100 tokens later"
    swapped = list(toks)
    swapped[99] = (swapped[99] + 1) % cfg["vocab"]
    assert bool(far(kh.plain(cfg, weights, swapped)[100:101], slice(100, 101)).all()), "a token's predecessor does not show"


# ------------------------------------------------------------------------------------------------- a key that stands out
BEACON = 17


def _plain_tokens(n, vocab, seed):
    return [t if t != BEACON else 3 for t in helpers.random_tokens(n, vocab, seed)]


def _beacon(kind, heads, kv_heads, dim, vdim, maps, push):
    """Channel 0 of the stream is the same positive number for every token and channel 1 is zero for all tokens but one.
    The last entry of every key head (of the first map) reads channel 1 and the last entry of every query head (of the first
    map) reads channel 0: every query looks, above all, for that one token, and the entry lies outside the part of the head
    that turns.  The output projection leaves both channels alone, so the same holds in the layer that runs the same
    tensors afterwards.  The token-pair table and the layer's norm leave both channels alone too."""
    def doctor(w):
        w["embed"][:, 0] = 1.0
        w["embed"][:, 1] = 0.0
        w["embed"][BEACON, 1] = 4.0
        w["bigram"][:, :2] = 0.0
        w["l0.norm1"][:2] = 1.0
        w["l0.mix.o"][:2] = 0.0
        w["l0.mix.o.b"][:2] = 0.0
        for h in range(kv_heads):
            row = h * maps * dim + dim - 1
            w["l0.mix.k"][row] = 0.0
            w["l0.mix.k"][row, 1] = 10.0
            w["l0.mix.k.b"][row] = 0.0
            if kind == "attention":
                w["l0.mix.v"][h * vdim] = 0.0               # a value entry that tells the token from the others
                w["l0.mix.v"][h * vdim, 1] = 5.0
        for h in range(heads):
            row = h * maps * dim + dim - 1
            w["l0.mix.q"][row] = 0.0
            w["l0.mix.q"][row, 0] = push
            w["l0.mix.q.b"][row] = 0.0
        if kind == "attention":
            w["l0.mix.q.norm"][dim - 1] = 1.0
            w["l0.mix.k.norm"][dim - 1] = 1.0
    return doctor


EDGES = {
    # (layer, the size's place, sizes): a window and a chunk narrower than a page run and several pages wide
    "window": (kc.sink(3, 1, 8, 1.0, 11, 4, 100.0), 11),
    "wide_window": (kc.sink(2, 2, 8, 1.0, 37, 6, 100.0), 37),
    "chunk": (kc.difference(2, 1, 8, 5, 1.0, 13, 8.0, 0.3), 13),
    "wide_chunk": (kc.difference(4, 2, 8, 10, 1.0, 50, 8.0, 0.3), 50),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(EDGES))
def test_a_key_at_the_edge(tmp_path, which, dtype):
    """Two layers on the same tensors (the second with a cache of its own).  The token every query looks for stands at a page's
    border and inside a page; the last position that sees it and the first that does not lie in a prompt (whole and in
    portions) and among tokens decoded one by one."""
    layer, size = EDGES[which]
    m = layer["mixer"]
    kind = layer["type"]
    layers = [layer, kc.again([layer], 0)]
    cfg = kc.model(layers, width=48, vocab=61, page=4)
    cfg, weights = kh.make_folder(str(tmp_path), cfg, seed=11, init_std=0.15,
                                  doctor=_beacon(kind, m["heads"], m["kv_heads"], m["dim"], m["vdim"], 2 if kind == "attention" else 1, 3.0))
    toks = _plain_tokens(max(230, 5 * size + 20), cfg["vocab"], 5)
    # in a chunk: places that a chunk one position shorter hides from the chunk's last position and that a chunk one position
    # longer shows to the next chunk's first (second and fifth chunk)
    places = (8, 101) if kind == "attention_2" else (size + 3, 4 * (size + 1) + 1)
    for p in places:
        toks[p] = BEACON
    reqs = {"b": toks}
    want = kh.plain(cfg, weights, toks)
    scale = float(want.abs().max())
    narrower, wider = copy.deepcopy(cfg), copy.deepcopy(cfg)
    for L in narrower["layers"]:
        L["mixer"]["mask"]["size"] = size - 1
    for L in wider["layers"]:
        L["mixer"]["mask"]["size"] = size + 1
    less, more = kh.plain(narrower, weights, toks), kh.plain(wider, weights, toks)
    edges = []
    for p in places:
        last = p + size - 1 if kind == "attention_2" else p // size * size + size - 1          # the last position that sees the token
        gone = last + 1
        assert float((want[last] - less[last]).abs().max()) > 0.1 * scale, "the last position that sees the token does not rest on it"
        assert float((want[gone] - more[gone]).abs().max()) > 0.1 * scale, "the first position beyond the token would not rest on it"
        edges += [last, gone]
    for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "decoded": helpers.schedule_tail(reqs, tail=130),
                              "from the start": helpers.schedule_tail(reqs, tail=10 ** 6), "portions": helpers.schedule_portions(reqs, seed=2),
                              "portions again": helpers.schedule_portions(reqs, seed=3)}.items():
        outputs, _ = helpers.run_replay(str(tmp_path), dtype, steps, mt, max_requests=2)
        got = helpers.collect(reqs, steps, outputs)["b"]
        kh.assert_close(got, want, dtype, f"{which} edge, {what}")
        for at in edges:                              # the edges themselves, held to the plain tolerance whatever the rest does
            err = float((got[at].double() - want[at]).abs().max()) / scale
            assert err <= (3 if dtype == "bfloat16" else 1) * kh.TOL[dtype], f"{which} edge, {what} {dtype}: position {at}: {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_away(tmp_path, dtype):
    """A window and a chunk of several hundred positions: the token every query looks for stands near the start, and positions
    hundreds of tokens on (in the prompt, in portions and decoded) still rest on it."""
    layers = [kc.sink(2, 1, 8, 1.0, 400, 4, 100.0), kc.difference(2, 1, 8, 5, 1.5, 500, 20.0, 0.3)]
    for layer in layers:
        m, kind = layer["mixer"], layer["type"]
        folder = str(tmp_path / kind)
        cfg, weights = kh.make_folder(folder, kc.model([layer], width=48, vocab=61, page=4), seed=12, init_std=0.15,
                                      doctor=_beacon(kind, m["heads"], m["kv_heads"], m["dim"], m["vdim"], 2 if kind == "attention" else 1, 3.0))
        toks = _plain_tokens(390, cfg["vocab"], 6)
        toks[5] = BEACON
        reqs = {"f": toks}
        want = kh.plain(cfg, weights, toks)
        without = list(toks)
        without[5] = 3
        other = kh.plain(cfg, weights, without)
        assert float((want[300:] - other[300:]).abs().max(-1).values.min()) > 0.05 * float(want.abs().max()), "positions hundreds of tokens on do not rest on the token"
        for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "decoded": helpers.schedule_tail(reqs, tail=60),
                                  "portions": helpers.schedule_portions(reqs, seed=4)}.items():
            outputs, _ = helpers.run_replay(folder, dtype, steps, mt, max_requests=2)
            kh.assert_close(helpers.collect(reqs, steps, outputs)["f"], want, dtype, f"far key, {kind}, {what}")


# ------------------------------------------------------------------------------------------------- whole models
LENGTHS = {"T1": [71, 130, 45, 96, 64, 33, 1, 58, 77], "T2": [85, 140, 37, 101, 2, 50, 90, 125, 44], "T3": [90, 217, 129, 48, 75, 40, 150, 66, 83],
           "T4": [70, 33, 131, 20, 64, 3, 95, 41, 58]}


@pytest.fixture(scope="module", params=sorted(LENGTHS))
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    cfg, weights = kh.make_folder(folder, kc.get(name), seed=7, init_std=0.08, doctor=_loud_maps)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(LENGTHS[name])}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs}


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_whole(model, dtype):
    steps, mt = helpers.schedule_whole(model["requests"])
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " whole")


def test_the_stream_after_every_layer(model):
    """The residual stream after each layer against the plain implementation's, float32: a layer that is wrong is named."""
    import quench6k_b200 as q
    toks = model["requests"]["r0"]
    want = []
    kh.plain_layers(model["cfg"], model["weights"], toks, want)
    runner = q.engine.ModelRunner.from_folder(model["folder"], dtype="float32", page_size=model["cfg"]["kv_page_size"], num_pages=64, max_requests=2)
    got = kh.streams_of(runner, toks)
    assert len(got) == len(want)
    for i, (a, b) in enumerate(zip(got, want)):
        err = float((a.double().cpu() - b).abs().max() / b.abs().max())
        assert err < 1e-4, f"{model['name']}: the stream after layer {i} ({model['cfg']['layers'][i]['type']}): {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_prefill_then_decode(model, dtype):
    steps, mt = helpers.schedule_tail(model["requests"], tail=40)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " tail")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_portions(model, dtype):
    steps, mt = helpers.schedule_portions(model["requests"], seed=5)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_mixed_batches_reuse_pages_and_slots(model, dtype):
    """Up to four live requests, unequal portions beside single tokens, requests that sit steps out; nine requests go
    through four slots and a pool of the live requests' size, so every slot and most pages are used again."""
    page = model["cfg"]["kv_page_size"]
    for seed in (0, 1):
        steps, mt = helpers.schedule_mixed(model["requests"], page, seed=seed, max_live=4)
        got = kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype,
                                    model["name"] + " mixed", max_requests=4)
    if dtype == "float32":
        # and the same requests each alone: what else is in the batch, and which pages and slots are used, changes nothing
        steps, mt = helpers.schedule_whole(model["requests"])
        outputs, _ = helpers.run_replay(model["folder"], dtype, steps, mt)
        alone = helpers.collect(model["requests"], steps, outputs)
        for rid in model["requests"]:
            kh.assert_close(got[rid], alone[rid], dtype, f"{model['name']} {dtype} {rid} batched against alone", tol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_many_decoding_together(model, dtype):
    page = model["cfg"]["kv_page_size"]
    reqs = {rid: t for rid, t in model["requests"].items() if len(t) > 12}
    steps, mt = helpers.schedule_wide_decode(reqs, page)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " wide decode",
                          max_requests=len(reqs))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """A short prompt and hundreds of tokens decoded one by one: windows, chunks and pages pass over decoded tokens, the
    recurrent state runs long, the decode steps are replayed from a recorded graph."""
    reqs = {"d": helpers.random_tokens(420, model["cfg"]["vocab"], 9)}
    steps, mt = helpers.schedule_tail(reqs, tail=410)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " long decode")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt(model, dtype):
    """A prompt of 1,100 tokens whole, in portions, and with its last tokens decoded: a recurrent state a thousand tokens old,
    windows and chunks many times over."""
    if model["name"] != "T1":
        pytest.skip("one of the models is enough for the length (the plain implementation is slow)")
    reqs = {"p": helpers.random_tokens(1100, model["cfg"]["vocab"], 21)}
    for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "portions": helpers.schedule_portions(reqs, seed=8),
                              "tail": helpers.schedule_tail(reqs, tail=40)}.items():
        kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, f"{model['name']} long prompt {what}")


def test_greedy_generation_through_the_engine(model):
    """Engine.generate (scheduler, continuous batching, device-side argmax, tokens that stay on the device for the next step,
    CUDA graphs) against greedy decoding with the plain implementation, float32; prompts of unequal length in one engine
    with few pages."""
    import quench6k_b200 as q
    cfg, weights = model["cfg"], model["weights"]
    prompts = [helpers.random_tokens(n, cfg["vocab"], 50 + n) for n in (5, 23, 1, 40, 12, 31)]
    page = cfg["kv_page_size"]
    eng = q.Engine.from_folder(model["folder"], dtype="float32", page_size=page, num_pages=4 * (64 // page + 2), max_requests=4,
                               max_batch_tokens=32)
    outs = eng.generate(prompts, q.SamplingParams(max_tokens=12, temperature=0))
    for prompt, out in zip(prompts, outs):
        toks = list(prompt)
        for i in range(12):
            logits = kh.plain(cfg, weights, toks)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < 1e-3 * float(logits.abs().max()):
                break                                  # a near-tie: float32 may pick either; the continuation is not comparable
            assert out.tokens[i] == int(logits.argmax()), f"{model['name']}: prompt of {len(prompt)}, generated token {i}"
            toks.append(out.tokens[i])
    eng.runner.manager.check()


def test_command_line_generates(model):
    """`generate` of the command line on a Kitodra model folder: the model class comes from config.json."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, weights = model["cfg"], model["weights"]
    prompt = helpers.random_tokens(11, cfg["vocab"], 77)
    r = subprocess.run([sys.executable, "-m", "quench6k_b200", "generate", "--model", model["folder"], "--prompt-ids", ",".join(map(str, prompt)),
                        "--n", "6", "--dtype", "float32", "--context", "512"], cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    toks = list(prompt)
    for _ in range(6):
        logits = kh.plain(cfg, weights, toks)[-1]
        top2 = logits.topk(2).values
        if float(top2[0] - top2[1]) < 1e-3 * float(logits.abs().max()):
            return
        toks.append(int(logits.argmax()))
    assert "prompt: 11 tokens" in r.stdout and f"ids: {toks[11:]}" in r.stdout

"""The Sigusun decoder in the engine against the plain implementation (tests/plain_sigusun.py): the new kernels alone,
each mechanism alone (models of one layer), whole prompts against token-by-token decoding, portions down to two tokens,
mixed batches with so few pages and slots that both are used again, long decoding, and greedy generation through the
engine's entry point.

Where random weights would hide a fault the inputs are made so that it shows: the score scale of an attention layer is
raised so that the softmax of every (position, head) rests on one or two keys (a key wrongly seen or hidden, one
position off at the window's edge or a page's border, then moves that position's logits by far more than rounding),
a model is built whose every query looks for ONE token (at a window's edge, or hundreds of positions back), sinks are
made large enough to take a good part of the weight, and retention decays are close to (or equal to) one so that the
first tokens of a long prompt still weigh in its last positions (a state that is lost, or started from another
request's, shows)."""
import pytest
import torch

import helpers
import plain_sigusun
import sigusun_configs as sc
import sigusun_helpers as sh

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


# ------------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("H, dk, dv, rd", [(3, 16, 24, 8), (2, 100, 20, 100), (1, 136, 33, 0), (5, 7, 9, 6), (2, 256, 16, 64)])
def test_retention_kernels_in_portions(H, dk, dv, rd):
    """Rotation, scaling and the recurrence over two requests, whole and cut into portions of changing size, against loops
    in double precision; the state lives in the request's slot from step to step, and a slot nobody owns stays as it is."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(H * dk + dv)
    lens = [75, 22]
    N = 2 * H * dk + H * dv + 3
    decay = torch.tensor([1.0, 0.99, 0.9, 0.5, 0.999][:H])
    inv_freq = (100.0 ** (-2.0 * torch.arange(rd // 2, dtype=torch.float64) / max(rd, 1))).float()
    seqs = [torch.randn(n, N, generator=g) for n in lens]
    want = []
    for x in seqs:
        n, xd = x.shape[0], x.double()
        pos = torch.arange(n)
        rot = lambda t: plain_sigusun.rotate(t, pos, rd, 100.0, neighbours=False) if rd else t
        q, k = rot(xd[:, :H * dk].view(n, H, dk)), rot(xd[:, H * dk:2 * H * dk].view(n, H, dk)) * 0.3
        v = xd[:, 2 * H * dk:2 * H * dk + H * dv].view(n, H, dv)
        o = torch.zeros(n, H, dv, dtype=torch.float64)
        for h in range(H):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            for t in range(n):
                S = float(decay[h]) * S + torch.outer(k[t, h], v[t, h])
                o[t, h] = S.T @ q[t, h]
        want.append(o.view(n, H * dv))
    for cuts in ([[75], [22]], [[1, 2, 30, 1, 17, 24], [20, 2]], [[40, 3, 32], [1, 1, 20]]):
        state = torch.zeros(4, H, dk, dv).cuda()
        state[1] = 7.0
        got, at = [[], []], [0, 0]
        for step in range(max(len(c) for c in cuts)):
            live = [i for i in (0, 1) if step < len(cuts[i])]
            ctx = helpers.make_context([cuts[i][step] for i in live], [at[i] for i in live], [[[0]] * len(live)])
            ctx.slot_ids = torch.tensor([[3, 0][i] for i in live], dtype=torch.int32).cuda()
            p = torch.cat([seqs[i][at[i]:at[i] + cuts[i][step]] for i in live]).contiguous().cuda()
            ops.retention_prep(p, H, dk, 0, H * dk, (inv_freq.cuda(), rd, False) if rd else None, 0.3, ctx.positions)
            o = ops.retention(p, 0, H * dk, 2 * H * dk, decay.cuda(), state, ctx.q_start, ctx.slot_ids, ctx.R, H, dk, dv)
            row = 0
            for i in live:
                got[i].append(o[row:row + cuts[i][step]].double().cpu())
                row += cuts[i][step]
                at[i] += cuts[i][step]
        for i in (0, 1):
            err = (torch.cat(got[i]) - want[i]).abs().max() / want[i].abs().max()
            assert err < 2e-5, f"cuts {cuts}, request {i}: {float(err):.3e}"
        assert bool((state[1] == 7.0).all()) and bool((state[2] == 0).all())


@pytest.mark.parametrize("D, slices, S, dt", [(50, 1, 0, torch.float32), (256, 3, 3, torch.bfloat16), (1000, 2, 2, torch.float32), (96, 0, 4, torch.bfloat16),
                                              (4096, 1, 0, torch.bfloat16), (13000, 2, 1, torch.float32)])
def test_add_of_a_normed_result(D, slices, S, dt):
    """h += rms_norm(partial sums in order + weighted rows) * w, and the stream afterwards in the operand dtype."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(D)
    T = 6
    h, w = torch.randn(T, D, generator=g), torch.randn(D, generator=g)
    a = torch.randn(slices, T, D, generator=g) if slices else None
    total = a.double().sum(0) if slices else torch.zeros(T, D, dtype=torch.float64)
    weighted = None
    if S:
        y, pw = torch.randn(T * S, D, generator=g), torch.rand(T, S, generator=g)
        rows = torch.randperm(T * S, generator=g).to(torch.int32)
        total = total + (pw.double()[:, :, None] * y.double()[rows.long()].view(T, S, D)).sum(1)
        weighted = (y.cuda(), rows.cuda(), pw.cuda())
    want = h.double() + plain_sigusun.rms_norm(total, w.double(), 1e-5)
    hh = h.clone().cuda()
    arg = None if a is None else (a[0] if slices == 1 else a).contiguous().cuda()
    out = ops.add_normed(hh, arg, w.cuda(), 1e-5, dt, weighted=weighted)
    assert (hh.double().cpu() - want).abs().max() < 2e-5
    assert (out.double().cpu() - want).abs().max() < (2e-5 if dt == torch.float32 else 0.05)
    again = ops.add_normed(hh, None, None, 0.0, dt)                     # nothing to add: the stream as it stands
    assert torch.equal(again, out) and (hh.double().cpu() - want).abs().max() < 2e-5


def test_gate_of_the_token_input():
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(5)
    p, e = torch.randn(2, 9, 7, generator=g), torch.randn(9, 30, generator=g)
    want = plain_sigusun.gelu_tanh(p.double().sum(0)) * e.double()[:, 14:21]
    got = ops.side_gate(p.cuda(), e.cuda(), 14, torch.float32)
    assert (got.double().cpu() - want).abs().max() < 1e-5


@pytest.mark.parametrize("T, K, I, limit", [(5, 24, 13, 0.7), (40, 64, 48, 1.5), (300, 128, 64, 0.2), (8, 256, 96, 1.1)])
def test_clamped_gate_in_the_products_epilogue(T, K, I, limit):
    """g' = min(g, L), u' = clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1), on the CUDA-core product in float32 and, where the
    shape allows it, on the tensor-core product in bfloat16."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(T)
    x, wg, wu = torch.randn(T, K, generator=g), torch.randn(I, K, generator=g) * 0.3, torch.randn(I, K, generator=g) * 0.3

    def want(x, wg, wu):
        gg = torch.clamp(x.double() @ wg.double().T, max=limit)
        uu = torch.clamp(x.double() @ wu.double().T, min=-limit, max=limit)
        return gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)

    got = ops.gemm_simt(x.cuda(), wg.cuda(), w2=wu.cuda(), act=("clamped", limit))
    assert (got.double().cpu() - want(x, wg, wu)).abs().max() < 1e-4
    xb, gb, ub = x.bfloat16(), wg.bfloat16(), wu.bfloat16()
    if ops.tc_supported(xb.cuda(), gb.cuda()) and I % 8 == 0:
        got = ops.gemm_tc(xb.cuda(), gb.cuda(), w2=ub.cuda(), act=("clamped", limit))
        assert (got.double().cpu() - want(xb, gb, ub)).abs().max() < 0.03
    if T <= 16:                                 # the kernel for a few tokens
        got = ops.gemm_skinny(xb.cuda(), gb.cuda(), w2=ub.cuda(), act=("clamped", limit))
        assert (got.double().cpu() - want(xb, gb, ub)).abs().max() < 0.03


# ------------------------------------------------------------------------------------------------- one mechanism alone
ONE = {
    "retention": (sc.retention(3, 16, 24, [0.999, 0.99, 1.0], 8, 500.0), 0),
    "retention_wide_keys": (sc.retention(2, 136, 33, [0.995, 0.9], 136, 10000.0), 0),
    "retention_no_rotation": (sc.retention(1, 40, 8, [0.99], 0, 1.0), 3),
    "retention_and_experts": (sc.retention(2, 8, 8, [0.98, 1.0], 4, 50.0, ff=(5, 2, 20, 0.8, 12, 1.4)), 0),
    "window": (sc.window(4, 8, 12, 10, 24, 0.6, 5, 100.0), 0),
    "window_of_pages": (sc.window(3, 16, 4, 4, 16, 2.0, 64, 10000.0), 0),
    "window_of_one": (sc.window(2, 16, 16, 16, 20, 1.0, 1, 50.0), 0),
    "window_never_reached": (sc.window(2, 40, 0, 40, 12, 1.5, 1000, 10000.0), 0),
    "window_and_all_experts": (sc.window(2, 8, 8, 8, 16, 0.5, 6, 20.0, ff=(3, 3, 20, 1.0, None, 0)), 4),
    "sink": (sc.sink(3, 12, 4, 8, 20, 0.5, 3000.0), 0),
    "sink_and_one_expert": (sc.sink(2, 8, 8, 16, 40, 0.5, 100.0, ff=(4, 1, 12, 0.6, 8, 0.9)), 6),
}


def _loud_sinks(weights):
    """Sinks of the size of the largest scores, and different from head to head: a sink takes a good part of its head's
    weight.  (The norm on the mixer's result takes out what all heads lose alike; what one head loses more than another
    stays.)"""
    for name, w in weights.items():
        if name.endswith(".sink"):
            w.copy_(torch.linspace(20.0, 0.0, w.numel()))


@pytest.fixture(scope="module", params=sorted(ONE))
def single(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    layer, side = ONE[name]
    cfg, weights = sh.make_folder(folder, sc.one_layer(layer, side=side), seed=3, init_std=0.3, doctor=_loud_sinks)
    reqs = {"long": helpers.random_tokens(330, cfg["vocab"], 1), "short": helpers.random_tokens(9, cfg["vocab"], 2),
            "one": helpers.random_tokens(1, cfg["vocab"], 3)}
    return name, folder, cfg, weights, reqs


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_whole_prompt(single, dtype):
    name, folder, cfg, weights, reqs = single
    steps, mt = helpers.schedule_whole(reqs)
    sh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_token_by_token(single, dtype):
    """Every token decoded alone from the first one on: each key is found through the cache, each state through its slot."""
    name, folder, cfg, weights, reqs = single
    reqs = {"long": reqs["long"][:150], "short": reqs["short"]}
    steps, mt = helpers.schedule_tail(reqs, tail=10 ** 6)
    sh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_portions(single, dtype):
    name, folder, cfg, weights, reqs = single
    for seed in (0, 1):
        steps, mt = helpers.schedule_portions(reqs, seed=seed)
        sh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} portions")


def test_a_fault_would_show(single):
    """The premise of the tests above: a key more or less in a window, a sink left out, or a state that forgot its first
    tokens, is far beyond the tolerance.  The plain implementation with the window one wider, without the sink, or
    started in the middle, differs from itself."""
    name, folder, cfg, weights, reqs = single
    if cfg["layers"][0]["mlp"] is not None:
        pytest.skip("written for the mixers alone")
    a = sh.plain(cfg, weights, reqs["long"])
    if name.startswith("window") and cfg["layers"][0]["mixer"]["mask"]["size"] < 32:
        other = sc.one_layer(ONE[name][0])
        other["layers"][0]["mixer"]["mask"]["size"] += 1
        b = sh.plain(other, weights, reqs["long"])
        moved = ((a - b).abs().max(-1).values / a.abs().max()) > 3 * sh.TOL["bfloat16"]
        assert moved.float().mean() > 0.15
    elif name.startswith("sink"):
        silent = dict(weights)
        silent["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], -30.0)
        b = sh.plain(cfg, silent, reqs["long"])
        moved = ((a - b).abs().max(-1).values / a.abs().max()) > 3 * sh.TOL["bfloat16"]
        assert moved.float().mean() > 0.15, "a sink left out does not show"
    elif name.startswith("retention"):
        b = sh.plain(cfg, weights, reqs["long"][150:])
        moved = (a[150:] - b).abs().max(-1).values / a.abs().max()
        assert (moved[:40] > 3 * sh.TOL["bfloat16"]).float().mean() > 0.5, "a lost state does not show in the next tokens"
        assert float(moved[100:].median()) > 100 * sh.TOL["float32"], "the state of the first 150 tokens no longer shows 100 tokens later"
    else:
        pytest.skip("written for the window, the sink and the recurrent state")


# ------------------------------------------------------------------------------------------------- a key that stands out
BEACON, NEAR, WIDE = 17, 11, 37


def _beacon_doctor(own, layers, heads, dim, rd, push):
    """Channel 0 of the stream is the same positive number for every ordinary token and channel 1 is zero for all tokens but
    one.  Entry 0 of the latent reads channel 1, entry 0 of every head's key reads entry 0 of the latent, and entry 0 of
    every head's query reads channel 0: every query looks, above all, for that one token.  The norms on the mixers' results
    leave both channels alone, so the same holds in every layer."""
    def doctor(w):
        w["embed"][:, 0] = 1.0
        w["embed"][:, 1] = 0.0
        w["embed"][BEACON, 1] = 4.0
        w["embed.norm"][:2] = 1.0
        for i in range(layers):
            w[f"l{i}.norm1"][:2] = 0.0
            if i in own:
                w[f"l{i}.mix.dkv"][0] = 0.0
                w[f"l{i}.mix.dkv"][0, 1] = 10.0
                w[f"l{i}.mix.dkv.norm"][0] = 1.0
            for h in range(heads[i]):
                w[f"l{i}.mix.uk"][h * dim] = 0.0
                w[f"l{i}.mix.uk"][h * dim, 0] = 1.0
                w[f"l{i}.mix.q"][h * (dim + rd)] = 0.0
                w[f"l{i}.mix.q"][h * (dim + rd), 0] = push
    return doctor


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_at_the_window_edge(tmp_path, dtype):
    """Two layers over ONE cached latent, the first under a narrow window and the second, which borrows the first one's
    latent, under a wider one.  The token every query looks for stands at a page's border and inside a page; for both
    windows the last position that sees it and the first that does not lie in a prompt (whole and in portions) and among
    tokens decoded one by one."""
    cfg = sc.model([sc.window(3, 8, 4, 8, 16, 1.0, NEAR, 100.0), sc.window(2, 8, 4, 12, 16, 1.0, WIDE, 100.0, kv_from=0)], width=48, vocab=61, page=4)
    cfg, weights = sh.make_folder(str(tmp_path), cfg, seed=11, init_std=0.15, doctor=_beacon_doctor({0}, 2, [3, 2], 8, 4, 1.5))
    toks = [t if t != BEACON else 3 for t in helpers.random_tokens(200, cfg["vocab"], 5)]
    for p in (8, 101):
        toks[p] = BEACON
    reqs = {"b": toks}
    want = sh.plain(cfg, weights, toks)
    scale = float(want.abs().max())
    edges = []
    for layer, size in ((0, NEAR), (1, WIDE)):
        narrower, wider = sc.model(cfg["layers"], 48, 61, 4), sc.model(cfg["layers"], 48, 61, 4)
        narrower["layers"][layer]["mixer"]["mask"]["size"] = size - 1
        wider["layers"][layer]["mixer"]["mask"]["size"] = size + 1
        less, more = sh.plain(narrower, weights, toks), sh.plain(wider, weights, toks)
        for p in (8, 101):
            last, gone = p + size - 1, p + size
            assert float((want[last] - less[last]).abs().max()) > 0.1 * scale, "the last position that sees the token does not rest on it"
            assert float((want[gone] - more[gone]).abs().max()) > 0.1 * scale, "the first position beyond the token would not rest on it"
            edges += [last, gone]
    for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "decoded": helpers.schedule_tail(reqs, tail=70),
                              "from the start": helpers.schedule_tail(reqs, tail=10 ** 6), "portions": helpers.schedule_portions(reqs, seed=2),
                              "portions again": helpers.schedule_portions(reqs, seed=3)}.items():
        outputs, _ = helpers.run_replay(str(tmp_path), dtype, steps, mt, max_requests=2)
        got = helpers.collect(reqs, steps, outputs)["b"]
        sh.assert_close(got, want, dtype, f"window edge, {what}")
        for at in edges:                              # the edges themselves, held to the plain tolerance whatever the rest does
            err = float((got[at].double() - want[at]).abs().max()) / scale
            assert err <= (3 if dtype == "bfloat16" else 1) * sh.TOL[dtype], f"window edge, {what} {dtype}: position {at}: {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_away_and_the_sink(tmp_path, dtype):
    """A causal layer with sinks: the token every query looks for stands among the first tokens of a prompt of hundreds, and
    the last positions (in the prompt and decoded) still rest on it; sinks as large as that score share the weight with it."""
    cfg = sc.model([sc.sink(3, 8, 4, 8, 16, 1.0, 100.0)], width=48, vocab=61, page=4)
    base = _beacon_doctor({0}, 1, [3], 8, 4, 1.5)

    def doctor(w):
        base(w)
        w["l0.mix.sink"].copy_(torch.tensor([30.0, 20.0, 10.0]))

    cfg, weights = sh.make_folder(str(tmp_path), cfg, seed=12, init_std=0.15, doctor=doctor)
    toks = [t if t != BEACON else 3 for t in helpers.random_tokens(520, cfg["vocab"], 6)]
    toks[5] = BEACON
    reqs = {"f": toks}
    want = sh.plain(cfg, weights, toks)
    scale = float(want.abs().max())
    without = list(toks)
    without[5] = 3
    other = sh.plain(cfg, weights, without)
    assert float((want[300:] - other[300:]).abs().max(-1).values.min()) > 0.1 * scale, "a position hundreds of tokens on does not rest on the token"
    silent = dict(weights)
    silent["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], -30.0)
    other = sh.plain(cfg, silent, toks)
    assert float((want[300:] - other[300:]).abs().max(-1).values.median()) > 0.1 * scale, "a sink left out does not show"
    for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "decoded": helpers.schedule_tail(reqs, tail=60),
                              "portions": helpers.schedule_portions(reqs, seed=4)}.items():
        outputs, _ = helpers.run_replay(str(tmp_path), dtype, steps, mt, max_requests=2)
        got = helpers.collect(reqs, steps, outputs)["f"]
        sh.assert_close(got, want, dtype, f"far key, {what}")


# ------------------------------------------------------------------------------------------------- whole models
LENGTHS = {"G1": [71, 130, 45, 96, 64, 33, 1, 58, 77], "G2": [85, 140, 37, 101, 2, 50, 90, 125, 44], "G3": [90, 257, 129, 48, 75, 40, 310, 66, 83],
           "G4": [70, 33, 131, 20, 64, 3, 95, 41, 58]}


@pytest.fixture(scope="module", params=sorted(LENGTHS))
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    cfg, weights = sh.make_folder(folder, sc.get(name), seed=7, init_std=0.08)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(LENGTHS[name])}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs}


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_whole(model, dtype):
    steps, mt = helpers.schedule_whole(model["requests"])
    sh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " whole")


def test_the_stream_after_every_layer(model):
    """The residual stream after each layer against the plain implementation's, float32: a layer that is wrong is named."""
    import quench6k_b200 as q
    toks = model["requests"]["r0"]
    want = []
    sh.plain_layers(model["cfg"], model["weights"], toks, want)
    runner = q.engine.ModelRunner.from_folder(model["folder"], dtype="float32", page_size=model["cfg"]["kv_page_size"], num_pages=64, max_requests=2)
    got = sh.streams_of(runner, toks)
    assert len(got) == len(want)
    for i, (a, b) in enumerate(zip(got, want)):
        err = float((a.double().cpu() - b).abs().max() / b.abs().max())
        assert err < 1e-4, f"{model['name']}: the stream after layer {i} ({model['cfg']['layers'][i]['type']}): {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_prefill_then_decode(model, dtype):
    steps, mt = helpers.schedule_tail(model["requests"], tail=40)
    sh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " tail")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_portions(model, dtype):
    steps, mt = helpers.schedule_portions(model["requests"], seed=5)
    sh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_mixed_batches_reuse_pages_and_slots(model, dtype):
    """Up to four live requests, unequal portions beside single tokens, requests that sit steps out; nine requests go
    through four slots and a pool of the live requests' size, so every slot and most pages are used again."""
    page = model["cfg"]["kv_page_size"]
    for seed in (0, 1):
        steps, mt = helpers.schedule_mixed(model["requests"], page, seed=seed, max_live=4)
        got = sh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype,
                                    model["name"] + " mixed", max_requests=4)
    if dtype == "float32":
        # and the same requests each alone: what else is in the batch, and which pages and slots are used, changes nothing
        steps, mt = helpers.schedule_whole(model["requests"])
        outputs, _ = helpers.run_replay(model["folder"], dtype, steps, mt)
        alone = helpers.collect(model["requests"], steps, outputs)
        for rid in model["requests"]:
            sh.assert_close(got[rid], alone[rid], dtype, f"{model['name']} {dtype} {rid} batched against alone", tol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_many_decoding_together(model, dtype):
    page = model["cfg"]["kv_page_size"]
    reqs = {rid: t for rid, t in model["requests"].items() if len(t) > 12}
    steps, mt = helpers.schedule_wide_decode(reqs, page)
    sh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " wide decode",
                          max_requests=len(reqs))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """A short prompt and hundreds of tokens decoded one by one: windows and pages pass over decoded tokens, the recurrent
    state runs long, the decode steps are replayed from a recorded graph."""
    reqs = {"d": helpers.random_tokens(420, model["cfg"]["vocab"], 9)}
    steps, mt = helpers.schedule_tail(reqs, tail=410)
    sh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " long decode")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt(model, dtype):
    """A prompt of 1,300 tokens whole, in portions, and with its last tokens decoded: windows and the causal layers' key
    ranges at lengths several times the short requests', a recurrent state a thousand tokens old."""
    if model["name"] not in ("G1", "G3"):
        pytest.skip("two of the models are enough for the length (the plain implementation is slow)")
    reqs = {"p": helpers.random_tokens(1300, model["cfg"]["vocab"], 21)}
    for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "portions": helpers.schedule_portions(reqs, seed=8),
                              "tail": helpers.schedule_tail(reqs, tail=40)}.items():
        sh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, f"{model['name']} long prompt {what}")


def test_greedy_generation_through_the_engine(model):
    """Engine.generate (scheduler, continuous batching, device-side argmax, CUDA graphs) against greedy decoding with the
    plain implementation, float32; prompts of unequal length in one engine with few pages."""
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
            logits = sh.plain(cfg, weights, toks)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < 1e-3 * float(logits.abs().max()):
                break                                  # a near-tie: float32 may pick either; the continuation is not comparable
            assert out.tokens[i] == int(logits.argmax()), f"{model['name']}: prompt of {len(prompt)}, generated token {i}"
            toks.append(out.tokens[i])
    eng.runner.manager.check()


def test_command_line_generates(model):
    """`generate` of the command line on a Sigusun model folder: the model class comes from config.json."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, weights = model["cfg"], model["weights"]
    prompt = helpers.random_tokens(11, cfg["vocab"], 77)
    r = subprocess.run([sys.executable, "-m", "quench6k_b200", "generate", "--model", model["folder"], "--prompt-ids", ",".join(map(str, prompt)),
                        "--n", "6", "--dtype", "float32", "--context", "128"], cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    toks = list(prompt)
    for _ in range(6):
        logits = sh.plain(cfg, weights, toks)[-1]
        top2 = logits.topk(2).values
        if float(top2[0] - top2[1]) < 1e-3 * float(logits.abs().max()):
            return
        toks.append(int(logits.argmax()))
    assert "prompt: 11 tokens" in r.stdout and f"ids: {toks[11:]}" in r.stdout

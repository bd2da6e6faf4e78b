"""Kitodra on the host: configuration, execution order, declared tensors, caches and states, stored names, and the plain
implementation's own pieces against closed forms and each other (no GPU)."""
import math
import tempfile

import pytest
import torch

import kitodra_configs as kc
import plain_kitodra as pk
from quench6k_b200.config.kitodra import KitodraConfig
from quench6k_b200.config.pedotar import ConfigError
from quench6k_b200.config.registry import architecture_of
from quench6k_b200.models.decoder import DecoderModel
from quench6k_b200.models.kitodra import build_spec, stored_name

F = torch.float64


@pytest.mark.parametrize("name", sorted(kc.ALL))
def test_config_round_trip_and_order(name):
    d = kc.get(name)
    cfg = KitodraConfig.from_dict(d)
    assert KitodraConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    spec = build_spec(cfg)
    own = [i for i, L in enumerate(d["layers"]) if L.get("weights_of") is None]
    assert [ls.prefix for ls in spec.layers] == [f"l{i}." for i in own]
    # every executed position runs the tensors of the layer the plain implementation takes, on a cache of its own
    assert [own[j] for j in spec.order] == [pk.weights_layer(d, i) for i in range(len(d["layers"]))]
    assert spec.kv_source == [None] * len(d["layers"]) and spec.head_name is None
    assert (spec.embed_add is None) == ("embedding" not in d)
    assert architecture_of(d).name == "Kitodra" and architecture_of({"architectures": ["kitodra"]}).name == "Kitodra"


def test_config_errors_name_the_key():
    def broken(name, change, match):
        d = kc.get(name)
        change(d)
        with pytest.raises(ConfigError, match=match):
            KitodraConfig.from_dict(d)

    broken("T1", lambda d: d["layers"][1]["mixer"].pop("scale"), "scale")
    broken("T1", lambda d: d["layers"][0]["mixer"]["decay"].pop(), "decay")
    broken("T1", lambda d: d["layers"][1]["mixer"]["rot"].update(dims=18), "rotating")
    broken("T1", lambda d: d["layers"][1]["mixer"].pop("mask"), "mask")
    broken("T1", lambda d: d["layers"][1]["mixer"].update(vdim=8), "vdim")
    broken("T1", lambda d: d["layers"][2]["mixer"].pop("softcap"), "softcap")
    broken("T1", lambda d: d["layers"][2]["mixer"].update(kv_heads=3), "kv_heads")
    broken("T1", lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "top")
    broken("T1", lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups")
    broken("T1", lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "kept groups")
    broken("T1", lambda d: d["layers"][3].update(weights_of=9), "weights_of")
    broken("T1", lambda d: d["layers"][3].update(weights_of=0), "differs")            # a window layer cannot run a lightning layer's tensors
    broken("T1", lambda d: (d["layers"][0].update(weights_of=4), d["layers"][4].update(weights_of=0)), "circle")
    broken("T1", lambda d: d["embedding"]["bigram"].pop("buckets"), "buckets")
    broken("T1", lambda d: d.pop("norm"), "norm")
    broken("T1", lambda d: d["layers"][0].update(type="retention"), "type")
    broken("T1", lambda d: d["layers"][0]["mlp"].pop("expert"), "expert")


def test_declared_tensors_caches_and_states():
    cfg = KitodraConfig.from_dict(kc.get("T1"))
    model = DecoderModel(build_spec(cfg))
    names = {t.name: tuple(t.shape) for t in model.tensors()}
    assert names["embed"] == (211, 96) and names["bigram"] == (102, 96) and names["final.norm"] == (96,) and "head" not in names
    assert names["l0.mix.q"] == (48, 96) and names["l0.mix.v"] == (72, 96) and names["l0.mix.g"] == (72, 96) and names["l0.mix.o"] == (96, 72)
    assert names["l0.mix.norm"] == (72,) and "l0.mix.q.b" not in names
    assert names["l0.mlp.router"] == (6, 96) and names["l0.mlp.correction"] == (6,) and names["l0.mlp.experts.gate"] == (6, 40, 96)
    assert names["l0.mlp.shared.up"] == (24, 96) and "l1.mlp.shared.up" not in names
    # the window layer: values are the keys, so no value projection; biases on q, k and o
    assert names["l1.mix.q"] == (64, 96) and names["l1.mix.k"] == (32, 96) and "l1.mix.v" not in names and "l1.mix.v.b" not in names
    assert names["l1.mix.q.b"] == (64,) and names["l1.mix.k.b"] == (32,) and names["l1.mix.o.b"] == (96,) and "l1.mix.q.norm" not in names
    # the difference layer: two maps side by side in q and k, one set of values, norm weights shared by heads and maps
    assert names["l2.mix.q"] == (4 * 2 * 8, 96) and names["l2.mix.k"] == (1 * 2 * 8, 96) and names["l2.mix.v"] == (12, 96)
    assert names["l2.mix.q.norm"] == (8,) and names["l2.mix.lq1"] == (8,) and names["l2.mix.lk2"] == (8,) and names["l2.mix.o"] == (96, 48)
    assert not any(n.startswith(("l3.", "l4.")) for n in names) and "l0.norm2" not in names          # borrowed tensors, one norm a layer
    assert stored_name("l0.mlp.e3.up") == ("l0.mlp.experts.up", 3) and stored_name("l12.mlp.e10.gate") == ("l12.mlp.experts.gate", 10)
    assert stored_name("l0.mlp.shared.gate") is None and stored_name("l0.mlp.router") is None
    states = model.state_shapes()
    assert states[0] == {"S": ((3, 16, 24), torch.float32)} and states[4] == states[0] and states[1] is None
    assert states[5] == {"prev": ((), torch.int32)}                      # the token before a portion, one per request
    reqs = model.cache_requests()
    assert reqs[0] is None and reqs[4] is None
    assert (reqs[1].kind, reqs[1].window, reqs[1].kv_heads, reqs[1].head_dim) == ("sliding", 7, 2, 16) and reqs[3].key() == reqs[1].key()
    assert (reqs[2].kind, reqs[2].window, reqs[2].kv_heads, reqs[2].v_heads, reqs[2].head_dim, reqs[2].v_dim) == ("chunked", 19, 2, 1, 8, 12)


# ----------------------------------------------------------------------------- the plain pieces against closed forms
def _w(d):
    return lambda n: d[n]


def test_pair_rows():
    bg = {"buckets": 7, "mul_prev": 2, "mul_cur": 9}
    assert pk.pair_rows([4, 1, 6, 6], bg).tolist() == [7, (8 + 9) % 7, (2 + 54) % 7, (12 + 54) % 7]
    assert pk.pair_rows([5], bg).tolist() == [7]


def test_rotation_turns_pairs_by_halves():
    x = torch.zeros(3, 1, 6, dtype=F)
    x[:, 0, 0] = 1.0                      # entry 0 pairs with entry 2 when 4 entries turn; entries 4 and 5 stay
    x[:, 0, 5] = 3.0
    y = pk.rotate_halves(x, torch.arange(3), 4, 10.0)
    for p in range(3):
        assert abs(float(y[p, 0, 0]) - math.cos(p)) < 1e-12 and abs(float(y[p, 0, 2]) - math.sin(p)) < 1e-12
        assert float(y[p, 0, 1]) == 0.0 and float(y[p, 0, 5]) == 3.0
    assert torch.allclose((y * y).sum(-1), (x * x).sum(-1))


def test_lightning_second_token_and_decay_of_one():
    g = torch.Generator().manual_seed(1)
    D, H, dk, dv = 10, 2, 3, 4
    m = {"heads": H, "dim": dk, "vdim": dv, "decay": [0.5, 1.0]}
    W = {n: torch.randn(s, generator=g, dtype=F) for n, s in (("q", (H * dk, D)), ("k", (H * dk, D)), ("v", (H * dv, D)), ("g", (H * dv, D)),
                                                               ("o", (D, H * dv)), ("norm", (H * dv,)))}
    h = torch.randn(5, D, generator=g, dtype=F)
    q, k, v = (pk.silu(h @ W[n].T) for n in "qkv")
    o = []
    for head, dec in enumerate(m["decay"]):
        qh, kh, vh = q[:, head * dk:(head + 1) * dk], k[:, head * dk:(head + 1) * dk], v[:, head * dv:(head + 1) * dv]
        o.append(sum(dec ** (1 - j) * (qh[1] @ kh[j]) * vh[j] for j in range(2)))       # the second token sees two keys
    want = (pk.rms_norm(torch.cat(o), W["norm"], 1e-5) * torch.sigmoid(h[1] @ W["g"].T)) @ W["o"].T
    assert torch.allclose(pk.lightning(h, _w(W), m, 1e-5)[1], want, atol=1e-12)


def _difference_weights(g, D, H, G, d, dv):
    W = {n: torch.randn(s, generator=g, dtype=F) for n, s in (("q", (H * 2 * d, D)), ("k", (G * 2 * d, D)), ("v", (G * dv, D)), ("o", (D, H * dv)),
                                                               ("q.b", (H * 2 * d,)), ("k.b", (G * 2 * d,)), ("v.b", (G * dv,)), ("o.b", (D,)),
                                                               ("q.norm", (d,)), ("k.norm", (d,)))}
    for n in ("lq1", "lk1", "lq2", "lk2"):
        W[n] = torch.randn(d, generator=g, dtype=F) * 0.3
    return W


def test_difference_attention_equal_maps_and_chunks():
    g = torch.Generator().manual_seed(2)
    D, H, G, d, dv, C = 12, 4, 2, 3, 5, 4
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.7, "softcap": 2.0, "diff": 0.25, "mask": {"size": C}}
    W = _difference_weights(g, D, H, G, d, dv)
    h = torch.randn(11, D, generator=g, dtype=F)
    full = pk.difference_attention(h, _w(W), m, 1e-6)
    # a position sees its own chunk only: the second chunk alone gives the same rows
    assert torch.allclose(pk.difference_attention(h[4:8], _w(W), m, 1e-6), full[4:8], atol=1e-12)
    # the first position of a chunk sees itself only: both maps return its value, o = (1 - L) v, normed
    lam = pk.difference_weight(_w(W), m)
    assert abs(lam - (math.exp(float(W["lq1"] @ W["lk1"])) - math.exp(float(W["lq2"] @ W["lk2"])) + 0.25)) < 1e-12
    v = (h[8] @ W["v"].T + W["v.b"]).view(G, dv)
    heads = torch.stack([pk.rms_norm((1 - lam) * v[hd // (H // G)], None, 1e-6) * 0.75 for hd in range(H)])
    assert torch.allclose(full[8], heads.reshape(-1) @ W["o"].T + W["o.b"], atol=1e-12)
    # a cap far above the scores changes nothing, a small one does
    loose = dict(m, softcap=1e6)
    s_uncapped = pk.difference_attention(h, _w(W), loose, 1e-6)
    assert not torch.allclose(s_uncapped, full, atol=1e-6)


def test_sink_attention_window_sink_and_values():
    g = torch.Generator().manual_seed(3)
    D, H, G, d = 9, 4, 2, 6
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 0.9, "mask": {"size": 3}, "rot": {"base": 100.0, "dims": 4}}
    W = {n: torch.randn(s, generator=g, dtype=F) for n, s in (("q", (H * d, D)), ("k", (G * d, D)), ("o", (D, H * d)), ("q.b", (H * d,)),
                                                               ("k.b", (G * d,)), ("o.b", (D,)))}
    h = torch.randn(8, D, generator=g, dtype=F)
    full = pk.sink_attention(h, _w(W), m, 1e-6)
    # the first token sees itself: weight e^s / (1 + e^s) on its own projected key (not normed, not rotated)
    kraw = (h[0] @ W["k"].T + W["k.b"]).view(G, d)
    q0 = pk.rms_norm((h[0] @ W["q"].T + W["q.b"]).view(H, d), None, 1e-6)                  # position 0: no turn
    k0 = pk.rms_norm(kraw, None, 1e-6)
    rows = []
    for hd in range(H):
        s = float(q0[hd] @ k0[hd // 2]) * 0.9
        rows.append(math.exp(s) / (1.0 + math.exp(s)) * kraw[hd // 2])
    assert torch.allclose(full[0], torch.cat(rows) @ W["o"].T + W["o.b"], atol=1e-12)
    # a window never reached equals a causal mask; one position narrower differs
    wide, wider = dict(m, mask={"size": 8}), dict(m, mask={"size": 800})
    assert torch.allclose(pk.sink_attention(h, _w(W), wide, 1e-6), pk.sink_attention(h, _w(W), wider, 1e-6), atol=1e-12)
    assert not torch.allclose(pk.sink_attention(h, _w(W), dict(m, mask={"size": 2}), 1e-6)[2:], full[2:], atol=1e-6)


def test_choice_of_experts_by_groups():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([2.0, -3.0, 1.0, 1.1, 0.5, 0.6], dtype=F)
    none = torch.zeros(6, dtype=F)
    # worth: group 0 = s(2) + s(-3), group 1 = s(1) + s(1.1), group 2 = s(.5) + s(.6): group 1 wins although expert 0 is the best
    chosen, wt = pk.choose_experts(z, none, r)
    assert sorted(chosen.tolist()) == [2, 3] and torch.allclose(wt.sort().values, torch.sigmoid(z[[2, 3]]).sort().values)
    # a correction steers the choice and leaves the weights alone; it may be negative (a group left out counts as minus infinity, not 0)
    corr = torch.tensor([0.0, 0.0, -5.0, -5.0, -2.0, -2.0], dtype=F)
    chosen, wt = pk.choose_experts(z, corr, r)
    assert sorted(chosen.tolist()) == [0, 1] and torch.allclose(wt.sort().values, torch.sigmoid(z[[0, 1]]).sort().values)
    corr = torch.tensor([-9.0, -9.0, -5.0, -5.0, -2.0, -2.0], dtype=F)
    chosen, _ = pk.choose_experts(z, corr, r)
    assert sorted(chosen.tolist()) == [4, 5]
    # all groups kept, or no groups: the plain top of the choice values
    for router in ({"experts": 6, "top": 3, "groups": {"count": 3, "keep": 3}}, {"experts": 6, "top": 3}):
        chosen, _ = pk.choose_experts(z, none, router)
        assert sorted(chosen.tolist()) == [0, 2, 3]


def test_clamped_expert_and_forced_choice():
    g = torch.Generator().manual_seed(4)
    h = torch.randn(3, 5, generator=g, dtype=F) * 3
    gate, up, down = (torch.randn(s, generator=g, dtype=F) for s in ((4, 5), (4, 5), (5, 4)))
    y = pk.clamped_expert(h, gate, up, down, 0.5)
    gg, uu = (h @ gate.T).clamp(max=0.5), (h @ up.T).clamp(-0.5, 0.5)
    assert torch.allclose(y, (gg / (1 + torch.exp(-1.702 * gg)) * (uu + 1)) @ down.T, atol=1e-12)
    assert bool((gg == 0.5).any()) and bool((uu == -0.5).any())             # the limits are met by these inputs


def _folder(cfg):
    from kitodra_helpers import make_folder
    with tempfile.TemporaryDirectory() as tmp:
        return make_folder(tmp, cfg, seed=1, init_std=0.3)


def test_forced_experts_equal_to_the_chosen_change_nothing_and_layers_share_tensors():
    cfg, weights = _folder(kc.get("T1"))
    toks = [3, 50, 50, 7, 200, 13, 13, 13, 99, 4, 8, 150, 6]
    a = pk.forward(cfg, weights, toks)
    chosen = dict(pk.forward.chosen)
    assert sorted(chosen) == [0, 1, 2, 3, 4] and chosen[0].shape == (13, 2) and chosen[1].shape == (13, 4)
    assert torch.allclose(pk.forward(cfg, weights, toks, forced=chosen), a, atol=1e-12)
    # layers 3 and 4 run with the tensors of 1 and 0: written out as layers of their own they give the same model
    own = kc.get("T1")
    extra = {}
    for i, j in ((3, 1), (4, 0)):
        own["layers"][i].pop("weights_of")
        extra.update({f"l{i}." + n[len(f"l{j}."):]: w for n, w in weights.items() if n.startswith(f"l{j}.")})
    assert torch.allclose(pk.forward(own, {**weights, **extra}, toks), a, atol=1e-12)
    # the token before matters: the same token after another one gives another row of the pair table
    b = pk.forward(cfg, weights, [3, 51] + toks[2:])
    assert not torch.allclose(a[2], b[2], atol=1e-6)
    # a prompt's first token takes the table's last row
    alone = pk.forward(cfg, weights, toks[:1])
    x = weights["embed"][3].double() + weights["bigram"][-1].double()
    assert torch.allclose(alone[0], a[0], atol=1e-12) and float(x.abs().sum()) > 0

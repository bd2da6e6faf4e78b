"""Sigusun on the host: configuration, declared tensors, caches and states, stored names, and the plain implementation's
own pieces against each other (no GPU)."""
import tempfile

import pytest
import torch

import plain_sigusun
import sigusun_configs as sc
from quench6k_b200.config.pedotar import ConfigError
from quench6k_b200.config.registry import architecture_of
from quench6k_b200.config.sigusun import SigusunConfig
from quench6k_b200.models.decoder import DecoderModel
from quench6k_b200.models.sigusun import build_spec, stored_name


@pytest.mark.parametrize("name", sorted(sc.ALL))
def test_config_round_trip(name):
    d = sc.get(name)
    cfg = SigusunConfig.from_dict(d)
    assert SigusunConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    spec = build_spec(cfg)
    assert spec.order == list(range(len(d["layers"]))) and spec.head_name == "head"
    assert spec.kv_source == [L["mixer"].get("kv_from") if L["type"] != "retention" else None for L in d["layers"]]
    assert architecture_of(d).name == "Sigusun" and architecture_of({"architectures": ["sigusun"]}).name == "Sigusun"


def test_config_errors_name_the_key():
    def broken(name, change, match):
        d = sc.get(name)
        change(d)
        with pytest.raises(ConfigError, match=match):
            SigusunConfig.from_dict(d)

    broken("G1", lambda d: d["layers"][1]["mixer"].pop("scale"), "scale")
    broken("G1", lambda d: d["layers"][0]["mixer"]["decay"].pop(), "decay")
    broken("G1", lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18), "rotating")
    broken("G1", lambda d: d["layers"][1]["mixer"].pop("mask"), "mask")
    broken("G1", lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "top")
    broken("G1", lambda d: d["layers"][2]["mixer"].update(kv_from=2), "kv_from")
    broken("G1", lambda d: d["layers"][2]["mixer"].update(kv_from=0), "kv_from")            # a retention layer caches no keys
    broken("G1", lambda d: d["layers"][2]["mixer"].update(kv_rank=16), "kv_rank")           # differs from the layer it reads
    broken("G2", lambda d: d["layers"][4]["mixer"].update(kv_from=1), "kv_from")            # that layer borrows its keys itself
    broken("G1", lambda d: d.pop("norm"), "norm")
    broken("G1", lambda d: d["layers"][0].update(type="attention"), "type")
    broken("G1", lambda d: d["layers"][0]["mlp"].pop("expert"), "expert")


def test_declared_tensors_caches_and_states():
    cfg = SigusunConfig.from_dict(sc.get("G1"))
    model = DecoderModel(build_spec(cfg))
    names = {t.name: tuple(t.shape) for t in model.tensors()}
    assert names["embed"] == (211, 96) and names["embed.norm"] == (96,) and names["final.norm"] == (96,) and names["head"] == (211, 96)
    assert names["side.embed"] == (211, 4 * 5)
    assert names["l0.mix.q"] == (48, 96) and names["l0.mix.v"] == (72, 96) and names["l0.mix.g"] == (72, 96) and names["l0.mix.o"] == (96, 72)
    assert names["l0.mlp.router"] == (5, 96) and names["l0.mlp.experts.gate"] == (5, 40, 96) and names["l0.mlp.experts.down"] == (5, 96, 40)
    assert names["l0.mlp.shared.up"] == (24, 96) and "l1.mlp.shared.up" not in names
    assert names["l0.side.gate"] == (5, 96) and names["l0.side.proj"] == (96, 5) and names["l0.side.norm"] == (96,)
    assert names["l1.mix.q"] == (4 * 20, 96) and names["l1.mix.dkv"] == (24 + 12, 96) and names["l1.mix.dkv.norm"] == (24,)
    assert names["l1.mix.uk"] == (32, 24) and names["l1.mix.uv"] == (40, 24) and names["l1.mix.o"] == (96, 40)
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names and names["l2.mix.uv"] == (32, 24)
    assert names["l3.mix.sink"] == (3,) and "l1.mix.sink" not in names
    assert "l3.norm1" in names and "l3.norm2" not in names                  # no feed-forward, no second norm
    assert stored_name("l0.mlp.e3.up") == ("l0.mlp.experts.up", 3) and stored_name("l12.mlp.e10.gate") == ("l12.mlp.experts.gate", 10)
    assert stored_name("l0.mlp.shared.gate") is None and stored_name("l0.mlp.router") is None
    assert model.state_shapes()[0] == {"S": ((3, 16, 24), torch.float32)}
    reqs = model.cache_requests()
    # layer 1's keys are read under its own window of 7 and layer 2's of 19: they are kept for the wider one
    assert reqs[0] is None and reqs[1].kind == "sliding" and reqs[1].window == 19 and reqs[2] is None and reqs[3].kind == "full"
    assert cfg.readers(1) == [2] and cfg.kept_window(1) == 19 and cfg.kept_window(3) is None
    g2 = SigusunConfig.from_dict(sc.get("G2"))
    assert g2.kept_window(0) is None and g2.kept_window(3) is None            # a causal layer reads them: every key is kept


def _folder(cfg):
    from sigusun_helpers import make_folder
    with tempfile.TemporaryDirectory() as tmp:
        return make_folder(tmp, cfg, seed=1, init_std=0.3)


def test_plain_pieces_agree_with_each_other():
    """Rotation keeps lengths and turns by the angle it says; retention's first two tokens in closed form; a window that
    is never reached equals none; a sink of minus infinity equals none and a large one silences the head; forced experts
    equal to the router's own choice change nothing; the clamp holds."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.arange(5)
    for neighbours in (False, True):
        y = plain_sigusun.rotate(x, pos, 6, 10.0, neighbours)
        assert torch.allclose(y[0], x[0]) and torch.allclose(y[..., 6:], x[..., 6:])
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
        a, b = (0, 1) if neighbours else (0, 3)
        turned = torch.atan2(y[3, 0, b], y[3, 0, a]) - torch.atan2(x[3, 0, b], x[3, 0, a])
        assert abs(float(torch.remainder(turned - 3.0 + 3.14159265, 2 * 3.14159265358979)) - 3.14159265) < 1e-6

    cfg, weights = _folder(sc.one_layer(sc.retention(2, 8, 6, [0.5, 1.0], 4, 50.0)))
    W = {k: v.double() for k, v in weights.items()}
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(2, cfg["width"], generator=g, dtype=torch.float64)
    w = lambda n: W[f"l0.mix.{n}"]
    got = plain_sigusun.retention(h, w, m, 1e-5)
    q = plain_sigusun.rotate((h @ w("q").T).view(2, 2, 8), torch.arange(2), 4, 50.0, False)
    k = plain_sigusun.rotate((h @ w("k").T).view(2, 2, 8), torch.arange(2), 4, 50.0, False) * 8 ** -0.5
    v = (h @ w("v").T).view(2, 2, 6)
    o = torch.stack([(q[1, i] @ k[1, i]) * v[1, i] + d * (q[1, i] @ k[0, i]) * v[0, i] for i, d in enumerate((0.5, 1.0))])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)
    want = (o.reshape(12) * plain_sigusun.silu(h[1] @ w("g").T)) @ w("o").T
    assert torch.allclose(got[1], want)

    cfg, weights = _folder(sc.one_layer(sc.sink(2, 8, 4, 6, 12, 0.5, 100.0)))
    toks = [3, 9, 27, 5, 5, 40, 11]
    a = plain_sigusun.forward(cfg, weights, toks)
    quiet = dict(weights, **{"l0.mix.sink": torch.full((2,), -1e4)})
    as_window = sc.one_layer(sc.window(2, 8, 4, 6, 12, 0.5, 1000, 100.0))
    assert torch.allclose(plain_sigusun.forward(cfg, quiet, toks), plain_sigusun.forward(as_window, weights, toks))
    assert not torch.allclose(a, plain_sigusun.forward(cfg, quiet, toks))
    W = {k: v.double() for k, v in weights.items()}
    x = plain_sigusun.rms_norm(W["embed"][torch.tensor(toks)], W["embed.norm"], cfg["norm"]["eps"])
    m = cfg["layers"][0]["mixer"]
    w = lambda n: W[f"l0.mix.{n}"]
    kv = plain_sigusun.latent_keys(x, w, m, 1e-5)
    loud = plain_sigusun.latent_attention(x, w, m, 1e-5, kv, sink=torch.tensor([60.0, 60.0], dtype=torch.float64))
    assert float(loud.abs().max()) < 1e-12

    cfg, weights = _folder(sc.one_layer(sc.retention(2, 8, 8, [0.9, 0.9], 4, 50.0, ff=(4, 2, 12, 0.6, 8, 0.3))))
    a = plain_sigusun.forward(cfg, weights, toks)
    chosen = dict(plain_sigusun.forward.chosen)
    assert torch.equal(a, plain_sigusun.forward(cfg, weights, toks, forced=chosen))
    assert not torch.allclose(a, plain_sigusun.forward(cfg, weights, toks, forced={0: (chosen[0] + 1) % 4}))
    hh = torch.randn(3, 5, generator=g, dtype=torch.float64) * 10
    eye = torch.eye(5, dtype=torch.float64)
    y = plain_sigusun.clamped_expert(hh, eye, eye, eye, 0.7)
    gg, uu = hh.clamp(max=0.7), hh.clamp(-0.7, 0.7)
    assert torch.allclose(y, gg * torch.sigmoid(1.702 * gg) * (uu + 1))
    streams = []
    plain_sigusun.forward(cfg, weights, toks, layers_out=streams)
    assert len(streams) == 1 and streams[0].shape == (len(toks), cfg["width"])

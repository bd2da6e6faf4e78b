"""Sigusun: from its typed configuration to the architecture-neutral ModelSpec.

A decoder whose layers each name their own mixer: retention (linear attention with a fixed decay per head, a matrix-valued
state per head and request, rotated q and k), or attention over a cached low-rank latent with one rotated key part shared
by the heads, either in a sliding window or causal with a learned sink per head; a latent layer may read the latent
another layer cached instead of making its own.  The feed-forward is a mixture of experts with a clamped gate
(g' = min(g, L), u' = clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1)), the weights a softmax over the chosen logits, plus
a shared expert of the same form.  Each sublayer reads the stream itself and its result passes an RMS norm before it is
added: x += norm1(mixer(x)); x += norm2(ff(x)).  After the feed-forward every layer takes a per-layer token input: with e
the layer's columns of the token's row of a side table, x += rms(side.proj (gelu_tanh(side.gate x) * e)) * side.norm.
The embedding output passes a norm; the head is a matrix of its own.

Tensor names: `embed`, `embed.norm`, `side.embed`, `final.norm`, `head`, and per layer i `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.<name>`, `l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down}}`, `l<i>.side.{gate,proj,norm}`.
"""
from __future__ import annotations

import re

from ..config.registry import register_architecture
from ..config.sigusun import ARCHITECTURE, SigusunConfig
from ..spec import LayerSpec, ModelSpec, PartSpec

_RETENTION_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o"}
_LATENT_NAMES = {"q": "q", "dkv": "dkv", "c_norm": "dkv.norm", "uk": "uk", "uv": "uv", "out": "o", "sinks": "sink"}
_MOE_NAMES = {"router": "router", "gate": "experts.gate", "up": "experts.up", "down": "experts.down"}
_SHARED_NAMES = {"gate": "gate", "up": "up", "down": "down"}
_SIDE_NAMES = {"gate": "gate", "proj": "proj", "norm": "norm"}

# experts are stored one by one and stacked as they are read
_ONE_EXPERT = re.compile(r"^(l\d+\.mlp)\.e(\d+)\.(gate|up|down)$")


def stored_name(name: str):
    m = _ONE_EXPERT.match(name)
    return (f"{m.group(1)}.experts.{m.group(3)}", int(m.group(2))) if m else None


_UNUSED_NORM = re.compile(r"^l\d+\.norm2$")      # a layer without a feed-forward has no use for its second norm


def _rotation(dim: int, rot: dict, pairing: str) -> PartSpec:
    if rot["dims"] > 0:
        return PartSpec("rope", {"head_dim": dim, "theta": rot["base"], "rotary_dim": rot["dims"], "pairing": pairing})
    return PartSpec("none", {"head_dim": dim})


def _mixer(cfg: SigusunConfig, i: int, norm_init: str) -> PartSpec:
    L = cfg.layers[i]
    kind, m, eps = L["type"], L["mixer"], cfg.norm_eps
    if kind == "retention":
        return PartSpec("retention", {"num_heads": m["heads"], "head_dim": m["dim"], "v_dim": m["vdim"], "decay": list(m["decay"]), "eps": eps,
                                      "pos": _rotation(m["dim"], m["rot"], "halves"), "names": _RETENTION_NAMES})
    borrows = m.get("kv_from") is not None
    return PartSpec("latent_attention", {
        "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_dim": m["vdim"], "kv_rank": m["kv_rank"],
        "scale": m["scale"], "eps": eps, "pos": _rotation(max(m["rot_dim"], 1), m["rot"], "neighbours"), "names": _LATENT_NAMES,
        "norm_init": norm_init, "window": m["mask"]["size"] if kind == "latent_attention" else None, "sinks": kind == "latent_attention_2",
        "borrows": borrows, "retain": None if borrows else cfg.kept_window(i)})


def _ffn(mlp):
    if mlp is None:
        return None
    r, shared = mlp["router"], mlp.get("shared")
    params = {"num_experts": r["experts"], "top_k": r["top"], "intermediate_size": mlp["expert"]["ff"], "scoring": "softmax",
              "renormalize": True, "gated": True, "act": ("clamped", mlp["expert"]["limit"]), "names": _MOE_NAMES}
    if shared is not None:
        params.update(shared_intermediate_size=shared["ff"], shared_act=("clamped", shared["limit"]), shared_prefix="shared.",
                      shared_names=_SHARED_NAMES)
    return PartSpec("moe", params)


def build_spec(cfg: SigusunConfig, norm_init: str = "ones") -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps, "init": norm_init, "weight_name": ""})
    layers = []
    for i, L in enumerate(cfg.layers):
        side = (PartSpec("token_side", {"dim": cfg.side_dim, "column": i * cfg.side_dim, "eps": cfg.norm_eps, "names": _SIDE_NAMES,
                                        "norm_init": norm_init}) if cfg.side_dim else None)
        layers.append(LayerSpec(prefix=f"l{i}.", mixer=_mixer(cfg, i, norm_init), ffn=_ffn(L.get("mlp")), norm=norm, block="outnorm", side=side))
    n = len(layers)
    kv_source = [L["mixer"].get("kv_from") if L["type"] != "retention" else None for L in cfg.layers]
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, order=list(range(n)), kv_source=kv_source,
                     final_norm=norm, embed_name="embed", head_name="head", final_norm_prefix="final.norm",
                     eos_token_ids=tuple(cfg.eos_token_id), name_alias=stored_name, ignorable=lambda name: bool(_UNUSED_NORM.match(name)),
                     sub_names={"norm1": "norm1", "norm2": "norm2", "mixer": "mix.", "ffn": "mlp.", "side": "side."},
                     embed_norm=norm, embed_norm_prefix="embed.norm",
                     side_table=("side.embed", n * cfg.side_dim) if cfg.side_dim else None)


register_architecture(ARCHITECTURE, SigusunConfig, build_spec, aliases=("sigusun",))

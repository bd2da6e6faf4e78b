"""Kitodra: from its typed configuration to the architecture-neutral ModelSpec.

A decoder whose layers each name their own mixer: "lightning" (linear attention with one fixed decay per head on
silu-activated q, k and v, all heads' results normed together and gated by a sigmoid), "attention" (difference attention:
two softmax maps per head over the same values inside chunks of positions, capped scores, normed q and k, no positions)
or "attention_2" (a sliding window with one extra term of score zero in the softmax denominator, a partial rotation by
halves, q and k divided by their root mean square, the values being the projected keys).  Mixer and feed-forward read the
same normed stream and are added together: x += mixer(norm1(x)) + ff(norm1(x)).  The feed-forward is a mixture of experts
with a clamped gate, sigmoid scores (a stored correction steers the choice only, the choice is limited to the best
groups of experts, the weights are the plain scores) and a shared expert.  A token-pair table is added to the embedding;
a layer may run with another layer's tensors on a cache and state of its own; the head is the embedding table.

Tensor names: `embed`, `bigram`, `final.norm`, and per layer i with tensors of its own `l<i>.norm1`, `l<i>.mix.<name>`,
`l<i>.mlp.{router, correction, e<j>.{gate,up,down}, shared.{gate,up,down}}`.
"""
from __future__ import annotations

import re

from ..config.kitodra import ARCHITECTURE, KitodraConfig
from ..config.registry import register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec

_LIGHTNING_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm"}
_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
                    "q_norm": "q.norm", "k_norm": "k.norm", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
_MOE_NAMES = {"router": "router", "correction": "correction", "gate": "experts.gate", "up": "experts.up", "down": "experts.down"}
_SHARED_NAMES = {"gate": "gate", "up": "up", "down": "down"}

# experts are stored one by one and stacked as they are read
_ONE_EXPERT = re.compile(r"^(l\d+\.mlp)\.e(\d+)\.(gate|up|down)$")


def stored_name(name: str):
    m = _ONE_EXPERT.match(name)
    return (f"{m.group(1)}.experts.{m.group(3)}", int(m.group(2))) if m else None


def _mixer(kind: str, m: dict, eps: float, norm_init: str) -> PartSpec:
    if kind == "lightning":
        return PartSpec("retention", {"num_heads": m["heads"], "head_dim": m["dim"], "v_dim": m["vdim"], "decay": list(m["decay"]), "eps": eps,
                                      "pos": PartSpec("none", {"head_dim": m["dim"]}), "k_scale": 1.0, "act": "silu", "out_norm": "all_heads",
                                      "gate": "sigmoid", "norm_init": norm_init, "names": _LIGHTNING_NAMES})
    common = {"num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"], "eps": eps, "scale": m["scale"],
              "bias": True, "o_bias": True, "qk_norm": True, "norm_init": norm_init, "names": _ATTENTION_NAMES}
    if kind == "attention":
        return PartSpec("attention", {**common, "pos": PartSpec("none", {"head_dim": m["dim"]}), "chunk": m["mask"]["size"],
                                      "softcap": m["softcap"], "maps": 2, "diff": m["diff"]})
    if kind == "attention_2":
        turn = m["rot"]["dims"]
        pos = (PartSpec("rope", {"head_dim": m["dim"], "theta": m["rot"]["base"], "rotary_dim": turn, "pairing": "halves"}) if turn > 0
               else PartSpec("none", {"head_dim": m["dim"]}))
        return PartSpec("attention", {**common, "pos": pos, "window": m["mask"]["size"], "fixed_sink": 0.0, "qk_norm_weight": False,
                                      "values_are_keys": True})
    raise ValueError(f"unknown mixer type {kind!r}")


def _ffn(mlp):
    if mlp is None:
        return None
    r, shared, groups = mlp["router"], mlp.get("shared"), mlp["router"].get("groups")
    params = {"num_experts": r["experts"], "top_k": r["top"], "intermediate_size": mlp["expert"]["ff"], "scoring": "sigmoid",
              "renormalize": False, "gated": True, "act": ("clamped", mlp["expert"]["limit"]), "correction": True, "names": _MOE_NAMES,
              "groups": (groups["count"], groups["keep"]) if groups is not None else None}
    if shared is not None:
        params.update(shared_intermediate_size=shared["ff"], shared_act=("clamped", shared["limit"]), shared_prefix="shared.",
                      shared_names=_SHARED_NAMES)
    return PartSpec("moe", params)


def build_spec(cfg: KitodraConfig, norm_init: str = "ones") -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps, "init": norm_init, "weight_name": ""})
    own = [i for i, L in enumerate(cfg.layers) if L.get("weights_of") is None]        # layers with tensors of their own
    layers = [LayerSpec(prefix=f"l{i}.", mixer=_mixer(cfg.layers[i]["type"], cfg.layers[i]["mixer"], cfg.norm_eps, norm_init),
                        ffn=_ffn(cfg.layers[i].get("mlp")), norm=norm, block="parallel", shared_norm=True) for i in own]
    order = [own.index(cfg.weights_layer(i)) for i in range(len(cfg.layers))]          # every position runs on a cache and state of its own
    bg = cfg.bigram
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, order=order, kv_source=[None] * len(order),
                     final_norm=norm, embed_name="embed", head_name=None, final_norm_prefix="final.norm",
                     eos_token_ids=tuple(cfg.eos_token_id), name_alias=stored_name,
                     sub_names={"norm1": "norm1", "norm2": "norm2", "mixer": "mix.", "ffn": "mlp."},
                     embed_add=PartSpec("token_pair", {"buckets": bg["buckets"], "mul_prev": bg["mul_prev"], "mul_cur": bg["mul_cur"], "name": ""})
                     if bg is not None else None, embed_add_prefix="bigram")


register_architecture(ARCHITECTURE, KitodraConfig, build_spec, aliases=("kitodra",))

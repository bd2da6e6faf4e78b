"""Typed configuration of the Kitodra decoder, read from config.json.

    {"architecture": "Kitodra", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "lightning" | "attention" | "attention_2", "mixer": {...}, "mlp": {...} | null, "weights_of": j}, ...]}

Every size and constant comes from the file; the layer list gives each layer's mixer and feed-forward with their own
sizes, so no two layers need agree on anything.  A layer with `weights_of: j` has no tensors of its own: it runs as
layer j does (that layer's mixer, feed-forward, norm, sizes and constants), on a cache and state of its own.  Mixer keys by type:
  lightning:    heads, dim, vdim, decay [heads]
  attention:    heads, kv_heads, dim, vdim, scale, softcap, diff, mask {size}          (two maps per head, chunks)
  attention_2:  heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims}       (window, values are the keys)
Feed-forward (kind "moe"): expert {ff, limit}, router {experts, top, groups {count, keep}}, shared {ff, limit} (optional).
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .pedotar import ConfigError

ARCHITECTURE = "Kitodra"

_MIXER_KEYS = {
    "lightning": ("heads", "dim", "vdim", "decay"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "diff", "mask"),
    "attention_2": ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"),
}


@dataclass
class KitodraConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[Dict[str, Any]]
    bigram: Optional[Dict[str, int]] = None   # {"buckets", "mul_prev", "mul_cur"}; None: no token-pair embedding
    eos_token_id: List[int] = field(default_factory=list)
    kv_page_size: Optional[int] = None       # engine-side hint, not a model size
    architectures: List[str] = field(default_factory=lambda: [ARCHITECTURE])

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KitodraConfig":
        missing = [k for k in ("vocab", "width", "norm", "layers") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config.json: 'norm' must hold 'eps'")
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        eos = d.get("eos_token_id") or []
        cfg = cls(vocab=d["vocab"], width=d["width"], norm_eps=float(d["norm"]["eps"]), layers=copy.deepcopy(d["layers"]),
                  bigram=copy.deepcopy(emb.get("bigram")), eos_token_id=[int(x) for x in ([eos] if isinstance(eos, int) else eos)],
                  kv_page_size=d.get("kv_page_size"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "KitodraConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                               "layers": copy.deepcopy(self.layers)}
        if self.bigram is not None:
            out["embedding"] = {"bigram": dict(self.bigram)}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        if self.kv_page_size is not None:
            out["kv_page_size"] = self.kv_page_size
        return out

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=1)

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        def need(cond: bool, msg: str) -> None:
            if not cond:
                raise ConfigError(msg)

        def positive(v) -> bool:
            return isinstance(v, int) and not isinstance(v, bool) and v > 0

        def number(v) -> bool:
            return isinstance(v, (int, float)) and not isinstance(v, bool)

        need(positive(self.vocab) and positive(self.width), f"vocab {self.vocab!r} and width {self.width!r} must be positive integers")
        need(self.norm_eps > 0, "norm.eps must be positive")
        if self.bigram is not None:
            b = self.bigram
            need(isinstance(b, dict) and positive(b.get("buckets")), "embedding.bigram.buckets must be a positive integer")
            for k in ("mul_prev", "mul_cur"):
                need(isinstance(b.get(k), int) and not isinstance(b.get(k), bool) and b[k] >= 0, f"embedding.bigram.{k} must be a non-negative integer")
        need(isinstance(self.layers, list) and len(self.layers) > 0, "layers must be a non-empty list")
        for i, L in enumerate(self.layers):
            need(isinstance(L, dict) and L.get("type") in _MIXER_KEYS, f"layer {i}: type {L.get('type') if isinstance(L, dict) else L!r} is none of "
                 + ", ".join(_MIXER_KEYS))
            m = L.get("mixer")
            need(isinstance(m, dict), f"layer {i}: 'mixer' must hold the mixer's sizes")
            lacking = [k for k in _MIXER_KEYS[L["type"]] if k not in m]
            need(not lacking, f"layer {i} ({L['type']}): mixer lacks " + ", ".join(lacking))
            for k in ("heads", "dim", "vdim"):
                need(positive(m[k]), f"layer {i}: mixer.{k} must be a positive integer, got {m[k]!r}")
            if L["type"] == "lightning":
                need(isinstance(m["decay"], list) and len(m["decay"]) == m["heads"] and all(number(x) and 0 <= x <= 1 for x in m["decay"]),
                     f"layer {i}: mixer.decay must hold one number in 0..1 per head")
            else:
                need(positive(m["kv_heads"]) and m["heads"] % m["kv_heads"] == 0,
                     f"layer {i}: {m['heads']} heads are not a multiple of {m['kv_heads']!r} kv_heads")
                need(number(m["scale"]) and m["scale"] > 0, f"layer {i}: mixer.scale must be a positive number")
                need(isinstance(m["mask"], dict) and positive(m["mask"].get("size")), f"layer {i}: mixer.mask.size must be a positive integer")
            if L["type"] == "attention":
                need(number(m["softcap"]) and m["softcap"] > 0, f"layer {i}: mixer.softcap must be a positive number")
                need(number(m["diff"]), f"layer {i}: mixer.diff must be a number")
            if L["type"] == "attention_2":
                need(m["vdim"] == m["dim"], f"layer {i}: the values are the keys, so vdim {m['vdim']} must equal dim {m['dim']}")
                rot = m["rot"]
                need(isinstance(rot, dict) and "base" in rot and "dims" in rot, f"layer {i}: mixer.rot must hold base and dims")
                need(isinstance(rot["dims"], int) and rot["dims"] % 2 == 0 and 0 <= rot["dims"] <= m["dim"],
                     f"layer {i}: {rot['dims']!r} rotating dimensions of a head of {m['dim']}")
                need(number(rot["base"]) and rot["base"] > 0, f"layer {i}: mixer.rot.base must be positive")
            mlp = L.get("mlp")
            if mlp is not None:
                need(isinstance(mlp, dict) and mlp.get("kind", "moe") == "moe", f"layer {i}: mlp must be null or of kind moe, got {mlp!r}")
                ex, ro, sh = mlp.get("expert"), mlp.get("router"), mlp.get("shared")
                need(isinstance(ex, dict) and positive(ex.get("ff")) and number(ex.get("limit")), f"layer {i}: mlp.expert must hold ff and limit")
                need(isinstance(ro, dict) and positive(ro.get("experts")) and positive(ro.get("top")), f"layer {i}: mlp.router must hold experts and top")
                need(ro["top"] <= ro["experts"], f"layer {i}: top {ro['top']} of {ro['experts']} experts")
                gr = ro.get("groups")
                if gr is not None:
                    need(isinstance(gr, dict) and positive(gr.get("count")) and positive(gr.get("keep")), f"layer {i}: mlp.router.groups must hold count and keep")
                    need(ro["experts"] % gr["count"] == 0 and gr["keep"] <= gr["count"],
                         f"layer {i}: {ro['experts']} experts in {gr['count']} groups, {gr['keep']} kept")
                    need(ro["top"] <= gr["keep"] * (ro["experts"] // gr["count"]),
                         f"layer {i}: top {ro['top']} exceeds the {gr['keep']} kept groups' experts")
                if sh is not None:
                    need(isinstance(sh, dict) and positive(sh.get("ff")) and number(sh.get("limit")), f"layer {i}: mlp.shared must hold ff and limit")
            j = L.get("weights_of")
            if j is not None:
                need(isinstance(j, int) and not isinstance(j, bool) and 0 <= j < len(self.layers) and j != i, f"layer {i}: weights_of {j!r} names no other layer")
        for i, L in enumerate(self.layers):
            if L.get("weights_of") is not None:
                j = self.weights_layer(i)
                need(self.layers[j].get("weights_of") is None, f"layer {i}: weights_of runs in a circle")
                need(self.layers[j]["type"] == L["type"], f"layer {i} uses layer {j}'s tensors but differs from it in type")
        for t in self.eos_token_id:
            need(0 <= t < self.vocab, f"eos_token_id {t} outside the vocabulary")
        if self.kv_page_size is not None:
            need(positive(self.kv_page_size), "kv_page_size must be a positive integer")

    # ------------------------------------------------------------------ derived
    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs with (itself, unless it names another)."""
        for _ in range(len(self.layers)):
            j = self.layers[i].get("weights_of")
            if j is None:
                return i
            i = j
        return i

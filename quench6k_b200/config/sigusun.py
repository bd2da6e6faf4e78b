"""Typed configuration of the Sigusun decoder, read from config.json.

    {"architecture": "Sigusun", "vocab": V, "width": D, "norm": {"eps": e}, "token_side": {"dim": s} | absent,
     "layers": [{"type": "retention" | "latent_attention" | "latent_attention_2", "mixer": {...}, "mlp": {...} | null}, ...]}

Every size and constant comes from the file; the layer list gives each layer's mixer and feed-forward with their own
sizes, so no two layers need agree on anything.  Mixer keys by type:
  retention:           heads, dim, vdim, decay [heads], rot {base, dims}
  latent_attention:    heads, dim, rot_dim, vdim, kv_rank, scale, mask {size}, rot {base, dims}, kv_from (optional)
  latent_attention_2:  heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, kv_from (optional)
Feed-forward (kind "moe"): expert {ff, limit}, router {experts, top}, shared {ff, limit} (optional).
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .pedotar import ConfigError

ARCHITECTURE = "Sigusun"

_LATENT = ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot")
_MIXER_KEYS = {
    "retention": ("heads", "dim", "vdim", "decay", "rot"),
    "latent_attention": _LATENT + ("mask",),
    "latent_attention_2": _LATENT,
}


@dataclass
class SigusunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[Dict[str, Any]]
    side_dim: int = 0                        # columns of the per-layer token input (0: the model has none)
    eos_token_id: List[int] = field(default_factory=list)
    kv_page_size: Optional[int] = None       # engine-side hint, not a model size
    architectures: List[str] = field(default_factory=lambda: [ARCHITECTURE])

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SigusunConfig":
        missing = [k for k in ("vocab", "width", "norm", "layers") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config.json: 'norm' must hold 'eps'")
        side = d.get("token_side")
        if side is not None and not (isinstance(side, dict) and "dim" in side):
            raise ConfigError("config.json: 'token_side' must hold 'dim'")
        eos = d.get("eos_token_id") or []
        cfg = cls(vocab=d["vocab"], width=d["width"], norm_eps=float(d["norm"]["eps"]), layers=copy.deepcopy(d["layers"]),
                  side_dim=side["dim"] if side is not None else 0,
                  eos_token_id=[int(x) for x in ([eos] if isinstance(eos, int) else eos)], kv_page_size=d.get("kv_page_size"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "SigusunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                               "layers": copy.deepcopy(self.layers)}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
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
        need(isinstance(self.side_dim, int) and not isinstance(self.side_dim, bool) and self.side_dim >= 0,
             f"token_side.dim must be a non-negative integer, got {self.side_dim!r}")
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
            rot = m["rot"]
            need(isinstance(rot, dict) and "base" in rot and "dims" in rot, f"layer {i}: mixer.rot must hold base and dims")
            need(number(rot["base"]) and rot["base"] > 0, f"layer {i}: mixer.rot.base must be positive")
            if L["type"] == "retention":
                need(isinstance(m["decay"], list) and len(m["decay"]) == m["heads"] and all(number(x) for x in m["decay"]),
                     f"layer {i}: mixer.decay must list one number per head")
                need(isinstance(rot["dims"], int) and rot["dims"] % 2 == 0 and 0 <= rot["dims"] <= m["dim"],
                     f"layer {i}: {rot['dims']!r} rotating dimensions of a head of {m['dim']}")
            else:
                need(positive(m["kv_rank"]), f"layer {i}: mixer.kv_rank must be a positive integer, got {m['kv_rank']!r}")
                need(isinstance(m["rot_dim"], int) and not isinstance(m["rot_dim"], bool) and m["rot_dim"] >= 0 and m["rot_dim"] % 2 == 0,
                     f"layer {i}: mixer.rot_dim must be an even non-negative integer, got {m['rot_dim']!r}")
                need(rot["dims"] == m["rot_dim"], f"layer {i}: the rotated part has {m['rot_dim']} entries and rot.dims is {rot['dims']!r}")
                need(number(m["scale"]) and m["scale"] > 0, f"layer {i}: mixer.scale must be a positive number")
                if L["type"] == "latent_attention":
                    need(isinstance(m["mask"], dict) and positive(m["mask"].get("size")), f"layer {i}: mixer.mask.size must be a positive integer")
                j = m.get("kv_from")
                if j is not None:
                    need(isinstance(j, int) and not isinstance(j, bool) and 0 <= j < i, f"layer {i}: kv_from {j!r} names no earlier layer")
                    src = self.layers[j]
                    need(src["type"] != "retention" and src["mixer"].get("kv_from") is None,
                         f"layer {i}: kv_from {j} must name a latent attention layer that makes its own keys")
                    sm = src["mixer"]
                    need((sm["kv_rank"], sm["rot_dim"], sm["rot"]["base"], sm["rot"]["dims"]) == (m["kv_rank"], m["rot_dim"], rot["base"], rot["dims"]),
                         f"layer {i}: kv_rank, rot_dim and rot differ from those of layer {j}, whose keys it reads")
            mlp = L.get("mlp")
            if mlp is None:
                continue
            need(isinstance(mlp, dict) and mlp.get("kind", "moe") == "moe", f"layer {i}: mlp must be null or of kind moe, got {mlp!r}")
            ex, ro, sh = mlp.get("expert"), mlp.get("router"), mlp.get("shared")
            need(isinstance(ex, dict) and positive(ex.get("ff")) and number(ex.get("limit")), f"layer {i}: mlp.expert must hold ff and limit")
            need(isinstance(ro, dict) and positive(ro.get("experts")) and positive(ro.get("top")), f"layer {i}: mlp.router must hold experts and top")
            need(ro["top"] <= ro["experts"], f"layer {i}: top {ro['top']} of {ro['experts']} experts")
            need(sh is None or (isinstance(sh, dict) and positive(sh.get("ff")) and number(sh.get("limit"))),
                 f"layer {i}: mlp.shared must be absent or hold ff and limit")
        for t in self.eos_token_id:
            need(0 <= t < self.vocab, f"eos_token_id {t} outside the vocabulary")
        if self.kv_page_size is not None:
            need(positive(self.kv_page_size), "kv_page_size must be a positive integer")

    # ------------------------------------------------------------------ derived
    def readers(self, j: int) -> List[int]:
        """The layers that read layer j's cached keys (kv_from = j)."""
        return [i for i, L in enumerate(self.layers) if L["type"] != "retention" and L["mixer"].get("kv_from") == j]

    def kept_window(self, j: int):
        """How many positions back layer j's cache must reach: the widest window among the layer and its readers, or None
        when one of them sees every earlier position."""
        widest = 0
        for i in [j] + self.readers(j):
            L = self.layers[i]
            if L["type"] != "latent_attention":
                return None
            widest = max(widest, L["mixer"]["mask"]["size"])
        return widest

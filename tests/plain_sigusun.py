"""A plain, slow implementation of the Sigusun decoder from its equations: one function per mechanism, whole sequences
at a time, double precision, loops where a loop is the clearest way to say it.  It shares nothing with the engine (no
part, no kernel, no cache): the tests compare the engine with it.

A model is (config dict, {tensor name: torch tensor}).  Tensor names: `embed`, `embed.norm`, `side.embed`, `final.norm`,
`head`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.side.*`.
"""
import math

import torch

F = torch.float64


# ----------------------------------------------------------------------------- small pieces
def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x, positions, dims, base, neighbours):
    """x [T, heads, n]: the last axis' first `dims` entries turn, pair i by position * base^(-2i/dims).  Pair i is
    (2i, 2i+1) with neighbours, else (i, i + dims/2); (u, v) -> (u cos - v sin, v cos + u sin)."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = (2 * i, 2 * i + 1) if neighbours else (i, i + dims // 2)
        out[..., a] = x[..., a] * c - x[..., b] * s
        out[..., b] = x[..., b] * c + x[..., a] * s
    return out


# ----------------------------------------------------------------------------- mixers (one sequence, positions 0..T-1)
def retention(h, w, m, eps):
    """Linear attention with one fixed decay per head, no softmax and no denominator, token by token:
    S <- decay S + k v^T, o = S^T q."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((h @ w("q").T).view(T, H, dk), pos, m["rot"]["dims"], m["rot"]["base"], neighbours=False)
    k = rotate((h @ w("k").T).view(T, H, dk), pos, m["rot"]["dims"], m["rot"]["base"], neighbours=False) * dk ** -0.5
    v = (h @ w("v").T).view(T, H, dv)
    o = torch.zeros((T, H, dv), dtype=F)
    for head in range(H):
        S = torch.zeros((dk, dv), dtype=F)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_norm(o, None, eps)
    return (o.reshape(T, H * dv) * silu(h @ w("g").T)) @ w("o").T


def latent_keys(h, w, m, eps):
    """What a latent attention layer caches: the normed latent c [T, kv_rank] and the one rotated key part [T, rot_dim]."""
    T, rank, rd = h.shape[0], m["kv_rank"], m["rot_dim"]
    d = h @ w("dkv").T
    c = rms_norm(d[:, :rank], w("dkv.norm"), eps)
    kr = rotate(d[:, None, rank:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"], neighbours=True)[:, 0]
    return c, kr


def latent_attention(h, w, m, eps, kv, window=None, sink=None):
    """Softmax attention whose keys and values are made per head from the cached pair kv = (c, rotated key part).
    window: position i sees j with 0 <= i - j < window (None: every j <= i).  sink [heads]: exp(sink) joins the
    denominator."""
    T = h.shape[0]
    H, dn, rd, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kv
    q = (h @ w("q").T).view(T, H, dn + rd)
    qr = rotate(q[..., dn:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"], neighbours=True)
    kn = (c @ w("uk").T).view(T, H, dn)
    v = (c @ w("uv").T).view(T, H, dv)
    out = torch.zeros((T, H, dv), dtype=F)
    for head in range(H):
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (kn[lo:i + 1, head] @ q[i, head, :dn] + kr[lo:i + 1] @ qr[i, head]) * m["scale"]
            top = s.max() if sink is None else torch.maximum(s.max(), sink[head])
            e = torch.exp(s - top)
            den = e.sum() + (torch.exp(sink[head] - top) if sink is not None else 0.0)
            out[i, head] = (e / den) @ v[lo:i + 1, head]
    return out.reshape(T, H * dv) @ w("o").T


# ----------------------------------------------------------------------------- feed-forward
def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed_experts(h, w, mlp, forced=None):
    """Each token's `top` experts by router logit, weighted by the softmax over the chosen logits; plus the shared
    expert.  forced [T, top]: use these experts instead of choosing.  Returns (result, chosen [T, top])."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w("router").T
    chosen = torch.topk(z, top, dim=-1).indices if forced is None else forced.to(torch.long)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        wt = torch.softmax(z[t, chosen[t]], dim=-1)
        for s in range(top):
            e = int(chosen[t, s])
            out[t] = out[t] + wt[s] * clamped_expert(h[t], w(f"e{e}.gate"), w(f"e{e}.up"), w(f"e{e}.down"), mlp["expert"]["limit"])
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, w("shared.gate"), w("shared.up"), w("shared.down"), mlp["shared"]["limit"])
    return out, chosen


def token_side(x, e, w, eps):
    """The per-layer token input: e [T, dim] is the layer's part of the tokens' side embedding."""
    y = (gelu_tanh(x @ w("gate").T) * e) @ w("proj").T
    return rms_norm(y, w("norm"), eps)


# ----------------------------------------------------------------------------- the model
def forward(cfg, weights, tokens, forced=None, layers_out=None):
    """Logits [T, vocab] of one sequence.  forced: {layer: [T, top]} experts to use in place of the router's choice.
    forward.chosen holds the experts each routed layer chose.  layers_out: a list that receives the stream after every layer."""
    W = {k: v.to(F) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = rms_norm(W["embed"][tok], W["embed.norm"], eps)
    side = cfg.get("token_side")
    cached = {}
    forward.chosen = {}
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        w = lambda n, i=i: W[f"l{i}.mix.{n}"]
        if L["type"] == "retention":
            y = retention(x, w, m, eps)
        elif L["type"] in ("latent_attention", "latent_attention_2"):
            if m.get("kv_from") is not None:
                kv = cached[m["kv_from"]]
            else:
                kv = cached[i] = latent_keys(x, w, m, eps)
            if L["type"] == "latent_attention":
                y = latent_attention(x, w, m, eps, kv, window=m["mask"]["size"])
            else:
                y = latent_attention(x, w, m, eps, kv, sink=w("sink"))
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, W[f"l{i}.norm1"], eps)
        if L.get("mlp") is not None:
            y, forward.chosen[i] = routed_experts(x, lambda n, i=i: W[f"l{i}.mlp.{n}"], L["mlp"], None if forced is None else forced.get(i))
            x = x + rms_norm(y, W[f"l{i}.norm2"], eps)
        if side is not None:
            d = side["dim"]
            x = x + token_side(x, W["side.embed"][tok, i * d:(i + 1) * d], lambda n, i=i: W[f"l{i}.side.{n}"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T

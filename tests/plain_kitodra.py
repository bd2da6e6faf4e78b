"""A plain, slow implementation of the Kitodra decoder from its equations: one function per mechanism, whole sequences
at a time, double precision, loops where a loop is the clearest way to say it.  It shares nothing with the engine (no
part, no kernel, no cache): the tests compare the engine with it.

A model is (config dict, {tensor name: torch tensor}).  Tensor names: `embed`, `bigram`, `final.norm`, and per layer i that
has weights of its own `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`.
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


def rotate_halves(x, positions, dims, base):
    """x [T, heads, n]: the first `dims` entries of the last axis turn; entry i pairs with entry i + dims/2 and the pair
    (u, v) becomes (u cos a - v sin a, v cos a + u sin a), a = position * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        ang = positions.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        out[..., i] = x[..., i] * c - x[..., i + half] * s
        out[..., i + half] = x[..., i + half] * c + x[..., i] * s
    return out


def pair_rows(tokens, bg):
    """The row of the token-pair table for every position: a hash of (token before, token); the table's last row for a
    sequence's first token."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(bg["buckets"] if t == 0 else (int(tokens[t - 1]) * bg["mul_prev"] + int(tok) * bg["mul_cur"]) % bg["buckets"])
    return torch.tensor(rows, dtype=torch.long)


# ----------------------------------------------------------------------------- mixers (one sequence, positions 0..T-1)
def lightning(h, w, m, eps):
    """Linear attention with one fixed decay per head on silu-activated q, k, v, token by token:
    S <- decay S + k v^T, o = S^T q; all heads' results normed as one vector, gated by a sigmoid."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w("q").T).view(T, H, dk)
    k = silu(h @ w("k").T).view(T, H, dk)
    v = silu(h @ w("v").T).view(T, H, dv)
    o = torch.zeros((T, H, dv), dtype=F)
    for head in range(H):
        S = torch.zeros((dk, dv), dtype=F)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    y = rms_norm(o.reshape(T, H * dv), w("norm"), eps) * torch.sigmoid(h @ w("g").T)
    return y @ w("o").T


def difference_weight(w, m):
    """The one number a difference-attention layer multiplies its second map by."""
    return float(torch.exp((w("lq1") * w("lk1")).sum()) - torch.exp((w("lq2") * w("lk2")).sum()) + m["diff"])


def difference_attention(h, w, m, eps):
    """Two softmax attentions per head over the same values, inside chunks of positions, the second subtracted from the
    first; scores capped by a tanh; q and k normed per head and map; no positions."""
    T = h.shape[0]
    H, G, d, dv, C = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]
    q = rms_norm((h @ w("q").T + w("q.b")).view(T, H, 2, d), w("q.norm"), eps)
    k = rms_norm((h @ w("k").T + w("k.b")).view(T, G, 2, d), w("k.norm"), eps)
    v = (h @ w("v").T + w("v.b")).view(T, G, dv)
    lam, cap = difference_weight(w, m), m["softcap"]
    out = torch.zeros((T, H, dv), dtype=F)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            lo = i // C * C
            maps = []
            for a in range(2):
                s = (k[lo:i + 1, g, a] @ q[i, head, a]) * m["scale"]
                s = cap * torch.tanh(s / cap)
                maps.append(torch.softmax(s, dim=0) @ v[lo:i + 1, g])
            o = maps[0] - lam * maps[1]
            out[i, head] = rms_norm(o, None, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * dv) @ w("o").T + w("o.b")


def sink_attention(h, w, m, eps, sink=True):
    """Softmax attention in a sliding window whose denominator holds one more term of score zero.  There is no value
    projection: what the weights are applied to is the key projection's raw result.  q and k turn over their first dims
    entries and are then brought to unit root mean square.  sink=False leaves the extra term out (for tests that ask
    whether it would show)."""
    T = h.shape[0]
    H, G, d, win = m["heads"], m["kv_heads"], m["dim"], m["mask"]["size"]
    pos = torch.arange(T)
    q = (h @ w("q").T + w("q.b")).view(T, H, d)
    k = (h @ w("k").T + w("k.b")).view(T, G, d)
    v = k.clone()
    q = rms_norm(rotate_halves(q, pos, m["rot"]["dims"], m["rot"]["base"]), None, eps)
    k = rms_norm(rotate_halves(k, pos, m["rot"]["dims"], m["rot"]["base"]), None, eps)
    out = torch.zeros((T, H, v.shape[-1]), dtype=F)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            lo = max(0, i - win + 1)
            s = (k[lo:i + 1, g] @ q[i, head]) * m["scale"]
            top = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - top)
            out[i, head] = (e / (e.sum() + (torch.exp(-top) if sink else 0.0))) @ v[lo:i + 1, g]
    return out.reshape(T, -1) @ w("o").T + w("o.b")


# ----------------------------------------------------------------------------- feed-forward
def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def choose_experts(z, correction, router):
    """z [E] router logits of one token -> (chosen experts, their weights).  The choice goes by sigmoid(z) + correction
    among the experts of the best groups (a group's worth: its two largest choice values added); the weights are sigmoid(z)."""
    E, top = router["experts"], router["top"]
    s = torch.sigmoid(z)
    c = s + correction
    groups = router.get("groups")
    if groups is not None and groups["count"] > 1:
        n = E // groups["count"]
        worth = torch.stack([torch.topk(c[g * n:(g + 1) * n], min(2, n)).values.sum() for g in range(groups["count"])])
        kept = torch.topk(worth, groups["keep"]).indices.tolist()
        masked = torch.full_like(c, -math.inf)
        for g in kept:
            masked[g * n:(g + 1) * n] = c[g * n:(g + 1) * n]
        c = masked
    chosen = torch.topk(c, top).indices
    return chosen, s[chosen]


def routed_experts(h, w, mlp, forced=None):
    """Each token's chosen experts weighted by their sigmoid scores (not renormalised), plus the shared expert.
    forced [T, top]: use these experts instead of choosing.  Returns (result, chosen [T, top])."""
    z = h @ w("router").T
    out = torch.zeros_like(h)
    all_chosen = []
    for t in range(h.shape[0]):
        chosen, wt = choose_experts(z[t], w("correction"), mlp["router"])
        if forced is not None:
            chosen = forced[t].to(torch.long)
            wt = torch.sigmoid(z[t, chosen])
        all_chosen.append(chosen)
        for s in range(chosen.numel()):
            e = int(chosen[s])
            out[t] = out[t] + wt[s] * clamped_expert(h[t], w(f"e{e}.gate"), w(f"e{e}.up"), w(f"e{e}.down"), mlp["expert"]["limit"])
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, w("shared.gate"), w("shared.up"), w("shared.down"), mlp["shared"]["limit"])
    return out, torch.stack(all_chosen)


# ----------------------------------------------------------------------------- the model
MIXERS = {"lightning": lightning, "attention": difference_attention, "attention_2": sink_attention}


def weights_layer(cfg, i):
    """The layer whose tensors layer i uses."""
    seen = set()
    while cfg["layers"][i].get("weights_of") is not None and i not in seen:
        seen.add(i)
        i = cfg["layers"][i]["weights_of"]
    return i


def forward(cfg, weights, tokens, forced=None, layers_out=None, mixers=None):
    """Logits [T, vocab] of one sequence.  forced: {layer: [T, top]} experts to use in place of the router's choice.
    forward.chosen holds the experts each routed layer chose.  layers_out: a list that receives the stream after every layer.
    mixers: other functions for some mixer types (tests that break a mechanism on purpose)."""
    W = {k: v.to(F) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = W["embed"][tok]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg is not None:
        x = x + W["bigram"][pair_rows(list(tokens), bg)]
    forward.chosen = {}
    for i, L in enumerate(cfg["layers"]):
        j = weights_layer(cfg, i)
        h = rms_norm(x, W[f"l{j}.norm1"], eps)
        y = {**MIXERS, **(mixers or {})}[L["type"]](h, lambda n, j=j: W[f"l{j}.mix.{n}"], L["mixer"], eps)
        if L.get("mlp") is not None:
            f, forward.chosen[i] = routed_experts(h, lambda n, j=j: W[f"l{j}.mlp.{n}"], L["mlp"], None if forced is None else forced.get(i))
            y = y + f
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["embed"].T

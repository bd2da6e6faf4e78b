"""Small Sigusun configurations for the tests.  They differ from each other in every size, in the order of the layer
types and in what a layer has, and they use values that are easy to get wrong when two of them happen to be equal
elsewhere: values wider and narrower than keys, rotations of part of a retention head, decays of one and far from one,
windows that are no multiple of the page size (and one position wide), a layer that reads another layer's latent under a
wider or a narrower window or without a window at all, layers without a feed-forward, without a shared expert, with one
expert per token and with all of them, models with and without the per-layer token input."""
import copy


def _ff(kind):
    """kind: None, or (experts, top, ff, limit, shared ff or None, shared limit)."""
    if kind is None:
        return None
    experts, top, ff, limit, sff, slimit = kind
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if sff:
        out["shared"] = {"ff": sff, "limit": slimit}
    return out


def retention(heads, dim, vdim, decay, dims, base, ff=None):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": dims}},
            "mlp": _ff(ff)}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base, kv_from):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def window(heads, dim, rot_dim, vdim, rank, scale, size, base, kv_from=None, ff=None):
    m = _latent(heads, dim, rot_dim, vdim, rank, scale, base, kv_from)
    m["mask"] = {"size": size}
    return {"type": "latent_attention", "mixer": m, "mlp": _ff(ff)}


def sink(heads, dim, rot_dim, vdim, rank, scale, base, kv_from=None, ff=None):
    return {"type": "latent_attention_2", "mixer": _latent(heads, dim, rot_dim, vdim, rank, scale, base, kv_from), "mlp": _ff(ff)}


def model(layers, width, vocab, page, side=0, eps=1e-5):
    out = {"architecture": "Sigusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "kv_page_size": page,
           "layers": [copy.deepcopy(L) for L in layers]}
    if side:
        out["token_side"] = {"dim": side}
    return out


def one_layer(layer, width=48, vocab=61, page=4, side=0):
    return model([layer], width, vocab, page, side)


G1 = model([retention(3, 16, 24, [0.9, 0.99, 1.0], 8, 500.0, ff=(5, 2, 40, 1.2, 24, 0.8)),
            window(4, 8, 12, 10, 24, 0.6, 7, 100.0, ff=(6, 3, 20, 0.9, None, 0)),
            window(2, 8, 12, 16, 24, 0.5, 19, 100.0, kv_from=1, ff=(4, 4, 12, 2.0, 16, 1.0)),
            sink(3, 12, 4, 8, 20, 0.4, 3000.0)], width=96, vocab=211, page=4, side=5)

G2 = model([sink(4, 16, 8, 16, 32, 0.3, 10000.0, ff=(3, 1, 24, 1.0, 40, 2.5)),
            window(2, 16, 8, 24, 32, 0.35, 33, 10000.0, kv_from=0),
            retention(2, 32, 16, [0.97, 0.999], 32, 10000.0, ff=(7, 2, 16, 0.7, None, 0)),
            window(4, 8, 16, 8, 16, 0.5, 9, 777.0, ff=(3, 3, 30, 1.1, 8, 0.6)),
            sink(2, 8, 16, 12, 16, 0.45, 777.0, kv_from=3)], width=64, vocab=97, page=8)

# widths at which the bfloat16 path takes its tensor-core products and attention kernels (multiples of 16)
G3 = model([window(4, 64, 32, 64, 128, 0.1, 100, 50000.0, ff=(8, 2, 64, 1.0, 128, 1.5)),
            retention(4, 64, 64, [0.95, 0.99, 0.995, 0.999], 32, 10000.0, ff=(16, 4, 32, 1.3, 64, 1.0)),
            window(8, 32, 32, 32, 128, 0.12, 48, 50000.0, kv_from=0, ff=(8, 2, 64, 0.9, None, 0)),
            sink(4, 32, 64, 48, 64, 0.1, 1000.0, ff=(4, 2, 96, 1.0, 32, 2.0)),
            retention(2, 128, 128, [0.98, 0.9995], 128, 1e6)], width=128, vocab=384, page=16, side=16)

# no size a multiple of 4: every product, norm and attention takes its general path
G4 = model([retention(5, 7, 9, [0.93, 0.97, 0.99, 0.995, 1.0], 6, 300.0, ff=(7, 3, 9, 0.7, 11, 1.3)),
            sink(3, 10, 6, 5, 13, 0.4, 50.0, ff=(3, 2, 13, 1.0, None, 0)),
            window(2, 6, 6, 14, 13, 0.3, 21, 50.0, kv_from=1),
            window(3, 5, 2, 7, 9, 0.5, 5, 20.0, ff=(2, 1, 6, 0.5, 5, 0.5))], width=50, vocab=33, page=3, side=3)

ALL = {"G1": G1, "G2": G2, "G3": G3, "G4": G4}


def get(name):
    return copy.deepcopy(ALL[name])

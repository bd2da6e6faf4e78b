"""Small Kitodra configurations for the tests.  They differ from each other in every size, in the order of the layer
types and in what a layer has, and they use values that are easy to get wrong when two of them happen to be equal or 1
elsewhere: values wider and narrower than keys, one key head and as many as heads, windows and chunks that are no multiple
of the page size (and one position wide), rotations of none, part and all of a head, decays of one and far from one,
layers that run with another (earlier or later) layer's tensors, layers without a feed-forward, without a shared expert
and without groups, one group kept and all of them, one expert chosen and all, and a model without the token-pair table."""
import copy


def ff(experts, top, width, limit, groups=None, shared=None):
    """groups: (count, keep) or None; shared: (width, limit) or None."""
    out = {"kind": "moe", "expert": {"ff": width, "limit": limit}, "router": {"experts": experts, "top": top}}
    if groups is not None:
        out["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def difference(heads, kv_heads, dim, vdim, scale, chunk, softcap, diff, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
                                           "diff": diff, "mask": {"size": chunk}}, "mlp": mlp}


def sink(heads, kv_heads, dim, scale, window, dims, base, mlp=None):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                                             "mask": {"size": window}, "rot": {"base": base, "dims": dims}}, "mlp": mlp}


def again(layers, j):
    """A layer that runs with layer j's tensors."""
    out = copy.deepcopy(layers[j])
    out["weights_of"] = j
    return out


def model(layers, width, vocab, page, bigram=(37, 5, 3), eps=1e-5):
    out = {"architecture": "Kitodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "kv_page_size": page,
           "layers": [copy.deepcopy(L) for L in layers]}
    if bigram is not None:
        out["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return out


def one_layer(layer, width=48, vocab=61, page=4, bigram=(37, 5, 3)):
    return model([layer], width, vocab, page, bigram)


def _t1():
    L = [lightning(3, 16, 24, [0.9, 0.99, 1.0], ff(6, 2, 40, 1.2, groups=(3, 2), shared=(24, 0.8))),
         sink(4, 2, 16, 0.6, 7, 8, 100.0, ff(4, 4, 20, 0.9, groups=(2, 2))),
         difference(4, 1, 8, 12, 0.5, 19, 5.0, 0.3, ff(5, 3, 12, 2.0, shared=(16, 1.0)))]
    return model(L + [again(L, 1), again(L, 0)], width=96, vocab=211, page=4, bigram=(101, 31, 7))


def _t2():
    L = [difference(2, 2, 16, 8, 0.3, 33, 30.0, 0.8, ff(8, 2, 24, 1.0, groups=(4, 1), shared=(40, 2.5))),
         lightning(2, 32, 16, [0.97, 0.999]),
         sink(3, 3, 8, 0.45, 9, 0, 777.0, ff(3, 1, 30, 1.1))]
    L = L + [copy.deepcopy(L[1])]
    L[3]["weights_of"] = 1
    L.append(sink(2, 1, 24, 0.35, 40, 24, 10000.0, ff(9, 3, 16, 0.7, groups=(3, 1), shared=(8, 0.6))))
    return model(L, width=64, vocab=97, page=8, bigram=None)


def _t3():
    # widths at which the bfloat16 path takes its tensor-core products and attention kernels
    L = [sink(4, 2, 64, 0.1, 100, 32, 50000.0, ff(8, 2, 64, 1.0, groups=(2, 1), shared=(128, 1.5))),
         lightning(4, 64, 64, [0.95, 0.99, 0.995, 0.999], ff(16, 4, 32, 1.3, groups=(4, 2), shared=(64, 1.0))),
         difference(4, 2, 32, 64, 0.15, 48, 25.0, 0.45, ff(8, 2, 64, 0.9, groups=(8, 3))),
         sink(8, 8, 128, 0.08, 200, 128, 1e6, ff(4, 2, 96, 1.0, shared=(32, 2.0))),
         lightning(2, 128, 128, [0.98, 0.9995])]
    return model(L + [again(L, 2), again(L, 0)], width=128, vocab=384, page=16, bigram=(521, 1000003, 99991))


def _t4():
    # no size a multiple of 4: every product, norm and attention takes its general path; a layer that names a LATER layer
    L = [lightning(5, 7, 9, [0.93, 0.97, 0.99, 0.995, 1.0], ff(6, 3, 9, 0.7, groups=(2, 1), shared=(11, 1.3))),
         sink(3, 1, 10, 0.4, 5, 6, 50.0, ff(3, 2, 13, 1.0)),
         difference(6, 3, 5, 7, 0.5, 21, 3.0, 0.1),
         difference(3, 3, 6, 14, 0.3, 1, 50.0, 0.0, ff(2, 1, 6, 0.5, shared=(5, 0.5)))]
    L = [again([None, None, None, L[2]], 3)] + L
    L[0]["weights_of"] = 3
    return model(L, width=50, vocab=33, page=3, bigram=(7, 2, 9))


ALL = {"T1": _t1(), "T2": _t2(), "T3": _t3(), "T4": _t4()}


def get(name):
    return copy.deepcopy(ALL[name])

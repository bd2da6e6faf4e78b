"""Kitodra configurations drawn at random over everything config.json allows (any order of the three kinds of layer, any
head counts and groups, key and value widths that are multiples of 16 or not, widths and vocabularies that are no multiple
of 8, decays up to one, windows and chunks from one position to longer than any prompt, rotations of none, part or all of
a head, experts from two up in one group or many with one to all of the groups kept and one to all of their experts
chosen, with and without a shared expert, layers without a feed-forward, layers that run on the tensors of any other
layer, with and without the token-pair table, pages of odd sizes), each replayed in mixed batches with reused pages and
slots in float32 and bfloat16 against the plain implementation: a size the kernels do not take must be handed to a kernel
that does, never computed wrongly."""
import copy
import random

import pytest

import helpers
import kitodra_helpers as kh

pytestmark = pytest.mark.gpu


def draw(seed, tensor_core=False):
    rng = random.Random(seed)
    n_layers = rng.choice([1, 2, 3, 4, 5, 6])
    even = lambda hi: 2 * rng.randint(0, hi // 2)

    def feed_forward():
        if rng.random() < 0.2:
            return None
        count = rng.choice([1, 1, 2, 3, 4])
        per = rng.choice([1, 2, 3, 5])
        experts = count * per if count * per > 1 else 2
        keep = rng.randint(1, count)
        router = {"experts": experts, "top": rng.randint(1, min(keep * (experts // count), 5))}
        if count > 1 or rng.random() < 0.3:
            router["groups"] = {"count": count, "keep": keep}
        out = {"kind": "moe", "expert": {"ff": rng.choice([8, 12, 24, 40, 64]), "limit": rng.choice([0.3, 1.0, 2.5, 7.0])}, "router": router}
        if rng.random() < 0.6:
            out["shared"] = {"ff": rng.choice([8, 20, 48, 96]), "limit": rng.choice([0.5, 1.5, 7.0])}
        return out

    def heads_and_groups():
        kv = rng.choice([1, 2, 3, 4])
        return kv * rng.choice([1, 1, 2, 3]), kv

    layers = []
    for i in range(n_layers):
        if layers and rng.random() < 0.3:                              # the tensors of another layer, earlier or (swapped below) later
            j = rng.randrange(len(layers))
            while layers[j].get("weights_of") is not None:
                j = layers[j]["weights_of"]
            layers.append({**copy.deepcopy(layers[j]), "weights_of": j})
            continue
        kind = rng.choice(["lightning", "attention", "attention_2"])
        if kind == "lightning":
            heads = rng.choice([1, 2, 3, 4, 6])
            dim = rng.choice([16, 32, 64, 128]) if tensor_core else rng.choice([6, 8, 16, 24, 32, 40, 64, 100])
            vdim = dim if rng.random() < 0.4 else rng.choice([4, 8, 12, 16, 32, 48, 64])
            m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [rng.choice([1.0, 1.0 - 2.0 ** -rng.randint(2, 10)]) for _ in range(heads)]}
        elif kind == "attention":
            heads, kv = heads_and_groups()
            dim, vdim = (rng.choice([16, 32, 64]), rng.choice([16, 32, 64, 96])) if tensor_core else (rng.choice([4, 6, 8, 16, 24, 40]), rng.choice([4, 5, 8, 16, 24, 33]))
            m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": rng.choice([0.05, 0.2, 0.5]), "softcap": rng.choice([0.5, 5.0, 50.0]),
                 "diff": rng.choice([0.0, 0.2, 0.5, 0.8]), "mask": {"size": rng.choice([1, 2, 7, 16, 30, 64, 500])}}
        else:
            heads, kv = heads_and_groups()
            dim = rng.choice([16, 32, 64, 128]) if tensor_core else rng.choice([4, 6, 8, 16, 24, 40, 64])
            m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": rng.choice([0.05, 0.125, 0.3]),
                 "mask": {"size": rng.choice([1, 2, 7, 16, 30, 64, 500])}, "rot": {"base": rng.choice([50.0, 10000.0, 1e6]), "dims": rng.choice([0, 2, even(dim), dim // 2 * 2])}}
        layers.append({"type": kind, "mixer": m, "mlp": feed_forward()})
    if len(layers) > 1 and layers[-1].get("weights_of") is None and layers[0].get("weights_of") is None and rng.random() < 0.3:
        # the first layer runs on the tensors of the last (a layer may name a later one)
        if not any(L.get("weights_of") == 0 for L in layers):
            layers[0] = {**copy.deepcopy(layers[-1]), "weights_of": len(layers) - 1}
    cfg = {"architecture": "Kitodra", "vocab": rng.choice([17, 100, 257, 1001]), "width": rng.choice([24, 40, 72, 100, 136, 264]),
           "norm": {"eps": rng.choice([1e-6, 1e-5, 3e-4])}, "kv_page_size": rng.choice([1, 3, 4, 8, 16, 24, 32]), "layers": layers}
    if tensor_core:
        cfg["width"], cfg["vocab"], cfg["kv_page_size"] = rng.choice([64, 128, 256]), rng.choice([128, 256, 1000]), rng.choice([8, 16, 32])
    if rng.random() < 0.75:
        cfg["embedding"] = {"bigram": {"buckets": rng.choice([1, 2, 61, 1000]), "mul_prev": rng.choice([0, 1, 31, 1_000_003]), "mul_cur": rng.choice([0, 1, 7, 999_983])}}
    return cfg


# the last six at sizes the tensor-core products and attention kernels take
@pytest.mark.parametrize("seed,tensor_core", [(s, False) for s in range(14)] + [(s, True) for s in range(14, 20)])
def test_random_configuration(tmp_path, seed, tensor_core):
    cfg = draw(seed, tensor_core)
    cfg_d, weights = kh.make_folder(str(tmp_path), cfg, seed=seed, init_std=0.08)
    V, page = cfg["vocab"], cfg["kv_page_size"]
    rng = random.Random(100 + seed)
    reqs = {f"r{i}": helpers.random_tokens(rng.randint(3, 90), V, 7 * seed + i) for i in range(5)}
    steps, mt = helpers.schedule_mixed(reqs, page, seed=seed, max_live=3)
    for dtype in ("float32", "bfloat16"):
        kh.replay_and_compare(str(tmp_path), cfg_d, weights, reqs, steps, mt, dtype, f"configuration {seed}: {cfg}", max_requests=3)
    from quench6k_b200 import ops
    assert ops.tc_status() == 0

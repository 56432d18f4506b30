"""Small configurations of the Fobilorn decoder for the tests, differing in every size and option, with helpers."""
import os

import numpy as np

from burn_lm_b200.config import preset


def layer(heads, kv_heads, dim, vdim, window, keep_first, mlp, v_mix=True, scale=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 2.0 * dim ** -0.5,
                      "v_mix": v_mix, "mask": {"size": window, "keep_first": keep_first}}}


def moe(experts, top, ff, shared_ff=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared_ff} if shared_ff else None}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model(vocab, width, buckets, mul_prev, mul_cur, layers, eps=1e-5):
    return {"architecture": "Fobilorn", "vocab": vocab, "width": width,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "norm": {"eps": eps},
            "layers": layers}


# every branch: dense, experts with and without a shared one, no feed-forward, layers in and out of the blending
FOB_A = preset("fobilorn_tiny")
# values that a model may happen to make equal or 1: as many kv heads as heads, keys as wide as values, one head,
# every expert chosen, one expert, no kept first tokens, a window longer than any test sequence, one blending layer
FOB_B = model(131, 64, 1, 1, 1, [
    layer(2, 2, 16, 16, 4096, 0, moe(3, 3, 16, 16), v_mix=True),
    layer(1, 1, 32, 32, 4096, 0, moe(1, 1, 24), v_mix=False),
    layer(3, 3, 8, 8, 4096, 5, dense(40), v_mix=False),
])
# windows that end inside the first page, at a page's border and beyond it; kept first tokens that fill more than a
# page; a window of one token; nine heads on three kv heads; sizes that are no multiples of 8
FOB_C = model(257, 72, 97, 1000003, 998244353, [
    layer(9, 3, 12, 20, 64, 70, dense(100)),
    layer(4, 1, 20, 12, 1, 2, moe(7, 3, 20, 36), v_mix=False),
    layer(2, 1, 40, 60, 129, 1, moe(4, 2, 28)),
    layer(5, 5, 16, 12, 37, 0, None),
], eps=1e-6)

# heads of 64 and of 128 lanes, the sizes the tensor-core kernels are mostly used with, values of 128 and of 72 lanes
# (sixteen value tiles), groups of four and of one query head a kv head, windows shorter and longer than a page
FOB_D = model(300, 128, 509, 7, 11, [
    layer(4, 1, 64, 64, 100, 4, dense(192)),
    layer(4, 2, 128, 128, 70, 0, moe(4, 2, 64, 64), v_mix=False),
    layer(2, 2, 64, 72, 40, 65, None, v_mix=False),
    layer(8, 1, 32, 64, 200, 1, moe(3, 1, 128)),
])

CONFIGS = {"fob_a": FOB_A, "fob_b": FOB_B, "fob_c": FOB_C, "fob_d": FOB_D}


def make_folder(tmp_path, name, seed=0, dtype="bfloat16"):
    from burn_lm_b200 import write_random_model

    folder = os.path.join(str(tmp_path), f"{name}-{dtype}-{seed}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(folder, CONFIGS[name], seed=seed, dtype=dtype)
    return folder


def random_tokens(seed, n, vocab):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=n)]


def row_error(got, want):
    """max |got - want| of every row, relative to the row's largest |want|."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return np.abs(got - want).max(axis=-1) / np.abs(want).max(axis=-1)

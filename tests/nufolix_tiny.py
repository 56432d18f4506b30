"""Small configurations of the Nufolix decoder for the tests, differing in every size and option, with helpers."""
import os

import numpy as np

from burn_lm_b200.config import preset


def parallel(heads, kv_heads, dim, vdim, rot_dims, r_heads, r_qk_heads, r_dim, r_vdim, r_conv, ff, left_scale=0.5, right_scale=1.25,
             softcap=15.0, base=10000.0, scale=None):
    return {"type": "parallel", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 2.0 * dim ** -0.5,
                               "softcap": softcap, "rot": {"dims": rot_dims, "base": base}},
                      "right": {"heads": r_heads, "kv_heads": r_qk_heads, "dim": r_dim, "vdim": r_vdim, "conv": r_conv},
                      "left_scale": left_scale, "right_scale": right_scale}}


def mamba2(heads, vdim, state, groups, conv, norm_groups, ff):
    return {"type": "mamba2", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def model(vocab, width, layers, scale=None, eps=1e-5, mult=0.8):
    return {"architecture": "Nufolix", "vocab": vocab, "width": width, "embedding": {"scale": scale or width ** 0.5},
            "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


# every branch (see the preset)
NUF_A = preset("nufolix_tiny")
# values that a model may happen to make equal or 1: one head everywhere, as many kv heads as heads, keys as wide as
# values, the whole head rotated and no lane rotated, one group, one norm part, a convolution of one tap (nothing carried)
# and of two, scales and the multiplier 1, only parallel layers first and only state-space layers last
NUF_B = model(131, 64, [
    parallel(1, 1, 32, 32, 32, 1, 1, 32, 32, 2, 48, left_scale=1.0, right_scale=1.0),
    parallel(2, 2, 16, 16, 0, 2, 2, 16, 16, 1, None, left_scale=1.0, right_scale=1.0, softcap=50.0),
    mamba2(1, 64, 16, 1, 1, 1, None),
    mamba2(2, 32, 8, 1, 2, 1, 64),
], scale=1.0, mult=1.0)
# sizes that are no multiples of 8 or of a warp: nine heads on three kv heads, heads of 12 and 20 lanes, values of 40
# lanes (a second, partly filled tile of the scan), states of 20 and of 5 rows, a width of 72, five taps
NUF_C = model(257, 72, [
    parallel(9, 3, 12, 20, 6, 3, 1, 20, 40, 5, 100, base=500.0),
    mamba2(3, 40, 20, 3, 5, 2, None),
    mamba2(5, 12, 5, 1, 2, 5, 40),
    parallel(2, 1, 20, 12, 20, 5, 5, 12, 12, 2, None, left_scale=-0.7, right_scale=0.3),
], eps=1e-6, mult=0.6)
# heads of 64 and of 128 lanes and states of 64 and 128 rows, the sizes of large models
NUF_D = model(300, 128, [
    parallel(4, 1, 64, 64, 32, 2, 1, 128, 64, 4, 192, base=1e6),
    mamba2(4, 64, 128, 1, 4, 1, None),
    parallel(2, 2, 128, 128, 128, 4, 2, 64, 32, 3, None),
    mamba2(8, 32, 64, 2, 4, 2, 256),
])

CONFIGS = {"nuf_a": NUF_A, "nuf_b": NUF_B, "nuf_c": NUF_C, "nuf_d": NUF_D}


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

"""The Nufolix decoder in the engine against the plain implementation (tests/plain/nufolix_plain.py): every
mechanism's kernels alone, then whole models through the step function, the cache, the scheduler and generation."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import nufolix_plain as P
from nufolix_tiny import CONFIGS, make_folder, random_tokens, row_error

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 4e-2
PAGE = 64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dev(x, dtype=torch.float32):
    return torch.tensor(np.asarray(x), dtype=dtype, device="cuda")


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device="cuda")


class Scratch:
    def scratch(self, name, n):
        return torch.empty(max(n, 1), dtype=torch.float32, device="cuda")


def step_of(portions, slots, starts):
    """A step that brings portions[s] tokens of the sequence in slots[s], which has starts[s] tokens already."""
    seq_of, pos, cu = [], [], [0]
    for s, (k, st) in enumerate(zip(portions, starts)):
        seq_of += [s] * k
        pos += list(range(st, st + k))
        cu.append(cu[-1] + k)
    return SimpleNamespace(token_seq=ints(seq_of), token_pos=ints(pos), slot_of_seq=ints(slots), cu_seqlens=ints(cu),
                           start_pos=ints(starts), n_tokens=len(seq_of), n_seqs=len(slots), max_q_len=max(portions),
                           max_kv_len=max(s + k for s, k in zip(starts, portions)), workspace=Scratch())


def engine_for(folder, dtype, max_tokens=4096, **kw):
    from burn_lm_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def close(got, want, tol):
    want = np.asarray(want)
    return np.abs(np.asarray(got, dtype=np.float64) - want).max() <= tol * max(1.0, np.abs(want).max())


# ---------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------
def test_scaled_embedding():
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(0)
    table = dev(rng.normal(size=(37, 50)), torch.bfloat16)
    out = torch.empty((4, 50), dtype=torch.float32, device="cuda")
    K.embed_scaled(ints([3, 36, 0, 3]), table, out, 7.25)
    assert np.array_equal(out.cpu().numpy(), table.float().cpu().numpy()[[3, 36, 0, 3]] * np.float32(7.25))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norm_behind_a_sublayer_and_the_next_norm_in_one_kernel(dtype):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(1)
    n, d, mult, eps = 9, 100, 0.7, 1e-5
    x, a, bias = rng.normal(size=(n, d)) * 3, rng.normal(size=(n, d)) * 40, rng.normal(size=d)
    wb, w = rng.normal(size=d) + 1, rng.normal(size=d) + 1
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for with_bias in (False, True):
        for delta_dtype in (torch.float32, dtype):
            resid = dev(x)
            delta = dev(a, delta_dtype)
            out = torch.empty((n, d), dtype=dtype, device="cuda")
            K.sandwich_norm(resid, delta, dev(wb), mult, eps, dev(w), eps, out, delta_bias=dev(bias) if with_bias else None)
            raw = delta.float().cpu().numpy().astype(np.float64) + (bias if with_bias else 0.0)
            stream = x + mult * P.rms_norm(raw, wb, eps)
            assert close(resid.cpu().numpy(), stream, 1e-5)                 # the stream took the normed output, in fp32
            assert close(out.float().cpu().numpy(), P.rms_norm(stream, w, eps), tol)
    # some rows only: the stream stays as it was
    resid = dev(x)
    rows = [5, 0, 5]
    out = torch.empty((3, d), dtype=dtype, device="cuda")
    K.sandwich_norm(resid, dev(a), dev(wb), mult, eps, dev(w), eps, out, rows=ints(rows))
    assert np.array_equal(resid.cpu().numpy(), x.astype(np.float32))
    assert close(out.float().cpu().numpy(), P.rms_norm((x + mult * P.rms_norm(a, wb, eps))[rows], w, eps), tol)
    # nothing pending: a plain norm; no norm next: only the add
    plain = torch.empty((n, d), dtype=dtype, device="cuda")
    K.sandwich_norm(resid, None, None, 1.0, eps, dev(w), eps, plain)
    assert np.array_equal(resid.cpu().numpy(), x.astype(np.float32)) and close(plain.float().cpu().numpy(), P.rms_norm(x, w, eps), tol)
    only = dev(x)
    K.sandwich_norm(only, dev(a), dev(wb), mult, eps, None, 0.0, None)
    assert close(only.cpu().numpy(), x + mult * P.rms_norm(a, wb, eps), 1e-5)
    # two outputs side by side: their weighted sum is taken first
    b2 = rng.normal(size=(n, d)) * 5
    resid = dev(x)
    K.sandwich_norm(resid, dev(a), dev(wb), mult, eps, dev(w), eps, plain, second=(0.6, dev(b2), -1.3), delta_bias=dev(bias))
    stream = x + mult * P.rms_norm(0.6 * a + -1.3 * b2 + bias, wb, eps)
    assert close(resid.cpu().numpy(), stream, 1e-5) and close(plain.float().cpu().numpy(), P.rms_norm(stream, w, eps), tol)


def test_xielu_with_a_bias():
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(2)
    z, b = rng.normal(size=(11, 70)) * 3, rng.normal(size=70)
    z[0, :4] = [0.0, -1e-4, 1e-4, -30.0]
    for p, q in ((0.3, -0.8), (-2.0, 1.5)):
        out = torch.empty((11, 70), dtype=torch.float32, device="cuda")
        K.bias_act(dev(z), dev(b), out, K.ACT_XIELU, dev([p, q]))
        assert close(out.cpu().numpy(), P.xielu(z.astype(np.float32).astype(np.float64) + b.astype(np.float32), p, q), 1e-5)


def _conv_case(rng, channels, taps, lengths):
    xs = [rng.normal(size=(n, channels)) for n in lengths]
    w, b = rng.normal(size=(channels, taps)), rng.normal(size=channels)
    return xs, w, b, [P.silu(P.causal_conv(x, w, b)) for x in xs]


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_convolution_carries_its_last_inputs(taps):
    """Two sequences side by side in portions of 1, 2 and many tokens, fewer than the taps and more; a slot used again by
    another sequence; a single-token step run twice."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(3)
    channels, lengths = 45, [23, 17]
    xs, w, b, want = _conv_case(rng, channels, taps, lengths)
    floats = 10 + (taps - 1) * channels
    state = torch.full((4, 2, floats), float("nan"), device="cuda")       # rubbish: a sequence's start must not read it
    slots, at = [3, 1], [0, 0]
    for portion in [(1, 2), (2, 1), (1, 1), (5, 3), (3, 1), (11, 9)]:
        st = step_of(portion, slots, at)
        x = np.concatenate([xs[s][at[s]: at[s] + k] for s, k in enumerate(portion)])
        wide = torch.zeros((len(x), channels + 6), device="cuda")
        wide[:, 4: 4 + channels] = dev(x)
        out = torch.full((len(x), channels + 3), 7.0, device="cuda")
        for again in range(2 if portion == (1, 1) else 1):        # a step of single tokens may run twice
            K.causal_conv(wide, 4, channels, dev(w), dev(b), out, 2, st, state, 10)
        row = 0
        for s, k in enumerate(portion):
            assert close(out[row: row + k, 2: 2 + channels].cpu().numpy(), want[s][at[s]: at[s] + k], 1e-5), (portion, s)
            row += k
            at[s] += k
        assert torch.all(out[:, :2] == 7.0) and torch.all(out[:, 2 + channels:] == 7.0)
    # the slot of the first sequence goes to a new one
    xs2, w2, b2, want2 = _conv_case(np.random.default_rng(4), channels, taps, [6])
    st = step_of((6,), [3], [0])
    out = torch.empty((6, channels), device="cuda")
    K.causal_conv(dev(xs2[0]), 0, channels, dev(w2), dev(b2), out, 0, st, state, 10)
    assert close(out.cpu().numpy(), want2[0], 1e-5)
    # rows of no sequence give zeros and carry nothing
    before = state.clone()
    st = SimpleNamespace(token_seq=ints([-1, -1]), cu_seqlens=ints([0, 0]), slot_of_seq=ints([1]), start_pos=ints([5]), n_tokens=2, n_seqs=1)
    out = torch.full((2, channels), 3.0, device="cuda")
    K.causal_conv(dev(rng.normal(size=(2, channels))), 0, channels, dev(w), dev(b), out, 0, st, state, 10)
    assert torch.all(out == 0) and torch.equal(torch.nan_to_num(before), torch.nan_to_num(state))


SCAN_SHAPES = [  # heads, groups (or qk heads), rows, value lanes
    (4, 2, 16, 24), (3, 3, 5, 40), (1, 1, 56, 24), (2, 1, 128, 64), (6, 2, 20, 12), (2, 2, 64, 100)]


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("heads,groups,n_state,dv", SCAN_SHAPES)
def test_state_space_scan_in_portions(heads, groups, n_state, dv, wide):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(5)
    lengths = [70, 9]
    gn, inner = groups * n_state, heads * dv
    a_log, d_skip, dt_bias = rng.normal(size=heads) * 0.5, rng.normal(size=heads), rng.normal(size=heads) * 0.5
    seqs, want = [], []
    for n in lengths:
        x, B, C, dt = rng.normal(size=(n, heads, dv)), rng.normal(size=(n, groups, n_state)), rng.normal(size=(n, groups, n_state)), rng.normal(size=(n, heads))
        seqs.append((x, B, C, dt))
        want.append(P.mamba2_scan(x, B, C, P.softplus(dt + dt_bias), a_log, d_skip, heads, groups).reshape(n, inner))
    floats = 7 + K.scan_state_floats(heads, n_state, dv)
    state = torch.full((3, 2, floats), float("nan"), device="cuda")
    slots, at = [2, 0], [0, 0]
    for portion in [(1, 1), (2, 1), (1, 2), (33, 3), (2, 1), (31, 1)]:
        st = step_of(portion, slots, at)
        rows = [np.concatenate([seqs[s][i][at[s]: at[s] + k].reshape(k, -1) for s, k in enumerate(portion)]) for i in range(4)]
        xbc = dev(np.concatenate([rows[0], rows[1], rows[2]], axis=1))
        dt = torch.zeros((xbc.shape[0], heads + 3), device="cuda")
        dt[:, 3:] = dev(rows[3])
        y = torch.zeros((xbc.shape[0], inner), device="cuda")
        for again in range(2 if max(portion) == 1 else 1):
            K.ssm_scan(xbc, 0, inner, inner + gn, dt, 3, dev(dt_bias), dev(a_log), dev(d_skip), y, heads, groups, n_state, dv, st, state, 7,
                       wide_sums=wide)
        row = 0
        for s, k in enumerate(portion):
            assert close(y[row: row + k].cpu().numpy(), want[s][at[s]: at[s] + k], 2e-6 if wide else 2e-5), (portion, s)
            row += k
            at[s] += k


@pytest.mark.parametrize("heads,qk_heads,dk,dv", SCAN_SHAPES)
def test_gated_delta_rule_in_portions(heads, qk_heads, dk, dv):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(6)
    lengths = [70, 9]
    a_log, dt_bias = rng.normal(size=heads) * 0.5, rng.normal(size=heads * dk) * 0.5
    seqs, want = [], []
    for n in lengths:
        q, k, v = rng.normal(size=(n, qk_heads, dk)), rng.normal(size=(n, qk_heads, dk)), rng.normal(size=(n, heads, dv))
        b, a = rng.normal(size=(n, heads)), rng.normal(size=(n, heads, dk))
        seqs.append((q, k, v, b, a))
        g = np.exp(-np.exp(a_log)[None, :, None] * P.softplus(a + dt_bias.reshape(heads, dk)))
        want.append(P.delta_rule_scan(P.unit(q) * dk ** -0.5, P.unit(k), v, P.sigmoid(b), g).reshape(n, heads * dv))
    floats = K.scan_state_floats(heads, dk, dv)
    state = torch.full((3, 2, floats), float("nan"), device="cuda")
    slots, at = [1, 2], [0, 0]
    for portion in [(1, 1), (1, 2), (2, 1), (33, 3), (2, 1), (31, 1)]:
        st = step_of(portion, slots, at)
        t = [dev(np.concatenate([seqs[s][i][at[s]: at[s] + k].reshape(k, -1) for s, k in enumerate(portion)])) for i in range(5)]
        qkv = torch.cat([t[0], t[1], t[2]], dim=1).contiguous()
        o = torch.zeros((qkv.shape[0], heads * dv), device="cuda")
        for again in range(2 if max(portion) == 1 else 1):
            K.delta_scan(qkv, 0, qkv, qk_heads * dk, qkv, 2 * qk_heads * dk, t[3], 0, t[4], 0, dev(dt_bias), dev(a_log), o, heads,
                         qk_heads, dk, dv, st, state, 0)
        row = 0
        for s, k in enumerate(portion):
            assert close(o[row: row + k].cpu().numpy(), want[s][at[s]: at[s] + k], 2e-5), (portion, s)
            row += k
            at[s] += k


def test_a_written_value_is_read_back_through_a_long_quiet_stretch():
    """The delta rule with beta = 1 and no decay stores v under a unit key; hundreds of tokens with orthogonal keys later a
    query along that key reads it back: a lost or cleared state would show."""
    from burn_lm_b200 import kernels as K
    heads, dk, dv, n = 1, 16, 8, 300
    k = np.zeros((n, 1, dk))
    k[:, 0, 1] = 1.0
    k[0, 0, :] = 0.0
    k[0, 0, 0] = 1.0                      # token 0 writes under lane 0, all others under lane 1
    v = np.random.default_rng(7).normal(size=(n, 1, dv))
    q = np.zeros((n, 1, dk))
    q[:, 0, 0] = 1.0
    b, a = np.full((n, 1), 40.0), np.full((n, 1, dk), -40.0)        # beta = 1, softplus(-40) = 0: no decay
    state = torch.zeros((1, 2, K.scan_state_floats(heads, dk, dv)), device="cuda")
    outs, at = [], 0
    for portion in [64, 1, 1, 130, 2, 102]:
        st = step_of((portion,), [0], [at])
        sl = slice(at, at + portion)
        qkv = dev(np.concatenate([q[sl].reshape(portion, -1), k[sl].reshape(portion, -1), v[sl].reshape(portion, -1)], axis=1))
        o = torch.zeros((portion, dv), device="cuda")
        K.delta_scan(qkv, 0, qkv, dk, qkv, 2 * dk, dev(b[sl]), 0, dev(a[sl].reshape(portion, -1)), 0, dev(np.zeros(dk)), dev([0.0]), o,
                     heads, 1, dk, dv, st, state, 0)
        outs.append(o.cpu().numpy())
        at += portion
    got = np.concatenate(outs)
    assert close(got, np.tile(v[0, 0] * dk ** -0.5, (n, 1)), 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_group_norm_with_its_gate_on_either_side(dtype):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(8)
    n, groups, size, eps = 6, 5, 24, 1e-5
    y, gate = rng.normal(size=(n, groups * size)) * 3, rng.normal(size=(n, groups * size + 4))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    w = rng.normal(size=groups * size) + 1
    out = torch.empty((n, groups * size), dtype=dtype, device="cuda")
    K.gated_group_norm(dev(y), dev(gate), 4, dev(w), size, K.GATE_FIRST, eps, out)
    u = (y * P.silu(gate[:, 4:])).reshape(n, groups, size)
    want = (u / np.sqrt((u * u).mean(axis=-1, keepdims=True) + eps)).reshape(n, -1) * w
    assert close(out.float().cpu().numpy(), want, tol)
    ws = rng.normal(size=size) + 1
    K.gated_group_norm(dev(y), dev(gate), 4, dev(ws), size, K.GATE_LAST, eps, out)
    u = y.reshape(n, groups, size)
    want = (u / np.sqrt((u * u).mean(axis=-1, keepdims=True) + eps) * ws).reshape(n, -1) * P.sigmoid(gate[:, 4:])
    assert close(out.float().cpu().numpy(), want, tol)


def _attend(dtype, H, G, dk, dv, rot, q, k, v, bias, talk, pb, scale, cap, portions, base=10000.0, ranges=1, pages=None, scalar_only=False):
    """q, k, v: projections before bias and rotation, [T, ...] of one sequence, run in the given portions through the append
    kernel and the attention; returns the outputs [T, H * dv]."""
    from burn_lm_b200 import kernels as K
    T = q.shape[0]
    n_pages = (T + PAGE - 1) // PAGE
    pages = pages or list(range(n_pages))
    pool = torch.full((max(pages) + 2, G * PAGE * (dk + dv)), float("nan"), dtype=dtype, device="cuda")
    table = ints(pages).reshape(1, -1)
    freq = dev([base ** (-2.0 * i / rot) for i in range(rot // 2)], torch.float64) if rot else None
    outs, at = [], 0
    for portion in portions:
        st = step_of((portion,), [0], [at])
        sl = slice(at, at + portion)
        proj = dev(np.concatenate([q[sl].reshape(portion, -1), k[sl].reshape(portion, -1), v[sl].reshape(portion, -1)], axis=1))
        qo = torch.empty((portion, H * dk), dtype=dtype, device="cuda")
        K.bias_rope_append(proj, dev(bias) if bias is not None else None, freq, rot, qo, pool, table, st, H, G, dk, dv)
        out = torch.zeros((portion, H * dv), dtype=dtype, device="cuda")
        partial = torch.empty(ranges * portion * H * dv, device="cuda") if ranges > 1 else None
        K.sigmoid_attention(qo, pool, table, st, out, H, G, dk, dv, scale, softcap=cap, talk=dev(talk) if talk is not None else None,
                            head_bias=dev(pb) if pb is not None else None, ranges=ranges, partial=partial, scalar_only=scalar_only)
        outs.append(out.float().cpu().numpy())
        at += portion
    return np.concatenate(outs)


def _plain_attention(H, G, dk, dv, rot, q, k, v, bias, talk, pb, scale, cap, base=10000.0):
    T = q.shape[0]
    if bias is not None:
        q = q + bias[: H * dk].reshape(H, dk)
        k = k + bias[H * dk: (H + G) * dk].reshape(G, dk)
        v = v + bias[(H + G) * dk:].reshape(G, dv)
    q, k = P.rotate(q, range(T), rot, base), P.rotate(k, range(T), rot, base)
    w = P.sigmoid_attention_weights(q, k, scale, cap, pb if pb is not None else np.zeros(H))
    if talk is not None:
        w = P.mix_heads(w, talk)
    return np.stack([w[h] @ v[:, h // (H // G)] for h in range(H)], axis=1).reshape(T, H * dv)


ATTENTION_SHAPES = [  # heads, kv heads, key lanes, value lanes, rotated lanes
    (4, 2, 24, 16, 16), (9, 3, 12, 20, 6), (1, 1, 32, 32, 32), (2, 2, 16, 16, 0), (4, 1, 64, 64, 32), (2, 2, 128, 128, 128),
    (6, 3, 48, 40, 32), (16, 4, 64, 128, 64)]


@pytest.mark.parametrize("H,G,dk,dv,rot", ATTENTION_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_attention_in_prompts_portions_and_single_tokens(dtype, H, G, dk, dv, rot):
    rng = np.random.default_rng(9)
    T = 150
    q, k, v = rng.normal(size=(T, H, dk)), rng.normal(size=(T, G, dk)), rng.normal(size=(T, G, dv))
    bias, talk, pb = rng.normal(size=(H + G) * dk + G * dv) * 0.3, rng.normal(size=(H, H)) * 0.5, rng.normal(size=H) - 3.0
    scale, cap = 2.0 * dk ** -0.5, 6.0
    want = _plain_attention(H, G, dk, dv, rot, q, k, v, bias, talk, pb, scale, cap)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for portions, ranges, pages in (((150,), 1, None), ((63, 1, 1, 2, 70, 5, 1, 1, 1, 1, 1, 1, 1, 1), 1, [4, 0, 2]), ((100, 50), 3, [1, 5, 3]),
                                    ((140,) + (1,) * 10, 2, None)):
        for scalar_only in ((False, True) if dtype == torch.bfloat16 else (False,)):     # prompts on and off the tensor cores
            got = _attend(dtype, H, G, dk, dv, rot, q, k, v, bias, talk, pb, scale, cap, portions, ranges=ranges, pages=pages,
                          scalar_only=scalar_only)
            assert close(got, want, tol), (portions, ranges, scalar_only)
    # without a cap, a mix or the biases
    got = _attend(dtype, H, G, dk, dv, rot, q, k, v, None, None, None, scale, 0.0, (90, 60))
    big = _plain_attention(H, G, dk, dv, rot, q, k, v, None, None, None, scale, 1e9)
    assert close(got, big, tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_key_far_back_at_page_borders_and_the_diagonal(dtype):
    """Every key is nearly shut (a head bias of -30) except one that a query's score lifts far above: the output is that
    key's value.  The key sits at the sequence's start, on both sides of page borders, on the diagonal, and one
    position after the query (which must not see it, in a prompt where that key is in the cache already)."""
    H, G, dk, dv, T = 2, 1, 16, 8, 400
    rng = np.random.default_rng(10)
    v = rng.normal(size=(T, G, dv))
    for key_at in (0, 63, 64, 127, 128, 255, 256, 320, 398, 399):
        for query_at in sorted({key_at - 1, key_at, min(key_at + 1, T - 1), T - 1} - {-1}):
            q, k = np.zeros((T, H, dk)), np.zeros((T, G, dk))
            k[key_at, 0, 3] = 8.0
            q[query_at, :, 3] = 8.0                       # score 64 * scale on the planted pair, 0 elsewhere
            pb = np.full(H, -30.0)
            for portions, ranges in (((T,), 1), ((T,), 4), ((key_at + 1,) + (1,) * (T - key_at - 1), 2) if key_at > 300 else ((200, 200), 3)):
                got = _attend(dtype, H, G, dk, dv, 0, q, k, v, None, np.eye(H), pb, 1.0, 0.0, portions, ranges=ranges)
                row = got[query_at].reshape(H, dv)
                if key_at <= query_at:
                    assert close(row, np.tile(v[key_at, 0], (H, 1)), 1e-4 if dtype == torch.float32 else 2e-2), (key_at, query_at, portions)
                else:
                    assert np.abs(row).max() < 1e-6, (key_at, query_at, portions)


def test_the_heads_mix_takes_every_heads_weight():
    """talk = a permutation: head h then applies the weights of another head to its own values."""
    H, G, dk, dv, T = 3, 3, 8, 4, 70
    rng = np.random.default_rng(11)
    q, k, v = rng.normal(size=(T, H, dk)), rng.normal(size=(T, G, dk)), rng.normal(size=(T, G, dv))
    talk = np.zeros((H, H))
    talk[0, 2] = talk[1, 0] = talk[2, 1] = 1.0
    got = _attend(torch.float32, H, G, dk, dv, 0, q, k, v, None, talk, None, 0.5, 0.0, (T,))
    w = P.sigmoid_attention_weights(q, k, 0.5, 1e9, np.zeros(H))
    want = np.stack([w[[2, 0, 1][h]] @ v[:, h] for h in range(H)], axis=1).reshape(T, -1)
    assert close(got, want, 2e-5)


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------
def _logits(engine, tokens, want, portions=None):
    from burn_lm_b200 import StepEntry
    slot = engine.acquire()
    rows, at = [], 0
    for k in portions or [len(tokens)]:
        w = [p - at for p in want if at <= p < at + k]
        out = engine.step([StepEntry(slot, tokens[at: at + k], w)])
        if w:
            rows.append(out.cpu().numpy().copy())
        at += k
    engine.release(slot)
    return np.concatenate(rows)


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype,tol", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompts_portions_and_single_tokens(tmp_path, name, dtype, tol):
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(1, 150, cfg["vocab"])
    want = P.forward(cfg, tensors, tokens)
    engine = engine_for(folder, dtype)
    every = list(range(len(tokens)))
    assert row_error(_logits(engine, tokens, every), want).max() < tol
    for portions in ([64, 64, 22], [1, 2, 61, 1, 1, 2, 2, 17, 63], [100] + [1] * 50, [2] * 75):
        assert row_error(_logits(engine, tokens, every, portions), want).max() < tol, portions
    # the first tokens alone, one at a time from an empty sequence
    assert row_error(_logits(engine, tokens[:9], list(range(9)), [1] * 9), want[:9]).max() < tol


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_stream_after_every_layer(tmp_path, name):
    from burn_lm_b200 import StepEntry
    from burn_lm_b200.parts import norm as N
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(2, 40, cfg["vocab"])
    _, after = P.forward(cfg, tensors, tokens, return_layers=True)
    engine = engine_for(folder, "float32")
    engine.use_graphs = False
    seen, plain_norm = [], N.RMSNorm.add_norm

    def watching(self, resid, delta, rows=None, lazy=False, handoff=None):
        out = plain_norm(self, resid, delta, rows=rows, lazy=lazy, handoff=handoff)
        if rows is None and isinstance(delta, N.PostNormed):
            seen.append(resid.detach().cpu().numpy().copy())
        return out

    N.RMSNorm.add_norm = watching
    try:
        slot = engine.acquire()
        engine.step([StepEntry(slot, tokens, [0])])
        engine.release(slot)
    finally:
        N.RMSNorm.add_norm = plain_norm
    at = 0          # `seen`: the stream after every sublayer but the last
    for i, layer in enumerate(cfg["layers"][:-1]):
        at += 2 if layer["mlp"] is not None else 1
        assert np.abs(seen[at - 1] - after[i]).max() < 1e-4 * np.abs(after[i]).max(), i


@pytest.mark.parametrize("name", ["nuf_a", "nuf_c"])
@pytest.mark.parametrize("dtype,tol", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_unequal_requests_together_through_used_slots_and_pages(tmp_path, name, dtype, tol):
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    engine = engine_for(folder, dtype, max_tokens=1024)
    for round_no in range(3):              # the same slots and pages serve three sets of requests
        lengths = [[1, 70, 130], [65, 3, 64, 20], [128, 2]][round_no]
        reqs = [random_tokens(10 * round_no + i, n + 12, cfg["vocab"]) for i, n in enumerate(lengths)]
        want = [P.forward(cfg, tensors, r) for r in reqs]
        slots = [engine.acquire() for _ in reqs]
        out = engine.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, lengths)]).cpu().numpy()
        for i, n in enumerate(lengths):
            assert row_error(out[i], want[i][n - 1]) < tol, (round_no, i)
        live = list(range(len(reqs)))
        for t in range(12):
            if t == 5:                      # the shortest request ends early
                gone = live.pop(int(np.argmin([lengths[i] for i in live])))
                engine.release(slots[gone])
            out = engine.step([StepEntry(slots[i], [reqs[i][lengths[i] + t]], [0]) for i in live]).cpu().numpy().copy()
            for j, i in enumerate(live):
                assert row_error(out[j], want[i][lengths[i] + t]) < tol, (round_no, i, t)
        for i in live:
            engine.release(slots[i])
    engine.verify()


def test_long_decoding(tmp_path):
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, "nuf_a")
    cfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(5, 330, cfg["vocab"])
    want = P.forward(cfg, tensors, tokens)
    engine = engine_for(folder, "float32")
    slot = engine.acquire()
    engine.step([StepEntry(slot, tokens[:30], [])])
    for p in range(30, len(tokens)):
        row = engine.step([StepEntry(slot, [tokens[p]], [0])]).cpu().numpy()[0]
        assert row_error(row, want[p]) < FP32_TOL, p
    engine.release(slot)


@pytest.mark.parametrize("name", ["nuf_a", "nuf_b"])
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, name)
    cfg, tensors = P.read_model_folder(folder)
    prompts = [random_tokens(20 + i, n, cfg["vocab"]) for i, n in enumerate([5, 70, 17])]
    want = [P.greedy(cfg, tensors, p, 10) for p in prompts]
    lm = blm.load(folder, dtype="float32", max_seq_len=256, max_batch=3)
    assert lm.generate(prompts, sample_len=10, ignore_stop=True).tokens == want
    assert lm.generate(prompts[::-1], sample_len=10, ignore_stop=True).tokens == want[::-1]      # used slots, another order


def test_the_device_side_decode_loop(tmp_path):
    """Steps replayed as a graph without the host, after a warm-up step that runs the first one twice: the state of a
    sequence is read from where that step found it."""
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, "nuf_a")
    cfg, tensors = P.read_model_folder(folder)
    prompts = [random_tokens(30 + i, n, cfg["vocab"]) for i, n in enumerate([33, 64])]
    want = [P.greedy(cfg, tensors, p, 9) for p in prompts]
    engine = engine_for(folder, "float32", max_tokens=1024)
    slots = [engine.acquire() for _ in prompts]
    first = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).argmax(dim=-1).tolist()
    assert first == [w[0] for w in want]
    more = engine.decode_run(slots, first, 8).cpu().numpy()
    assert more.T.tolist() == [w[1:] for w in want]
    again = engine.decode_run(slots, [w[-1] for w in want], 3)       # the captured graph once more, from where it stopped
    longer = [P.greedy(cfg, tensors, p, 12) for p in prompts]
    assert again.cpu().numpy().T.tolist() == [w[9:] for w in longer]


def test_the_trace_runner_as_a_child_process(tmp_path):
    folder = make_folder(tmp_path, "nuf_c")
    cfg, tensors = P.read_model_folder(folder)
    a, b = random_tokens(40, 75, cfg["vocab"]), random_tokens(41, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[70]], "want": []}, {"id": "b", "tokens": [b[5]], "want": [0]}], "end": []}]
    steps += [{"step": 2 + t, "entries": [{"id": "a", "tokens": [a[71 + t]], "want": [0]}] + ([{"id": "b", "tokens": [b[6 + t]], "want": [0]}] if t < 3 else []),
               "end": ["b"] if t == 2 else []} for t in range(4)]
    out = tmp_path / "out"
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                               "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
        wa, wb = P.forward(cfg, tensors, a), P.forward(cfg, tensors, b)
        read = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        assert row_error(read(0), np.stack([wa[0], wa[69], wb[4]])).max() < tol
        assert row_error(read(1), wb[5][None]).max() < tol
        for t in range(4):
            rows = [wa[71 + t]] + ([wb[6 + t]] if t < 3 else [])
            assert row_error(read(2 + t), np.stack(rows)).max() < tol, t


def test_the_command_line_on_the_preset(tmp_path):
    program = [sys.executable, os.path.join(ROOT, "bin", "burn-lm")]
    folder = str(tmp_path / "n")
    r = subprocess.run(program + ["random", folder, "--preset", "nufolix_tiny", "--seed", "4", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and f"wrote {folder}" in r.stdout, r.stderr
    cfg, tensors = P.read_model_folder(folder)
    prompt = random_tokens(5, 23, cfg["vocab"])
    want = P.greedy(cfg, tensors, prompt, 12)
    r = subprocess.run(program + ["run", folder, "--dtype", "float32", "--sample-len", "12", "--max-seq-len", "128",
                                  ",".join(map(str, prompt))], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert lines[0].split() == [str(t) for t in want], (lines[0], want)


def test_sampling_with_a_temperature_runs_inside_the_captured_step(tmp_path):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "nuf_a")
    lm = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=2)
    prompts = [random_tokens(50, 20, 320), random_tokens(51, 66, 320)]
    a = lm.generate(prompts, sample_len=12, temperature=0.8, seed=7, ignore_stop=True).tokens
    b = lm.generate(prompts, sample_len=12, temperature=0.8, seed=7, ignore_stop=True).tokens
    assert a == b and all(len(t) == 12 for t in a)          # the same draws from the same seed, through used slots


def test_a_slowly_decaying_head_keeps_its_long_past_in_the_32_bit_path():
    """Decays close to 1 sum hundreds of tokens into a state far larger than its read-out; with sums held in float64 inside a
    step the read-out stays within float32 rounding of the plain implementation, also across portions."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(12)
    heads, groups, n_state, dv, n = 2, 1, 40, 24, 900
    x, B, C = rng.normal(size=(n, heads, dv)), rng.normal(size=(n, groups, n_state)), rng.normal(size=(n, groups, n_state))
    dt_raw = rng.normal(size=(n, heads)) - 5.0                       # softplus(-5) = 0.007: a memory of hundreds of tokens
    a_log, d_skip, dt_bias = np.zeros(heads), np.ones(heads), np.zeros(heads)
    f32 = lambda t: t.astype(np.float32).astype(np.float64)
    want = P.mamba2_scan(f32(x), f32(B), f32(C), P.softplus(f32(dt_raw)), a_log, d_skip, heads, groups).reshape(n, -1)
    state = torch.zeros((1, 2, K.scan_state_floats(heads, n_state, dv)), device="cuda")
    outs, at = [], 0
    for portion in (500, 1, 1, 398):
        st = step_of((portion,), [0], [at])
        sl = slice(at, at + portion)
        xbc = dev(np.concatenate([x[sl].reshape(portion, -1), B[sl].reshape(portion, -1), C[sl].reshape(portion, -1)], axis=1))
        y = torch.zeros((portion, heads * dv), device="cuda")
        K.ssm_scan(xbc, 0, heads * dv, heads * dv + groups * n_state, dev(dt_raw[sl]), 0, dev(dt_bias), dev(a_log), dev(d_skip), y, heads,
                   groups, n_state, dv, st, state, 0, wide_sums=True)
        outs.append(y.cpu().numpy())
        at += portion
    err = np.abs(np.concatenate(outs) - want).max(axis=1) / np.abs(want).max(axis=1)
    assert err.max() < 2e-6, err.max()


@pytest.mark.parametrize("kinds", ["mamba2 only", "parallel only", "mamba2 last"])
def test_models_of_one_kind_of_layer(tmp_path, kinds):
    """No keys and values at all, no recurrent layer of the first kind at all, and another order of layers."""
    from burn_lm_b200 import write_random_model
    from nufolix_tiny import mamba2, model, parallel
    layers = {"mamba2 only": [mamba2(2, 16, 8, 1, 3, 1, 40), mamba2(4, 8, 16, 2, 2, 2, None)],
              "parallel only": [parallel(2, 1, 16, 8, 8, 2, 2, 8, 16, 2, None), parallel(3, 3, 8, 16, 0, 1, 1, 16, 8, 3, 24)],
              "mamba2 last": [parallel(2, 2, 16, 16, 16, 2, 1, 16, 16, 4, 32), parallel(4, 2, 8, 8, 4, 4, 4, 8, 8, 2, None),
                              mamba2(3, 8, 8, 3, 4, 3, None)]}[kinds]
    cfg = model(97, 48, layers)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=3, dtype="bfloat16")
    pcfg, tensors = P.read_model_folder(folder)
    tokens = random_tokens(7, 90, 97)
    want = P.forward(pcfg, tensors, tokens)
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        engine = engine_for(folder, dtype)
        assert row_error(_logits(engine, tokens, list(range(90)), [70] + [1] * 20), want).max() < tol
        assert row_error(_logits(engine, tokens, list(range(90)), [3, 64, 2, 21]), want).max() < tol

"""The Fobilorn decoder in the engine against the plain implementation (tests/plain/fobilorn_plain.py): every
mechanism's kernels alone, then whole models through the step function, the cache, the scheduler and generation."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import fobilorn_plain as P
from fobilorn_tiny import CONFIGS, make_folder, random_tokens, row_error
import traces

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 4e-2
PAGE = 64


def dev(x, dtype=torch.float32):
    return torch.tensor(np.asarray(x), dtype=dtype, device="cuda")


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device="cuda")


def step_of(positions, seq_of=None, slots=(0,)):
    """What the kernels read of a step: the rows' sequences and positions."""
    n = len(positions)
    seq_of = list(seq_of) if seq_of is not None else [0] * n
    cu, starts = [0], []
    for s in range(len(slots)):
        cu.append(cu[-1] + sum(1 for x in seq_of if x == s))
        starts.append(next((p for p, x in zip(positions, seq_of) if x == s), 0))
    return SimpleNamespace(token_seq=ints(seq_of), token_pos=ints(positions), slot_of_seq=ints(slots), cu_seqlens=ints(cu),
                           start_pos=ints(starts), n_tokens=n)


def engine_for(folder, dtype, max_tokens=4096, **kw):
    from burn_lm_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


# ---------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_adds_and_squashes(dtype):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(0)
    n, d = 7, 100
    x = rng.normal(size=(n, d)) * 2
    deltas = [rng.normal(size=(n, d)) for _ in range(3)]
    w, b, alpha = rng.normal(size=d) + 1, rng.normal(size=d), 0.7
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for k in range(4):
        resid = dev(x)
        ds = [dev(t, dtype) for t in deltas[:k]]
        out = torch.empty((n, d), dtype=dtype, device="cuda")
        K.add_dyt(resid, ds, dev(w), dev(b), dev([alpha]), out)
        total = x + sum(t.float().cpu().numpy().astype(np.float64) for t in ds) if k else x
        assert np.abs(resid.cpu().numpy() - total).max() < 1e-5                # the stream took the sum, in fp32
        want = P.dynamic_tanh(total, w, b, alpha)
        assert np.abs(out.float().cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())
    # some rows only: the stream stays as it was
    resid = dev(x)
    rows = [5, 0, 5]
    out = torch.empty((3, d), dtype=dtype, device="cuda")
    K.add_dyt(resid, [dev(deltas[0], dtype)], dev(w), dev(b), dev([alpha]), out, rows=ints(rows))
    assert np.array_equal(resid.cpu().numpy(), x.astype(np.float32))
    want = P.dynamic_tanh((x + dev(deltas[0], dtype).float().cpu().numpy())[rows], w, b, alpha)
    assert np.abs(out.float().cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())


def test_pair_embedding_keeps_the_previous_token_by_position():
    """Portions of a sequence, two sequences side by side, a slot's pages handed to another sequence: the row of the
    table of pairs always comes from the token one position back, and from the last row at position 0."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(1)
    vocab, d, buckets, mp, mc = 50, 24, 13, 1000003, 7
    table, pairs = rng.normal(size=(vocab, d)), rng.normal(size=(buckets + 1, d))
    w, b, alpha = rng.normal(size=d) + 1, rng.normal(size=d), 1.3
    ids_pool = torch.full((6, PAGE), -7, dtype=torch.int32, device="cuda")         # rubbish that must never be read
    block_table = ints([2, 5, 0, 0, 4, 1, 0, 0]).reshape(2, 4)
    seqs = {0: random_tokens(3, 130, vocab), 1: random_tokens(4, 70, vocab)}
    want = {s: P.dynamic_tanh(P.embedding(t, table, pairs, buckets, mp, mc), w, b, alpha) for s, t in seqs.items()}
    at = {0: 0, 1: 0}
    for portion in [(63, 5), (2, 1), (1, 60), (64, 4)]:          # (tokens of sequence 0, of sequence 1); borders of pages inside
        toks, seq_of, pos = [], [], []
        for s, k in enumerate(portion):
            toks += seqs[s][at[s]: at[s] + k]
            seq_of += [s] * k
            pos += list(range(at[s], at[s] + k))
        st = step_of(pos, seq_of, slots=(0, 1))
        out = torch.empty((len(toks), d), dtype=torch.float32, device="cuda")
        K.embed_pairs(ints(toks), dev(table), dev(pairs), out, st, ids_pool, block_table, buckets, mp, mc,
                      norm=(dev(w), dev(b), dev([alpha])))
        row = 0
        for s, k in enumerate(portion):
            assert np.abs(out[row: row + k].cpu().numpy() - want[s][at[s]: at[s] + k]).max() < 1e-5, (portion, s)
            row += k
            at[s] += k
    # the same step again (a captured step's warm-up, say) changes nothing: the line is written by position
    again = torch.empty_like(out)
    K.embed_pairs(ints(toks), dev(table), dev(pairs), again, st, ids_pool, block_table, buckets, mp, mc,
                  norm=(dev(w), dev(b), dev([alpha])))
    assert torch.equal(out, again)
    # rows of no sequence take the first-token row and write nothing
    before = ids_pool.clone()
    st = step_of([0, 0], [-1, -1], slots=(0,))
    out = torch.empty((2, d), dtype=torch.float32, device="cuda")
    K.embed_pairs(ints([3, 4]), dev(table), dev(pairs), out, st, ids_pool, block_table, buckets, mp, mc)
    assert torch.equal(before, ids_pool)
    assert np.abs(out.cpu().numpy() - (table[[3, 4]] + pairs[buckets])).max() < 1e-5


def _append_and_attend(dtype, q, k, v, positions, block_table, n_pages, scale, window, keep, sink=True, gate=None, pool=None,
                       n_splits=1):
    """Append rows (one sequence in slot 0) and attend; q [T, H, dk], k [T, G, dk], v [T, G, dv] given as they enter the
    scores (no norm).  Returns (out [T, H, dv], pool).  Portions of 8 rows and more in bfloat16 with sizes in multiples of
    8 run the tensor-core prompt kernel, all else the row kernel (its keys cut over `n_splits` blocks)."""
    from burn_lm_b200 import kernels as K
    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    if pool is None:
        pool = torch.full((n_pages, K.kv_page_elems(G, dk, dv)), float("nan"), dtype=dtype, device="cuda")
    cols = [q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)] + ([gate] if gate is not None else [])
    proj = dev(np.concatenate(cols, axis=1))
    st = step_of(positions)
    q_out = torch.empty((T, H * dk), dtype=dtype, device="cuda")
    K.qk_norm_append(proj, st, pool, block_table, q_out, H, G, dk, dv)
    out = torch.empty((T, H * dv), dtype=dtype, device="cuda")
    scratch = torch.empty(K.attention_sink_scratch_floats(T, H, dv, n_splits), dtype=torch.float32, device="cuda") if n_splits > 1 else None
    K.attention_sink(q_out, st, pool, block_table, out, H, G, dk, dv, scale, window, keep, sink=sink,
                     gate=proj[:, (H + G) * dk + G * dv:] if gate is not None else None, gate_stride=proj.stride(0),
                     max_q_len=T, n_splits=n_splits, scratch=scratch)
    return out.float().cpu().numpy().reshape(T, H, dv), pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,window,keep", [(4, 2, 16, 8, 50, 3), (3, 3, 24, 40, 64, 0), (8, 1, 12, 12, 7, 66), (2, 1, 40, 260 // 10, 1000, 0),
                                                   (4, 2, 128, 128, 90, 5), (2, 2, 64, 72, 33, 0), (20, 1, 32, 32, 64, 64)])
def test_attention_against_plain_in_prompts_and_token_by_token(dtype, H, G, dk, dv, window, keep):
    """A prompt in one step, the same in portions, then single tokens: windows and kept first tokens that cross pages,
    pages out of order, the sink, the gate."""
    rng = np.random.default_rng(2)
    T = 200
    q, k, v = rng.normal(size=(T, H, dk)), rng.normal(size=(T, G, dk)), rng.normal(size=(T, G, dv))
    gate = rng.normal(size=(T, H))
    scale = 1.5 * dk ** -0.5
    if dtype == torch.bfloat16:          # what the cache rounds
        q, k, v = (dev(t, dtype).float().cpu().numpy().astype(np.float64) for t in (q, k, v))
    want = np.stack([P.attend(q[:, h], k[:, h // (H // G)], v[:, h // (H // G)], scale, window, keep) * P.sigmoid(gate[:, h:h + 1])
                     for h in range(H)], axis=1)
    block_table = ints([5, 2, 7, 0, 3, 0, 0, 0]).reshape(1, 8)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for cuts in ([T], [64, 1, 63, 2, 70], [130] + [1] * 70, [9, 100, 7, 84]):
        pool, at = None, 0
        for n in cuts:
            sl = slice(at, at + n)
            got, pool = _append_and_attend(dtype, q[sl], k[sl], v[sl], range(at, at + n), block_table, 8, scale, window, keep,
                                           gate=gate[sl], pool=pool, n_splits=3 if n < 8 and at > 100 else 1)
            assert np.abs(got - want[sl]).max() < tol * np.abs(want).max(), (cuts[:3], at, n)
            at += n
    # without the sink and without a gate the same kernel is a plain windowed softmax
    got, _ = _append_and_attend(dtype, q, k, v, range(T), block_table, 8, scale, window, keep, sink=False)
    plain = np.stack([P.attend(q[:, h], k[:, h // (H // G)], v[:, h // (H // G)], scale, window, keep, sink=False) for h in range(H)], axis=1)
    assert np.abs(got - plain).max() < tol * np.abs(plain).max()
    assert np.abs(plain - want).max() > 0.05          # and the sink is not nothing


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_key_that_stands_out_is_seen_exactly_where_the_mask_says(dtype):
    """One key's score is made to tower over all others and its value is a mark of its own.  Far back among hundreds,
    at the borders of pages, just inside and just outside the window and the kept first tokens: the output is the
    mark exactly when the design lets the query see the key, in a prompt's step and for a token decoded alone."""
    rng = np.random.default_rng(3)
    T, dk, dv, window, keep = 400, 16, 8, 100, 10
    scale = 1.0
    block_table = ints([6, 1, 4, 0, 5, 2, 3, 7]).reshape(1, 8)
    probes = [(399, 300), (399, 299), (399, 9), (399, 10), (399, 0), (399, 399), (300, 201), (300, 200), (164, 65), (164, 64),
              (163, 64), (163, 63), (128, 127), (128, 29), (128, 28), (64, 63), (64, 0), (109, 10), (108, 9), (5, 0), (0, 0)]
    for i, j in probes:
        q, k, v = rng.normal(size=(T, 1, dk)) * 0.1, rng.normal(size=(T, 1, dk)) * 0.1, rng.normal(size=(T, 1, dv)) * 0.1
        u = np.zeros(dk)
        u[j % dk] = 1.0
        k[j, 0], q[i, 0] = 40.0 * u, u
        v[j, 0] = 5.0 + np.arange(dv)
        if dtype == torch.bfloat16:
            q, k, v = (dev(t, dtype).float().cpu().numpy().astype(np.float64) for t in (q, k, v))
        tol = 1e-4 if dtype == torch.float32 else 1e-1     # marks of 5 to 12 in bfloat16
        sees = P.visible(i, j, window, keep)
        assert sees == (j <= i and (i - j < window or j < keep))
        want = P.attend(q[:, 0], k[:, 0], v[:, 0], scale, window, keep)
        assert (np.abs(want[i] - v[j, 0]).max() < 1e-3) == sees, (i, j)
        # the prompt in one step
        got, pool = _append_and_attend(dtype, q, k, v, range(T), block_table, 8, scale, window, keep)
        assert np.abs(got[:, 0] - want).max() < tol, ("prompt", i, j)
        assert (np.abs(got[i, 0] - v[j, 0]).max() < 10 * tol) == sees, ("prompt", i, j)
        # the query decoded alone over the cache the prompt left, its keys in one block and cut over several
        for n_splits in (1, 4):
            one, _ = _append_and_attend(dtype, q[i:i + 1], k[i:i + 1], v[i:i + 1], [i], block_table, 8, scale, window, keep, pool=pool,
                                        n_splits=n_splits)
            assert np.abs(one[0, 0] - want[i]).max() < tol, ("decoded", i, j, n_splits)
            assert (np.abs(one[0, 0] - v[j, 0]).max() < 10 * tol) == sees, ("decoded", i, j, n_splits)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_projection_norm_and_value_blend(dtype):
    """q and k are divided by the root mean square of the whole row, not per head; blended values are what is cached
    and what a later layer would see."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(4)
    T, H, G, dk, dv, eps = 9, 3, 1, 8, 6, 1e-3
    qc, kc, vc = H * dk, G * dk, G * dv
    proj = rng.normal(size=(T, qc + kc + vc + H))
    proj[:, :dk] *= 20.0                  # one head much larger than the others: a per-head norm would give other numbers
    wq, wk, lam = rng.normal(size=qc) + 1, rng.normal(size=kc) + 1, 0.3
    v_first = rng.normal(size=(T, vc))
    pool = torch.zeros((2, K.kv_page_elems(G, dk, dv)), dtype=dtype, device="cuda")
    bt = ints([1, 0]).reshape(1, 2)
    st = step_of(range(60, 60 + T))       # the rows cross from the first page of the sequence into its second
    q_out = torch.empty((T, qc), dtype=dtype, device="cuda")
    v_out = torch.empty((T, vc), dtype=torch.float32, device="cuda")
    K.qk_norm_append(dev(proj), st, pool, bt, q_out, H, G, dk, dv, q_weight=dev(wq), k_weight=dev(wk), eps=eps, blend=dev([lam]),
                     values_in=dev(v_first), values_out=v_out)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    want_q = P.rms_unit(proj[:, :qc], eps) * wq
    per_head = (P.rms_unit(proj[:, :qc].reshape(T, H, dk), eps).reshape(T, qc)) * wq
    assert np.abs(want_q - per_head).max() > 0.5
    assert np.abs(q_out.float().cpu().numpy() - want_q).max() < tol * np.abs(want_q).max()
    want_k = P.rms_unit(proj[:, qc:qc + kc], eps) * wk
    want_v = (1 - lam) * proj[:, qc + kc: qc + kc + vc] + lam * v_first
    assert np.abs(v_out.cpu().numpy() - want_v).max() < 1e-5
    pages = pool.float().cpu().numpy()
    for t in range(T):
        pos = 60 + t
        page, r = (1, pos) if pos < 64 else (0, pos - 64)
        got_k = pages[page][: G * PAGE * dk].reshape(G, PAGE, dk)[:, r].reshape(-1)
        got_v = pages[page][G * PAGE * dk:].reshape(G, PAGE, dv)[:, r].reshape(-1)
        assert np.abs(got_k - want_k[t]).max() < tol * np.abs(want_k).max()
        assert np.abs(got_v - want_v[t]).max() < tol * np.abs(want_v).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff,shared", [(6, 2, 24, True), (1, 1, 40, False), (5, 5, 8, True), (9, 1, 33, False)])
def test_mixture_of_experts_against_plain(dtype, experts, top, ff, shared):
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(5)
    n, d = 77, 48
    h = dev(rng.normal(size=(n, d)), dtype)
    hp = h.float().cpu().numpy().astype(np.float64)
    w = {"router": rng.normal(size=(experts, d)) * 0.5}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (rng.normal(size=(ff, d)) * 0.3, rng.normal(size=(ff, d)) * 0.3,
                                                           rng.normal(size=(d, ff)) * 0.3)
    if dtype == torch.bfloat16:
        w = {k: (dev(v, dtype).float().cpu().numpy().astype(np.float64) if k != "router" else v) for k, v in w.items()}
    ids, weights = K.moe_route(h, dev(w["router"]), top)
    want_ids, want_w = P.route(hp, w["router"], top)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.abs(weights.cpu().numpy() - want_w).max() < 1e-5
    gate_up = dev(np.stack([np.concatenate([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]), dtype)
    down = dev(np.stack([w[f"e{e}.down"] for e in range(experts)]), dtype)
    extra = dev(rng.normal(size=(n, d)), dtype) if shared else None
    add = extra.float().cpu().numpy() if shared else 0.0
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    want_in = P.moe_ff(hp, w, experts, top, False) + add
    want_out = P.moe_ff(hp, w, experts, top, False, on_input=False) + add
    assert np.abs(want_in - want_out).max() > 0.05 * np.abs(want_in).max()      # where the weight stands matters
    got = K.moe_experts(h, ids, weights, gate_up, down, extra=extra, weight_on_input=True).float().cpu().numpy()
    assert np.abs(got - want_in).max() < tol * np.abs(want_in).max()
    got = K.moe_experts(h, ids, weights, gate_up, down, extra=extra, weight_on_input=False).float().cpu().numpy()
    assert np.abs(got - want_out).max() < tol * np.abs(want_out).max()


def test_rows_of_no_sequence_may_hold_anything():
    """A captured prompt step is padded with rows that belong to no sequence; after the first layer they may hold
    anything, a NaN too.  The router still names experts that exist for them, the other rows' results do not change,
    and the prompt kernel leaves zeros in them."""
    from burn_lm_b200 import kernels as K
    rng = np.random.default_rng(6)
    n, d, experts, top, ff = 40, 32, 5, 2, 16
    h = dev(rng.normal(size=(n, d)), torch.bfloat16)
    router = dev(rng.normal(size=(experts, d)))
    gate_up = dev(rng.normal(size=(experts, 2 * ff, d)) * 0.3, torch.bfloat16)
    down = dev(rng.normal(size=(experts, d, ff)) * 0.3, torch.bfloat16)
    ids, w = K.moe_route(h, router, top)
    clean = K.moe_experts(h, ids, w, gate_up, down)
    h2 = h.clone()
    h2[33:] = float("nan")
    ids2, w2 = K.moe_route(h2, router, top)
    assert int(ids2.min()) >= 0 and int(ids2.max()) < experts
    got = K.moe_experts(h2, ids2, w2, gate_up, down)
    assert torch.equal(got[:33], clean[:33])
    # the prompt kernel: 20 rows of a sequence, 12 of none
    H, G, dk, dv = 2, 1, 16, 8
    pool = torch.zeros((2, K.kv_page_elems(G, dk, dv)), dtype=torch.bfloat16, device="cuda")
    st = step_of(list(range(20)) + [0] * 12, [0] * 20 + [-1] * 12)
    proj = dev(rng.normal(size=(32, (H + G) * dk + G * dv)))
    q = torch.empty((32, H * dk), dtype=torch.bfloat16, device="cuda")
    bt = ints([1, 0]).reshape(1, 2)
    K.qk_norm_append(proj, st, pool, bt, q, H, G, dk, dv)
    out = torch.full((32, H * dv), float("nan"), dtype=torch.bfloat16, device="cuda")
    K.attention_sink(q, st, pool, bt, out, H, G, dk, dv, 0.5, 16, 2, max_q_len=32)
    assert bool(torch.isfinite(out).all()) and float(out[20:].abs().max()) == 0.0 and float(out[:20].abs().max()) > 0.0


# ---------------------------------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,stored,tolerance", [("float32", "float32", FP32_TOL), ("float32", "bfloat16", FP32_TOL),
                                                    ("bfloat16", "bfloat16", BF16_TOL)])
def test_whole_prompts(tmp_path, name, dtype, stored, tolerance):
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name, seed=3, dtype=stored)
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, dtype)
    for n, length in enumerate([1, 2, 5, 64, 65, 150]):
        toks = random_tokens(10 + n, length, cfg["vocab"])
        slot = eng.acquire()
        got = eng.step([StepEntry(slot, toks, list(range(length)))]).cpu().numpy()
        eng.release(slot)
        want = P.forward(cfg, tensors, toks)
        err = row_error(got, want)
        assert err.max() < tolerance, (name, dtype, length, err.max(), int(err.argmax()))


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_layer_in_32_bit(tmp_path, name):
    """The stream after every layer, read back from the model's forward by cutting the schedule short."""
    from burn_lm_b200 import Engine, StepEntry
    from burn_lm_b200.model import load_model
    folder = make_folder(tmp_path, name, seed=8, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    toks = random_tokens(5, 90, cfg["vocab"])
    _, streams = P.forward(cfg, tensors, toks, return_layers=True)
    model = load_model(folder, "float32")
    eng = Engine(model, max_tokens=256)
    seen = []
    for layer in model.layers:                   # watch the stream through the norm that reads it next
        norm, inner = layer.block.norm, layer.block.norm.add_norm
        def spy(resid, delta, rows=None, lazy=False, handoff=None, inner=inner):
            out = inner(resid, delta, rows=rows, lazy=lazy, handoff=handoff)
            seen.append(resid.clone())
            return out
        norm.add_norm = spy
    slot = eng.acquire()
    eng.use_graphs = False
    eng.step([StepEntry(slot, toks, [])])
    assert len(seen) == len(cfg["layers"])
    for i in range(1, len(seen)):                # the norm of layer i has just added layer i - 1's outputs
        got = seen[i].cpu().numpy()
        assert np.abs(got - streams[i - 1]).max() < 1e-4 * np.abs(streams[i - 1]).max(), i


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_portions_and_decoding_against_the_whole_prompt(tmp_path, name, dtype, tolerance):
    """A prompt cut into portions of several sizes, down to two tokens and one, then decoded token by token past
    every window of the configuration: every position's logits against the plain implementation on the whole."""
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name, seed=4, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, dtype)
    toks = random_tokens(21, 330, cfg["vocab"])
    want = P.forward(cfg, tensors, toks)
    for cuts in ([64, 2, 62, 3, 1, 17], [130, 2], [1, 1, 2, 60, 64]):
        cuts = cuts + [1] * (len(toks) - sum(cuts))
        slot = eng.acquire()
        at, rows = 0, []
        for n in cuts:
            rows.append(eng.step([StepEntry(slot, toks[at: at + n], list(range(n)))]).cpu().numpy().copy())
            at += n
        eng.release(slot)
        err = row_error(np.concatenate(rows), want)
        assert err.max() < tolerance, (name, dtype, cuts[:6], err.max(), int(err.argmax()))
    assert eng.cache.free_pages == eng.cache.n_pages


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_batches_of_unequal_requests_and_reused_pages(tmp_path, name, dtype, tolerance):
    """Requests of unequal lengths start together and are decoded together, the shorter ones ending earlier, batch
    after batch in a cache so small that pages and slots are used again; every request against itself alone."""
    folder = make_folder(tmp_path, name, seed=6, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    lengths = [1, 70, 33, 129, 2, 200, 64, 90, 17]
    requests = {f"r{i}": random_tokens(40 + i, n, cfg["vocab"]) for i, n in enumerate(lengths)}
    steps = traces.batched(requests, 3, [5, 40, 1])
    eng = engine_for(folder, dtype, max_tokens=traces.max_live_tokens(steps))
    got = traces.run_in_process(eng, steps, str(tmp_path / "out"), cfg["vocab"])
    for rid, toks in requests.items():
        err = row_error(got[rid], P.forward(cfg, tensors, toks))
        assert err.max() < tolerance, (name, dtype, rid, err.max(), int(err.argmax()))
    # the same requests in other company and other slots: the same logits beyond rounding
    steps2 = traces.batched(dict(reversed(list(requests.items()))), 4, [2, 9, 30, 1])
    eng2 = engine_for(folder, dtype, max_tokens=traces.max_live_tokens(steps2))
    got2 = traces.run_in_process(eng2, steps2, str(tmp_path / "out2"), cfg["vocab"])
    for rid in requests:
        assert row_error(got2[rid], got[rid]).max() < (1e-5 if dtype == "float32" else tolerance), rid


def test_long_decoding_gives_pages_back_and_keeps_the_first(tmp_path):
    """Hundreds of tokens decoded one by one: the windowed lines hold a few pages only, the kept first tokens stay, and
    the logits still agree with the plain implementation at the end."""
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, "fob_c", seed=9, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, "float32", max_tokens=64 * 12)
    toks = random_tokens(77, 700, cfg["vocab"])
    slot = eng.acquire()
    eng.step([StepEntry(slot, toks[:3], [])])
    rows = {}
    for p in range(3, len(toks)):
        out = eng.step([StepEntry(slot, [toks[p]], [0])])
        if p % 97 == 0 or p >= len(toks) - 3:
            rows[p] = out.cpu().numpy()[0].copy()
    held = {g.need: len(g.live_pages(slot)) for g in eng.cache._kv_groups}
    for need, pages in held.items():
        if need.window:
            assert pages <= (need.window + PAGE - 1) // PAGE + 1 + (need.keep_first + PAGE - 1) // PAGE, need
    want = P.forward(cfg, tensors, toks)
    for p, got in rows.items():
        assert row_error(got[None], want[p:p + 1]).max() < FP32_TOL, p
    eng.release(slot)
    assert eng.cache.free_pages == eng.cache.n_pages


@pytest.mark.parametrize("name", ["fob_a", "fob_c"])
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    """burn_lm_b200.load(...).generate(...): prompts of unequal lengths in batches, greedy, against greedy decoding with
    the plain implementation."""
    import burn_lm_b200 as B
    folder = make_folder(tmp_path, name, seed=12, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    lm = B.load(folder, dtype="float32", max_seq_len=256, max_batch=3)
    prompts = [random_tokens(60 + i, n, cfg["vocab"]) for i, n in enumerate([1, 9, 66, 30])]
    n_new = 12
    out = lm.generate(prompts, temperature=0.0, sample_len=n_new, ignore_stop=True, batch_size=3)
    for prompt, res in zip(prompts, out.results):
        seq = list(prompt)
        for _ in range(n_new):
            logits = P.forward(cfg, tensors, seq)[-1]
            top2 = np.sort(logits)[-2:]
            nxt = int(np.argmax(logits))
            if top2[1] - top2[0] < 1e-3 * np.abs(logits).max():
                break                                    # a close call decides nothing
            seq.append(nxt)
        made = seq[len(prompt):]
        assert list(res.tokens)[: len(made)] == made, (name, len(prompt))
    # the same through captured decode steps that feed themselves on the device
    eng = lm.engine
    slots = [eng.acquire() for _ in prompts[:2]]
    from burn_lm_b200 import StepEntry
    first = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts[:2])]).argmax(dim=-1).tolist()
    hist = eng.decode_run(slots, first, 6).cpu().numpy()
    for i, res in enumerate(out.results[:2]):
        assert [first[i]] + hist[:-1, i].tolist() == list(res.tokens)[:6] or len(res.tokens) < 6


def test_the_command_line_serves_the_design(tmp_path):
    """`bin/burn-lm random --preset fobilorn_tiny` writes a folder, `bin/burn-lm run` generates from it in a child
    process; the tokens are the plain implementation's greedy ones."""
    import subprocess
    import sys
    program = [sys.executable, os.path.join(traces.ROOT, "bin", "burn-lm")]
    folder = str(tmp_path / "f")
    r = subprocess.run(program + ["random", folder, "--preset", "fobilorn_tiny", "--seed", "4", "--dtype", "bfloat16"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and f"wrote {folder}" in r.stdout, r.stderr
    cfg, tensors = P.read_model_folder(folder)
    prompt = random_tokens(5, 23, cfg["vocab"])
    r = subprocess.run(program + ["run", folder, "--dtype", "float32", "--sample-len", "10", "--max-seq-len", "128",
                                  ",".join(map(str, prompt))], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = [int(t) for t in [ln for ln in r.stdout.splitlines() if ln.strip()][0].split()]
    seq = list(prompt)
    for t in got:
        logits = P.forward(cfg, tensors, seq)[-1]
        order = np.argsort(logits)
        if logits[order[-1]] - logits[order[-2]] < 1e-3 * np.abs(logits).max():
            break                                        # a close call decides nothing
        assert t == int(order[-1]), (len(seq) - len(prompt), t)
        seq.append(t)
    assert len(got) == 10 and len(seq) > len(prompt)
    r = subprocess.run(program + ["models"], capture_output=True, text=True, timeout=300)
    assert "Fobilorn" in r.stdout and "fobilorn_tiny" in r.stdout


def test_trace_runner_chooses_the_model_by_its_configuration(tmp_path):
    """bin/trace_run on a Fobilorn folder: whole prompts, then the same decoded and batched, in 32-bit."""
    folder = make_folder(tmp_path, "fob_a", seed=2, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    requests = {f"q{i}": random_tokens(90 + i, n, cfg["vocab"]) for i, n in enumerate([1, 40, 75])}
    steps = traces.whole(requests) + traces.tail({k + "t": v for k, v in requests.items()}, 8, first_step=10) \
        + traces.batched({k + "b": v for k, v in requests.items()}, 3, [3, 1, 6], first_step=100)
    got = traces.run_program(folder, "float32", steps, str(tmp_path / "o"), cfg["vocab"])
    for rid, toks in requests.items():
        want = P.forward(cfg, tensors, toks)
        for suffix in ("", "t", "b"):
            assert row_error(got[rid + suffix], want).max() < FP32_TOL, rid + suffix


def test_trace_runner_has_room_for_partly_filled_pages(tmp_path):
    """--max-tokens counts the tokens requests hold, not pages: requests of 1, 65 and 129 tokens together hold 195
    tokens and six pages of 64 when no window lets pages go."""
    folder = make_folder(tmp_path, "fob_b", seed=2, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    requests = {f"q{i}": random_tokens(70 + i, n, cfg["vocab"]) for i, n in enumerate([1, 65, 129])}
    steps = traces.batched(requests, 3, [1, 4, 2])
    got = traces.run_program(folder, "float32", steps, str(tmp_path / "o"), cfg["vocab"], max_tokens=195)
    for rid, toks in requests.items():
        assert row_error(got[rid], P.forward(cfg, tensors, toks)).max() < FP32_TOL, rid

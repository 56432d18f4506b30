"""The Nufolix decoder without a GPU: its configuration, its plan and stored names, the cache of a run that keeps two
things, and the plain implementation's mechanisms against closed forms."""
import copy

import numpy as np
import pytest

from plain import nufolix_plain as P
from nufolix_tiny import CONFIGS, NUF_A, make_folder, random_tokens


def test_configuration_round_trip_and_errors():
    from burn_lm_b200.config import ConfigError, NufolixConfig
    for cfg in CONFIGS.values():
        typed = NufolixConfig.from_dict(cfg)
        assert NufolixConfig.from_dict(typed.to_dict()) == typed
        assert len(typed.layers) == len(cfg["layers"])
    for path, value, key in ((("layers", 0, "type"), "conv", "layers[0].type"),
                             (("layers", 1, "mixer", "left", "kv_heads"), 3, "layers[1].mixer.left.kv_heads"),
                             (("layers", 1, "mixer", "left", "rot", "dims"), 7, "layers[1].mixer.left.rot.dims"),
                             (("layers", 1, "mixer", "right", "conv"), 0, "layers[1].mixer.right.conv"),
                             (("layers", 0, "mixer", "groups"), 4, "layers[0].mixer.groups"),
                             (("layers", 0, "mixer", "norm_groups"), 5, "layers[0].mixer.norm_groups"),
                             (("layers", 1, "mlp", "kind"), "moe", "layers[1].mlp.kind"),
                             (("residual_mult",), "x", "residual_mult"), (("embedding", "scale"), None, "embedding.scale")):
        bad = copy.deepcopy(NUF_A)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=key.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
            NufolixConfig.from_dict(bad)


def test_the_plan_names_the_stored_tensors():
    from burn_lm_b200.model import plan_of, tensor_specs_of
    arch, typed, plan = plan_of(NUF_A)
    assert arch.name == "Nufolix" and plan.head.tensors["weight"] == plan.embedding.tensors["table"] == "embed"
    names = {s.name: tuple(s.shape) for s in tensor_specs_of(NUF_A)}
    assert names["embed"] == (320, 96) and names["final.norm"] == (96,)
    assert names["l0.mix.in"] == (2 * 96 + 2 * 2 * 24 + 6, 96) and names["l0.mix.conv"] == (96 + 96, 4) and "l0.norm2" not in names
    assert names["l1.mix.left.q.b"] == (96,) and names["l1.mix.left.talk"] == (4, 4) and names["l1.mix.left.pb"] == (4,)
    assert names["l1.mix.right.v.conv"] == (96, 3) and names["l1.mix.right.dt_bias"] == (4 * 16,) and names["l1.mlp.act"] == (2,)
    assert names["l1.mix.right.a1"] == (-1, 96) and names["l1.mix.right.g2"] == (96, -1)       # read off the stored tensors
    assert {"l1.norm1", "l1.norm1b", "l1.norm2", "l1.norm2b", "l3.norm1b"} <= set(names) and "l3.norm2b" not in names


def test_a_free_dimension_is_read_from_the_stored_tensor(tmp_path):
    import torch
    from burn_lm_b200.weights.loader import TensorSpec, WeightsError, load_tensors, shape_fits
    from burn_lm_b200.weights.safetensors_io import write_safetensors
    assert shape_fits((-1, 4), (9, 4)) and not shape_fits((-1, 4), (9, 5)) and not shape_fits((-1, 4), (4,))
    write_safetensors(str(tmp_path / "model.safetensors"), {"a": torch.zeros(7, 4), "b": torch.zeros(3, 7)})
    got = load_tensors(str(tmp_path), [TensorSpec("a", (-1, 4)), TensorSpec("b", (3, -1))], torch.float32, "cpu")
    assert tuple(got["a"].shape) == (7, 4) and tuple(got["b"].shape) == (3, 7)
    with pytest.raises(WeightsError):
        load_tensors(str(tmp_path), [TensorSpec("a", (-1, 5)), TensorSpec("b", (3, -1))], torch.float32, "cpu")


def test_a_run_that_keeps_keys_and_a_state():
    import torch
    from burn_lm_b200.cache import Cache
    from burn_lm_b200.parts.base import CacheNeed
    from burn_lm_b200.plan import ScheduleEntry
    kv = CacheNeed("kv", n_kv_heads=2, head_dim=8, value_dim=4)
    state = CacheNeed("state", state_shape=(2, 10))
    other = CacheNeed("state", state_shape=(2, 6))
    cache = Cache([(kv, state), other, (kv, state)], [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)], 256, 3, 256,
                  torch.float32, "cpu")
    v0, v1, v2 = cache.view(0), cache.view(1), cache.view(2)
    assert v0.kind == "kv+state" and v0.pool is not None and tuple(v0.state.shape) == (3, 2, 10) and v1.kind == "state"
    assert v0.block_table is v2.block_table and v0.pool.data_ptr() != v2.pool.data_ptr() and v0.state.data_ptr() != v2.state.data_ptr()
    slot = cache.acquire()
    v0.state[slot] += 1.0
    cache.reserve([(slot, 70)])
    cache.release(slot)
    assert cache.acquire() == slot and float(v0.state[slot].abs().sum()) == 0.0       # a state starts at zero


def test_random_folders_hold_what_the_plain_implementation_reads(tmp_path):
    folder = make_folder(tmp_path, "nuf_c")
    cfg, tensors = P.read_model_folder(folder)
    logits, after = P.forward(cfg, tensors, random_tokens(0, 12, cfg["vocab"]), return_layers=True)
    assert logits.shape == (12, cfg["vocab"]) and len(after) == len(cfg["layers"]) and np.isfinite(logits).all()
    # causal: a later token changes nothing before it
    again = P.forward(cfg, tensors, random_tokens(0, 12, cfg["vocab"])[:7] + [3, 1, 4, 1, 5])
    assert np.abs(again[:7] - logits[:7]).max() < 1e-12 and np.abs(again[7:] - logits[7:]).max() > 1e-6


# the plain implementation's mechanisms against closed forms --------------------------------------------------
def test_plain_convolution_and_activation():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(9, 2)), rng.normal(size=(2, 4))
    y = P.causal_conv(x, w)
    for c in range(2):
        assert np.allclose(y[:, c], np.convolve(x[:, c], w[c, ::-1])[:9])
    assert np.allclose(P.causal_conv(x, w[:, 3:]), x * w[:, 3])           # one tap: the current token's
    for p, q in ((0.3, -1.0), (2.0, 2.0)):
        z = np.array([-1e-7, 0.0, 1e-7])
        assert np.allclose(P.xielu(z, p, q), 0.5 * z, atol=1e-12)          # continuous at zero with slope 1/2
        assert np.isclose(P.xielu(np.array([2.0]), p, q)[0], np.log1p(np.exp(p)) * 4 + 1)
        assert np.isclose(P.xielu(np.array([-50.0]), p, q)[0], (0.5 + np.log1p(np.exp(q))) * 49 - 25)


def test_plain_rotation_depends_on_the_distance_only():
    rng = np.random.default_rng(1)
    q, k = rng.normal(size=(1, 1, 12)), rng.normal(size=(1, 1, 12))
    dots = [float((P.rotate(q, [i], 8, 100.0) * P.rotate(k, [j], 8, 100.0)).sum()) for i, j in ((5, 2), (13, 10), (103, 100))]
    assert np.allclose(dots, dots[0])
    assert np.array_equal(P.rotate(q, [9], 8, 100.0)[..., 8:], q[..., 8:]) and np.array_equal(P.rotate(q, [0], 8, 100.0), q)
    one = P.rotate(np.array([[[1.0, 0.0, 0.0, 0.0]]]), [1], 4, 100.0)[0, 0]       # lane 0 pairs with lane 2, frequency 1
    assert np.allclose(one, [np.cos(1.0), 0.0, np.sin(1.0), 0.0])


def test_plain_attention_weights_are_not_normalised():
    q, k = np.zeros((3, 2, 4)), np.zeros((3, 1, 4))
    w = P.sigmoid_attention_weights(q, k, 1.0, 10.0, np.array([0.0, np.log(3.0)]))
    assert np.allclose(w[0], np.tril(np.full((3, 3), 0.5))) and np.allclose(w[1], np.tril(np.full((3, 3), 0.75)))
    q[2, 0, 0], k[1, 0, 0] = 100.0, 100.0                           # a capped score: sigmoid(10 tanh(1000)) = sigmoid(10)
    assert np.isclose(P.sigmoid_attention_weights(q, k, 1.0, 10.0, np.zeros(2))[0, 2, 1], 1 / (1 + np.exp(-10.0)))
    mixed = P.mix_heads(w, np.array([[0.0, 2.0], [1.0, -1.0]]))
    assert np.allclose(mixed[0], 2 * w[1]) and np.allclose(mixed[1], w[0] - w[1])


def test_plain_scans_against_sums_written_out():
    rng = np.random.default_rng(2)
    T, N, dv = 6, 3, 2
    x, B, C, dt = rng.normal(size=(T, 1, dv)), rng.normal(size=(T, 1, N)), rng.normal(size=(T, 1, N)), rng.uniform(0.1, 1, size=(T, 1))
    y = P.mamba2_scan(x, B, C, dt, np.array([0.2]), np.array([0.5]), 1, 1)
    a = -np.exp(0.2)
    for t in range(T):      # y_t = sum_s exp(a (dt_(s+1) + ... + dt_t)) dt_s (C_t . B_s) x_s + D x_t
        want = 0.5 * x[t, 0] + sum(np.exp(a * dt[s + 1: t + 1, 0].sum()) * dt[s, 0] * (C[t, 0] @ B[s, 0]) * x[s, 0] for s in range(t + 1))
        assert np.allclose(y[t, 0], want)
    # the delta rule with orthonormal keys, beta 1 and no decay is a table: a key's latest value comes back
    k = np.eye(4)[[0, 1, 2, 1, 0]][:, None, :]
    v = rng.normal(size=(5, 1, 3))
    o = P.delta_rule_scan(k, k, v, np.ones((5, 1)), np.ones((5, 1, 4)))
    assert np.allclose(o[:, 0], v[:, 0])
    # with a decay g on every row, what was stored t steps ago comes back times g^t
    q = np.tile(np.eye(4)[0], (5, 1))[:, None, :]
    o = P.delta_rule_scan(q, np.eye(4)[[0, 1, 2, 3, 1]][:, None, :], v, np.ones((5, 1)), np.full((5, 1, 4), 0.5))
    assert np.allclose(o[:, 0], [v[0, 0] * 0.5 ** t for t in range(5)])
    # a unit vector has length one (up to the epsilon), whatever its size
    assert np.allclose((P.unit(rng.normal(size=(3, 7)) * 100) ** 2).sum(-1), 1.0, atol=1e-6)

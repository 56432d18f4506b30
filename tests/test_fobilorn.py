"""What needs no GPU of the Fobilorn decoder: its configuration reader, its plan and tensor list, the registry, the
cache's kept first pages and paged lines of ids, and the plain implementation's own mechanisms."""
import copy
import os

import numpy as np
import pytest
import torch

from plain import fobilorn_plain as P
from fobilorn_tiny import CONFIGS, FOB_A, FOB_C, make_folder

from burn_lm_b200 import ConfigError, architecture, plan_of, preset
from burn_lm_b200.cache import Cache
from burn_lm_b200.config import FobilornConfig
from burn_lm_b200.model import tensor_specs_of
from burn_lm_b200.parts.base import CacheNeed
from burn_lm_b200.plan import ScheduleEntry


def test_the_architecture_is_registered_and_chosen_by_the_configuration():
    assert architecture("Fobilorn").config_class is FobilornConfig
    arch, typed, plan = plan_of(copy.deepcopy(FOB_A))
    assert arch.name == "Fobilorn" and plan.vocab_size == FOB_A["vocab"] and len(plan.layers) == len(FOB_A["layers"])
    assert typed.to_dict() == FobilornConfig.from_dict(typed.to_dict()).to_dict()
    for got, want in zip(typed.to_dict()["layers"], FOB_A["layers"]):
        assert got == want


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_size_comes_from_the_configuration(name):
    cfg = CONFIGS[name]
    specs = {s.name: tuple(s.shape) for s in tensor_specs_of(cfg)}
    width = cfg["width"]
    assert specs["embed"] == (cfg["vocab"], width) and specs["head"] == (cfg["vocab"], width)
    assert specs["bigram"] == (cfg["embedding"]["bigram"]["buckets"] + 1, width)
    for n in ("embed.norm", "final.norm"):
        assert specs[n] == (width,) and specs[n + ".b"] == (width,) and specs[n + ".alpha"] == ()
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        assert specs[f"l{i}.mix.q"] == (m["heads"] * m["dim"], width) and specs[f"l{i}.mix.k"] == (m["kv_heads"] * m["dim"], width)
        assert specs[f"l{i}.mix.v"] == (m["kv_heads"] * m["vdim"], width) and specs[f"l{i}.mix.o"] == (width, m["heads"] * m["vdim"])
        assert specs[f"l{i}.mix.g"] == (m["heads"], width) and specs[f"l{i}.mix.q.norm"] == (m["heads"] * m["dim"],)
        assert (f"l{i}.mix.vmix" in specs) == bool(m["v_mix"])
        mlp = layer["mlp"]
        if mlp is None:
            assert not any(k.startswith(f"l{i}.mlp.") for k in specs)
        elif mlp["kind"] == "dense":
            assert specs[f"l{i}.mlp.gate"] == (mlp["ff"], width) and specs[f"l{i}.mlp.down"] == (width, mlp["ff"])
        else:
            e = mlp["router"]["experts"]
            assert specs[f"l{i}.mlp.router"] == (e, width) and specs[f"l{i}.mlp.e{e - 1}.up"] == (mlp["expert"]["ff"], width)
            assert f"l{i}.mlp.e{e}.up" not in specs
            assert (f"l{i}.mlp.shared.gate" in specs) == (mlp["shared"] is not None)


def test_the_first_blending_layer_is_the_source():
    _, _, plan = plan_of(copy.deepcopy(FOB_A))
    kinds = [lp.part("mixer").spec.value_blend for lp in plan.layers]
    assert kinds == ["source", None, "blend", "blend"]


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "recurrent", "type"), (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mlp", "router", "top"), 9, "top"),
    (("norm", "eps"), -1.0, "eps"), (("embedding", "bigram", "buckets"), 0, "buckets"), (("layers", 0, "mixer", "mask", "size"), 0, "size"),
])
def test_configuration_errors_name_the_key(path, value, word):
    cfg = copy.deepcopy(FOB_A)
    at = cfg
    for p in path[:-1]:
        at = at[p]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        plan_of(cfg)
    assert word in str(e.value)


def test_random_folder_round_trip(tmp_path):
    folder = make_folder(tmp_path, "fob_c", seed=1)
    cfg, tensors = P.read_model_folder(folder)
    assert set(tensors) == {s.name for s in tensor_specs_of(FOB_C)}
    assert tensors["embed.norm.alpha"].shape == () and cfg["architecture"] == "Fobilorn"
    assert P.forward(cfg, tensors, [3, 1, 4, 1, 5]).shape == (5, FOB_C["vocab"])
    assert "fobilorn_tiny" in __import__("burn_lm_b200").preset_names() and preset("fobilorn_tiny")["architecture"] == "Fobilorn"


def test_kept_first_pages_stay_and_id_lines_are_paged():
    win = CacheNeed("kv", n_kv_heads=1, head_dim=8, window=70, value_dim=4, keep_first=65)
    ids = CacheNeed("ids", window=2)
    c = Cache([win], [ScheduleEntry(0)], 64 * 10, 2, 64 * 10, torch.float32, torch.device("cpu"), named={"embedding": ids})
    v, e = c.view(0), c.named_view("embedding")
    assert v.pool.shape == (10, 1 * 64 * (8 + 4)) and v.keep_first == 65 and v.window == 70
    assert e.kind == "ids" and e.pool.dtype == torch.int32 and e.pool.shape == (10, 64)
    a = c.acquire()
    length = 0
    gw = next(g for g in c._kv_groups if g.need == win)
    gi = next(g for g in c._kv_groups if g.need == ids)
    for grow in [100, 1, 200, 63, 1, 1, 150]:
        c.reserve([(a, length + grow)])
        length += grow
        c.set_length(a, length)
        pages = gw.pages_of[a]
        assert pages[0] is not None and pages[1] is not None              # positions 0..64 are kept for good
        first_needed = max(0, (length - grow) - 70 + 1) // 64
        for i, p in enumerate(pages):
            assert (p is None) == (2 <= i < first_needed), (length, i)
        table = gw.block_table[a].tolist()
        assert all(table[i] == p for i, p in enumerate(pages) if p is not None)
        assert sum(p is not None for p in gi.pages_of[a]) <= 4
    c.release(a)
    assert gw.pages.free_count == gi.pages.free_count == c.n_pages


def test_plain_mechanisms():
    # the sink: a row that sees one key of score 0 puts half its weight on it
    p = P.sink_softmax(np.zeros((1, 1)), np.ones((1, 1), dtype=bool))
    assert abs(p[0, 0] - 0.5) < 1e-12
    # the mask
    assert P.visible(10, 10, 1, 0) and not P.visible(10, 9, 1, 0) and P.visible(10, 1, 1, 2) and not P.visible(10, 2, 1, 2)
    assert not P.visible(3, 4, 100, 100)
    # pairs: the first token takes the last row; the hash reads the previous token
    rows = P.bigram_rows([5, 6, 5], 11, 3, 2)
    assert rows.tolist() == [11, (5 * 3 + 6 * 2) % 11, (6 * 3 + 5 * 2) % 11]
    # routing: the largest scores, the lower index first on a tie, weights not renormalised
    ids, w = P.route(np.array([[1.0, 0.0]]), np.array([[2.0, 0.0], [2.0, 0.0], [-1.0, 0.0], [3.0, 0.0]]), 3)
    assert ids.tolist() == [[3, 0, 1]] and abs(w.sum() - (P.sigmoid(3.0) + 2 * P.sigmoid(2.0))) < 1e-12


def test_a_blend_scalar_stored_in_a_layer_that_does_not_blend_is_left_unread(tmp_path):
    import torch
    from safetensors.torch import load_file, save_file
    from burn_lm_b200.weights.loader import load_tensors
    folder = make_folder(tmp_path, "fob_a", seed=3)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    assert "l1.mix.vmix" not in tensors                       # layer 1 of this configuration does not blend
    tensors["l1.mix.vmix"] = torch.tensor(0.25, dtype=torch.bfloat16)
    save_file(tensors, path)
    _, _, plan = plan_of(copy.deepcopy(FOB_A))
    got = load_tensors(folder, tensor_specs_of(FOB_A), torch.float32, "cpu", plan.ignorable_tensors)
    assert "l1.mix.vmix" not in got and "l0.mix.vmix" in got
    # and the source layer's scalar, which nothing reads, may be absent
    del tensors["l0.mix.vmix"], tensors["l1.mix.vmix"]
    save_file(tensors, path)
    got = load_tensors(folder, tensor_specs_of(FOB_A), torch.float32, "cpu", plan.ignorable_tensors)
    assert "l0.mix.vmix" not in got and "l2.mix.vmix" in got

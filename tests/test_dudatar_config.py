"""Dudatar off the device: the configuration reader, the run order it makes, the checkpoint's
tensor names, the rank taken from a tensor's shape, and the plain implementation against
closed forms of its own mechanisms."""
import copy
import json
import os

import pytest
import torch

import plain_dudatar as plain
from dudatar_configs import DUDATAR_TINY, dudatar_config, dudatar_config_dict, make_dudatar_dir


def test_registry_reads_the_architecture_key_and_round_trips():
    from tinyserve_b200.config import DudatarConfig, architecture_of, config_from_dict
    raw = dudatar_config_dict("X")
    assert architecture_of(raw) == "Dudatar"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, DudatarConfig) and cfg.vocab == 200 and cfg.width == 64
    assert config_from_dict(cfg.to_dict()) == cfg
    assert "logit_softcap" not in dudatar_config("Y").to_dict() and "loop" not in dudatar_config("Y").to_dict()


@pytest.mark.parametrize("damage,text", [
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot"),
    (lambda r: r["layers"][1]["mixer"].pop("rank"), "rank"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["layers"][2]["mlp"].update(kind="experts"), "kind"),
    (lambda r: r["norm"].update(eps=0), "eps"),
])
def test_a_damaged_configuration_is_refused(damage, text):
    from tinyserve_b200.config import ConfigError, config_from_dict
    raw = dudatar_config_dict("X")
    damage(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_run_order_passes_caches_and_states():
    from tinyserve_b200.parts import build_model
    model = build_model(dudatar_config("X"))
    runs = [(c.layer, [arg for _, arg in c.before]) for c in model.calls]
    assert runs == [(0, [0]), (1, []), (0, [1]), (1, []), (0, [2]), (1, []), (2, [])]
    assert runs == [(i, [] if t is None else [t]) for i, t in plain.run_order(dudatar_config_dict("X"))]
    # every run has a state of its own; only the runs with softmax attention have cache entries
    assert [c.state for c in model.calls] == list(range(7))
    assert [c.cache for c in model.calls] == [0, -1, 1, -1, 2, -1, 3]
    assert len(model.cache_groups) == 2 and model.group_sizes == [3, 1]       # two head geometries
    z = build_model(dudatar_config("Z"))
    assert [c.layer for c in z.calls] == [0, 1, 2, 1, 2, 3] and [len(c.before) for c in z.calls] == [0, 1, 0, 1, 0, 0]
    y = build_model(dudatar_config("Y"))
    assert not y.stream_ops and [c.layer for c in y.calls] == [0, 1, 2] and all(not c.before for c in y.calls)
    assert model.capturable and y.capturable


def test_a_loop_over_no_layer_or_of_one_pass():
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.parts import build_model
    raw = dudatar_config_dict("Z")
    raw["loop"] = {"start": 2, "stop": 2, "times": 5}
    model = build_model(config_from_dict(raw))
    assert [c.layer for c in model.calls] == [0, 1, 2, 3] and not model.stream_ops
    raw["loop"] = {"start": 0, "stop": 4, "times": 1}
    model = build_model(config_from_dict(raw))
    assert [(c.layer, len(c.before)) for c in model.calls] == [(0, 1), (1, 0), (2, 0), (3, 0)]
    assert plain.run_order(raw) == [(0, 0), (1, None), (2, None), (3, None)]


def test_checkpoint_names_and_the_rank_from_a_shape(tmp_path):
    from safetensors import safe_open
    from tinyserve_b200.config import ConfigError, load_model_config
    folder = make_dudatar_dir(tmp_path, "X", seed=3)
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as fh:
        names = set(fh.keys())
        assert fh.get_slice("l1.mix.a1").get_shape() == [8, 64]
        assert fh.get_slice("l0.mix.left.g").get_shape() == [4, 64]
        assert fh.get_slice("loop.step").get_shape() == [3, 64] and fh.get_slice("loop.in").get_shape() == [64, 128]
    assert {"embed", "head", "final.norm", "loop.in", "loop.step", "l0.norm1", "l0.mix.left.q", "l0.mix.left.out",
            "l0.mix.right.g", "l0.mix.right.out", "l0.mlp.gate", "l1.mix.a2", "l1.mix.a2.b", "l1.mix.norm",
            "l2.mlp.down"} <= names
    assert not any(n.startswith("l1.mlp") for n in names), "a layer without a feed-forward has no such tensors"
    assert not any(n.endswith(".weight") or n.endswith(".bias") for n in names)
    # a configuration that does not give the rank takes it from the first factor's rows
    with open(os.path.join(folder, "config.json")) as fh:
        raw = json.load(fh)
    del raw["layers"][1]["mixer"]["rank"]
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(raw, fh)
    assert load_model_config(folder).layers[1]["mixer"]["rank"] == 8
    os.remove(os.path.join(folder, "model.safetensors"))
    with pytest.raises(ConfigError, match="rank"):
        load_model_config(folder)


def test_loader_lists_what_does_not_fit(tmp_path):
    from safetensors.torch import load_file, save_file
    from tinyserve_b200.parts import build_model
    from tinyserve_b200.weights import WeightError, check_checkpoint
    from tinyserve_b200.weights.loader import _index_folder
    folder = make_dudatar_dir(tmp_path, "Y", seed=4)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    tensors["l1.mix.left.k"] = tensors["l1.mix.left.k"][:-1].contiguous()
    tensors["extra"] = tensors.pop("l2.mix.a2.b")
    save_file(tensors, path)
    index, dup = _index_folder(folder)
    with pytest.raises(WeightError) as err:
        check_checkpoint(build_model(dudatar_config("Y")), index, dup)
    assert err.value.missing == ["l2.mix.a2.b"] and err.value.unexpected == ["extra"]
    assert [w[0] for w in err.value.wrong_shape] == ["l1.mix.left.k"]


# ----------------------------------------------------------------------------- the plain implementation itself
def test_plain_scan_equals_its_closed_form():
    """o_t = sum_{s <= t} (q_t . (prod_{s < r <= t} a_r) k_s) v_s, written out."""
    g = torch.Generator().manual_seed(0)
    T, n, nv = 9, 4, 3
    q, k, v = (torch.randn(T, d, generator=g, dtype=torch.float64) for d in (n, n, nv))
    a = torch.rand(T, n, generator=g, dtype=torch.float64)
    want = torch.zeros(T, nv, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            want[t] += (q[t] * a[s + 1:t + 1].prod(0) * k[s]).sum() * v[s]
    assert torch.allclose(plain.matrix_state_scan(q, k, v, a), want, atol=1e-12)


def test_plain_rotation_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(1)
    x, y = (torch.randn(1, 1, 12, generator=g, dtype=torch.float64) for _ in range(2))
    dot = lambda p, s: (plain.rotate(x, torch.tensor([p]), 8, 50.0) * plain.rotate(y, torch.tensor([s]), 8, 50.0)).sum()
    assert abs(dot(7, 3) - dot(104, 100)) < 1e-9 and abs(dot(7, 3) - dot(8, 3)) > 1e-6
    assert torch.equal(plain.rotate(x, torch.tensor([5]), 8, 50.0)[..., 8:], x[..., 8:])
    assert torch.equal(plain.rotate(x, torch.tensor([0]), 8, 50.0), x)


def test_plain_prefix_property(tmp_path):
    """Causal: the logits of a prefix do not change when tokens follow."""
    folder = make_dudatar_dir(tmp_path, "X", seed=5)
    cfg, weights = plain.load_folder(folder)
    ids = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    full = plain.logits(cfg, weights, ids)
    assert torch.allclose(full[:6], plain.logits(cfg, weights, ids[:6]), atol=1e-12)
    assert full.abs().max() <= cfg["logit_softcap"]

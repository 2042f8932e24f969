"""Delilorn off the device: the configuration reader, the run order and cache entries it makes, the
checkpoint's tensor names, the stretched rotary frequencies, pages of kept first tokens in the cache
manager, and the plain implementation against closed forms of its own mechanisms."""
import math

import pytest
import torch

import plain_delilorn as plain
from delilorn_configs import (DELILORN_TINY, delilorn_config, delilorn_config_dict, make_delilorn_dir,
                              random_delilorn_config_dict)


def test_registry_reads_the_architecture_key_and_round_trips():
    from tinyserve_b200.config import DelilornConfig, architecture_of, config_from_dict
    raw = delilorn_config_dict("P")
    assert architecture_of(raw) == "Delilorn"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, DelilornConfig) and cfg.vocab == 180 and cfg.width == 64
    assert config_from_dict(cfg.to_dict()) == cfg
    for seed in range(20):
        drawn = config_from_dict(random_delilorn_config_dict(seed))
        assert config_from_dict(drawn.to_dict()) == drawn


@pytest.mark.parametrize("damage,text", [
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][2]["mixer"].update(decay=[0.5]), "decay"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].update(high=0.5), "scaling"),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=4), "rot"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_rank=32), "kv_from"),
    (lambda r: r["layers"][1]["mlp"].update(kind="dense"), "kind"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda r: r["norm"].update(eps=0), "eps"),
])
def test_a_damaged_configuration_is_refused(damage, text):
    from tinyserve_b200.config import ConfigError, config_from_dict
    raw = delilorn_config_dict("P")
    damage(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_a_reader_of_another_cache_may_leave_the_row_sizes_out():
    from tinyserve_b200.config import config_from_dict
    raw = delilorn_config_dict("P")
    for key in ("kv_rank", "rot_dim", "rot"):
        del raw["layers"][3]["mixer"][key]
    assert config_from_dict(raw) == delilorn_config("P")


def test_run_order_caches_and_states():
    from tinyserve_b200.parts import build_model
    p = build_model(delilorn_config("P"))
    # the window layer and the latent layer have a cache entry each; the second latent layer reads the first's
    assert [(c.cache, c.writes_cache, c.state) for c in p.calls] == [(0, True, -1), (1, True, -1), (-1, True, 0), (1, False, -1)]
    assert [g.kind for g in p.cache_groups] == ["window", "full"] and p.cache_groups[0].keep_first == 3
    assert [t.name for t in p.cache_groups[1].tensors] == ["latent"] and p.cache_groups[1].tensors[0].heads == 1
    assert p.cache_groups[1].tensors[0].width == 32          # 24 + 8 in rows of a multiple of 16
    r = build_model(delilorn_config("R"))
    assert [c.cache for c in r.calls] == [0, 0, 1, 2, -1, 0] and [c.writes_cache for c in r.calls] == [True, False, True, True, True, False]
    assert r.group_sizes == [1, 1, 1] and r.cache_groups[2].tensors[0].width == 112      # 72 + 32 -> 112
    q = build_model(delilorn_config("Q"))
    assert [c.state for c in q.calls] == [0, -1, -1, -1, 1]
    assert [(g.kind, g.window, g.keep_first) for g in q.cache_groups] == [("window", 17, 0), ("window", 9, 21), ("full", 0, 0)]
    assert p.capturable and q.capturable and r.capturable
    assert q.blocks[2].ffn is None and q.lm_head is None


def test_checkpoint_names(tmp_path):
    from safetensors import safe_open
    folder = make_delilorn_dir(tmp_path, "P", seed=3)
    with safe_open(f"{folder}/model.safetensors", "pt") as fh:
        names = set(fh.keys())
        shapes = {k: tuple(fh.get_slice(k).get_shape()) for k in names}
    assert {"embed", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.o",
            "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv",
            "l1.mix.sink", "l1.mix.g", "l1.mix.o", "l1.mlp.router", "l1.mlp.e5.up", "l1.mlp.e5.down",
            "l2.mix.norm", "l2.mix.g", "l3.mix.uk", "l3.mix.sink"} <= names
    assert not {"l2.norm2", "l2.norm2b", "l3.mix.dkv", "l3.mix.dkv.norm", "head", "l1.mlp.e6.up"} & names
    assert shapes["l1.mix.dkv"] == (32, 64) and shapes["l1.mix.uq"] == (3 * 24, 40) and shapes["l1.mix.sink"] == (3,)
    assert shapes["l2.mix.norm"] == (64,) and shapes["l1.mlp.e0.down"] == (64, 24) and shapes["l1.mlp.router"] == (6, 64)
    cfg, weights = plain.load_folder(folder)
    assert weights["l0.norm1"].abs().max() <= 0.11, "block norms are stored around zero"
    assert (weights["l2.mix.norm"] - 1).abs().max() <= 0.11, "the norms inside mixers are stored as they are"


def test_loader_lists_what_does_not_fit(tmp_path):
    from safetensors.torch import load_file, save_file
    from tinyserve_b200.parts import build_model
    from tinyserve_b200.weights.loader import WeightError, _index_folder, check_checkpoint
    folder = make_delilorn_dir(tmp_path, "P", seed=4)
    weights = load_file(f"{folder}/model.safetensors")
    weights["l3.mix.dkv"] = weights.pop("l1.mix.dkv")
    weights["l1.mlp.e2.up"] = weights["l1.mlp.e2.up"][:8].contiguous()
    save_file(weights, f"{folder}/model.safetensors")
    index, dup = _index_folder(folder)
    with pytest.raises(WeightError) as err:
        check_checkpoint(build_model(delilorn_config("P")), index, dup)
    assert err.value.missing == ["l1.mix.dkv"] and err.value.unexpected == ["l3.mix.dkv"]
    assert [w[0] for w in err.value.wrong_shape] == ["l1.mlp.e2.up"]
    # the norms around a feed-forward that layer 2 does not have may be there; nobody reads them
    weights = load_file(f"{make_delilorn_dir(tmp_path / 'b', 'P', seed=4)}/model.safetensors")
    weights["l2.norm2"], weights["l2.norm2b"] = weights["l0.norm2"].clone(), weights["l0.norm2"].clone()
    weights["l1.norm3"] = weights["l0.norm2"].clone()
    save_file(weights, f"{tmp_path / 'b'}/model.safetensors")
    index, dup = _index_folder(str(tmp_path / "b"))
    with pytest.raises(WeightError) as err:
        check_checkpoint(build_model(delilorn_config("P")), index, dup)
    assert err.value.unexpected == ["l1.norm3"] and not err.value.missing


@pytest.mark.parametrize("rot", [
    {"base": 1e6, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 1024}},
    {"base": 1e4, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
    {"base": 100.0, "dims": 64, "scaling": {"factor": 2.0, "low": 2.0, "high": 3.0, "original": 40}},
    {"base": 5e5, "dims": 48},
])
def test_stretched_frequencies(rot):
    from tinyserve_b200.parts.rotary import Rotary
    part = Rotary(rot["dims"], rot["base"], "half", rot.get("scaling"))
    cos, sin = Rotary.tables(part.rotary_dim, part.theta, 300, part.scaling)
    f = plain.frequencies(rot)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert (cos.double() - ang.cos()).abs().max() < 1e-6 and (sin.double() - ang.sin()).abs().max() < 1e-6
    if "scaling" in rot:
        sc = rot["scaling"]
        plain_f = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
        waves = 2 * math.pi / plain_f
        kinds = {"kept": (waves < sc["original"] / sc["high"]), "stretched": (waves > sc["original"] / sc["low"])}
        assert torch.equal(f[kinds["kept"]], plain_f[kinds["kept"]])
        assert torch.allclose(f[kinds["stretched"]], plain_f[kinds["stretched"]] / sc["factor"])
        between = ~kinds["kept"] & ~kinds["stretched"]
        assert ((f[between] <= plain_f[between]) & (f[between] >= plain_f[between] / sc["factor"])).all()
        assert kinds["kept"].any() and kinds["stretched"].any(), "the case has both ends"


def test_pages_of_kept_first_tokens_stay(tmp_path):
    from tinyserve_b200.cache.manager import CacheManager, GroupSpec
    mgr = CacheManager([GroupSpec("window", 10, 5), GroupSpec("window", 10, 0), GroupSpec("full")], 40, 4, 2)
    mgr.begin("a")
    for n in (7, 1, 1, 30, 1, 2, 9):
        assert mgr.allocate("a", n)
        mgr.commit("a", n)
        mgr.check_invariants()
    held = [[i for i, p in enumerate(mgr.block_table("a", g)) if p] for g in range(3)]
    total = mgr.num_computed("a")
    first_needed = (total - 10 + 1) // 4
    assert held[1] == list(range(first_needed, -(-total // 4)))
    assert held[0] == [0, 1] + held[1], "the two pages that hold the five kept tokens are never given back"
    assert held[2] == list(range(-(-total // 4)))
    # the released entries reach the device's copy of the row as null pages
    changes, receipt = mgr.table_updates("a", 0)
    mgr.table_synced(receipt)
    assert mgr.allocate("a", 8)
    mgr.commit("a", 8)
    changes, _ = mgr.table_updates("a", 0)
    assert all(i >= 2 for i, _ in changes) and any(page == 0 for _, page in changes)
    mgr.free("a")
    mgr.check_invariants()
    assert all(p.num_free == p.num_usable for p in mgr.pools)


def test_plain_scan_equals_its_closed_form():
    """o_t = sum_(s <= t) decay^(t - s) (q_t . k_s) v_s for the lightning mixer's recurrence."""
    torch.manual_seed(0)
    T, n, nv, width = 9, 4, 6, 8
    W = {"q": torch.randn(n, width).double(), "k": torch.randn(n, width).double(), "v": torch.randn(nv, width).double(),
         "g": torch.randn(nv, width).double(), "o": torch.eye(nv).double(), "norm": torch.ones(nv).double()}
    h = torch.randn(T, width).double()
    m = {"heads": 1, "dim": n, "vdim": nv, "decay": [0.8]}
    got = plain.lightning(h, W, "", m, 1e-6)
    q, k, v = plain.silu(h @ W["q"].T), plain.silu(h @ W["k"].T), plain.silu(h @ W["v"].T)
    o = torch.stack([sum(0.8 ** (t - s) * (q[t] @ k[s]) * v[s] for s in range(t + 1)) for t in range(T)])
    want = plain.unit_rms(o, 1e-6) * torch.sigmoid(h @ W["g"].T)
    assert (got - want).abs().max() < 1e-12


def test_plain_sink_takes_weight_and_mask_has_edges():
    assert [j for j in range(12) if plain.visible(11, j, {"size": 4, "keep_first": 2})] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(12) if plain.visible(3, j, {"size": 4, "keep_first": 2})] == [0, 1, 2, 3]
    assert [j for j in range(6) if plain.visible(4, j, None)] == [0, 1, 2, 3, 4]
    # one token, one head: the softmax weight of the only key is 1 / (1 + exp(sink - score))
    torch.manual_seed(1)
    m = {"heads": 1, "dim": 4, "rot_dim": 2, "vdim": 3, "q_rank": 5, "kv_rank": 6, "scale": 0.7, "rot": {"base": 10.0, "dims": 2}}
    W = {"dq": torch.randn(5, 8), "dq.norm": torch.ones(5), "uq": torch.randn(6, 5), "dkv": torch.randn(8, 8),
         "dkv.norm": torch.ones(6), "uk": torch.randn(4, 6), "uv": torch.randn(3, 6), "sink": torch.tensor([0.3]),
         "g": torch.zeros(3, 8), "o": torch.eye(3)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(1, 8).double()
    kv = plain.latent_kv(h, W, "", m, 1e-6)
    got = plain.latent_attention(h, W, "", m, 1e-6, kv)[0]
    cq = plain.unit_rms(h @ W["dq"].T, 1e-6)
    q = (cq @ W["uq"].T)[0]
    score = (q[:4] @ (W["uk"] @ kv[0][0]) + q[4:] @ kv[1][0]) * 0.7      # position 0: nothing turns
    want = 0.5 * (W["uv"] @ kv[0][0]) / (1 + torch.exp(W["sink"][0] - score))
    assert (got - want).abs().max() < 1e-12


def test_plain_prefix_property(tmp_path):
    folder = make_delilorn_dir(tmp_path, "Q", seed=5)
    cfg, weights = plain.load_folder(folder)
    ids = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(2)).tolist()
    whole = plain.logits(cfg, weights, ids)
    assert (plain.logits(cfg, weights, ids[:23]) - whole[:23]).abs().max() < 1e-9

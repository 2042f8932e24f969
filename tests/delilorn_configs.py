"""Tiny Delilorn configurations for the tests; they differ from one another in every size, in the
order of the layers and in which options are there at all."""
from __future__ import annotations


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


DELILORN_TINY = {
    # attention first (a window of 24 beside 3 kept tokens, stretched frequencies), a lightning layer
    # without a feed-forward, a latent layer and one that reads its cache two layers later
    "P": {
        "vocab": 180, "width": 64, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "attention", "mlp": _moe(40, 4, 2), "mixer": {
                "heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3,
                "rot": {"base": 1e4, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
                "mask": {"size": 24, "keep_first": 3}}},
            {"type": "latent_attention", "mlp": _moe(24, 6, 1), "mixer": _latent(3, 16, 8, 24, 40, 24, 0.25, 1e4)},
            {"type": "lightning", "mlp": None, "mixer": {"heads": 2, "dim": 16, "vdim": 32, "decay": [0.9, 0.99]}},
            {"type": "latent_attention", "mlp": _moe(32, 3, 3), "mixer": _latent(2, 8, 8, 16, 16, 24, 0.5, 1e4, kv_from=1)},
        ]},
    # lightning first and last, sizes that are no power of two, a window without kept tokens and one
    # that keeps more tokens than a page holds, attention without a mask and without rotation, one expert of one
    "Q": {
        "vocab": 301, "width": 96, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "lightning", "mlp": _moe(56, 5, 2), "mixer": {"heads": 3, "dim": 20, "vdim": 24, "decay": [0.5, 0.95, 0.999]}},
            {"type": "attention", "mlp": _moe(48, 1, 1), "mixer": {
                "heads": 3, "kv_heads": 3, "dim": 48, "vdim": 16, "scale": 0.2, "rot": {"base": 5e5, "dims": 48},
                "mask": {"size": 17, "keep_first": 0}}},
            {"type": "attention", "mlp": None, "mixer": {
                "heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.4,
                "rot": {"base": 100.0, "dims": 16}, "mask": {"size": 9, "keep_first": 21}}},
            {"type": "attention", "mlp": _moe(72, 7, 4), "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 48, "scale": 0.3}},
            {"type": "lightning", "mlp": _moe(56, 2, 2), "mixer": {"heads": 1, "dim": 32, "vdim": 64, "decay": [0.97]}},
        ]},
    # head sizes the tensor-core kernels take, latent layers in a chain of three readers, a latent
    # whose cache row fills its stored width exactly and one that does not
    "R": {
        "vocab": 384, "width": 128, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "latent_attention", "mlp": _moe(64, 8, 2), "mixer": _latent(4, 32, 16, 32, 64, 48, 0.15, 1e6)},
            {"type": "latent_attention", "mlp": None, "mixer": _latent(8, 16, 16, 16, 32, 48, 0.3, 1e6, kv_from=0)},
            {"type": "attention", "mlp": _moe(96, 4, 4), "mixer": {
                "heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125,
                "rot": {"base": 1e4, "dims": 32, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 32}},
                "mask": {"size": 64, "keep_first": 16}}},
            {"type": "latent_attention", "mlp": _moe(64, 8, 2), "mixer": _latent(2, 64, 32, 64, 96, 72, 0.1, 1e4)},
            {"type": "lightning", "mlp": _moe(32, 16, 5), "mixer": {"heads": 4, "dim": 64, "vdim": 32,
                                                                   "decay": [0.9, 0.99, 0.999, 0.9999]}},
            {"type": "latent_attention", "mlp": _moe(64, 2, 1), "mixer": _latent(4, 32, 16, 32, 64, 48, 0.15, 1e6, kv_from=0)},
        ]},
}


def delilorn_config_dict(name: str) -> dict:
    import copy
    return dict(copy.deepcopy(DELILORN_TINY[name]), architecture="Delilorn")


def delilorn_config(name: str):
    from tinyserve_b200.config import config_from_dict
    return config_from_dict(delilorn_config_dict(name))


def decisive_routers(folder: str, factor: float = 10.0) -> str:
    """The routers of a random model multiplied by ``factor``: with weights of 0.02 all experts score
    alike, and which of them a token takes would hang on the last bit of a sum."""
    import os
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)
    for name in weights:
        if name.endswith(".router"):
            weights[name] = (weights[name].float() * factor).to(weights[name].dtype)
    save_file(weights, path)
    return folder


def make_delilorn_dir(folder, name: str, seed: int = 0) -> str:
    from tinyserve_b200.weights import write_random_model
    return decisive_routers(write_random_model(delilorn_config(name), str(folder), seed=seed))


def random_delilorn_config_dict(seed: int) -> dict:
    """A configuration drawn from a seed: sizes that are no power of two and no multiple of 16 among
    them, any order of layer kinds, latent layers that read an earlier one's cache, windows with and
    without kept tokens, layers without feed-forward."""
    import random
    r = random.Random(seed)
    even = lambda lo, hi: 2 * r.randint(lo // 2, hi // 2)
    width = 8 * r.randint(4, 14)
    layers = []

    def rot(dims):
        out = {"base": r.choice([100.0, 1e4, 7e5]), "dims": dims}
        if r.random() < 0.5:
            out["scaling"] = {"factor": r.choice([2.0, 4.0, 8.0]), "low": 1.0, "high": r.choice([2.0, 4.0]),
                              "original": r.choice([16, 64, 256])}
        return out

    for i in range(r.randint(1, 5)):
        experts = r.randint(1, 9)
        mlp = None if r.random() < 0.25 else _moe(8 * r.randint(2, 10), experts, r.randint(1, experts))
        kind = r.choice(["lightning", "latent_attention", "attention"])
        if kind == "lightning":
            heads = r.randint(1, 4)
            mixer = {"heads": heads, "dim": r.choice([4, 8, 12, 20, 24, 36, 40, 64]), "vdim": r.choice([6, 10, 16, 24, 30, 48, 72]),
                     "decay": [round(1.0 - 2.0 ** -r.uniform(1, 9), 6) for _ in range(heads)]}
        elif kind == "latent_attention":
            earlier = [j for j, l in enumerate(layers) if l["type"] == "latent_attention" and "kv_from" not in l["mixer"]]
            if earlier and r.random() < 0.5:
                src = r.choice(earlier)
                m = layers[src]["mixer"]
                mixer = _latent(r.randint(1, 5), even(4, 40), m["rot_dim"], r.choice([6, 10, 16, 24]), 8 * r.randint(1, 6),
                                m["kv_rank"], r.choice([0.1, 0.3]), m["rot"]["base"], kv_from=src)
                mixer["rot"] = dict(m["rot"])
            else:
                mixer = _latent(r.randint(1, 5), even(4, 40), even(2, 24), r.choice([6, 10, 16, 24]), 8 * r.randint(1, 6),
                                r.choice([8, 12, 20, 40, 56]), r.choice([0.1, 0.3]), r.choice([100.0, 1e4, 7e5]))
        else:
            kv = r.randint(1, 3)
            dim = even(8, 72)
            mixer = {"heads": kv * r.randint(1, 3), "kv_heads": kv, "dim": dim, "vdim": r.choice([8, 16, 24, 40, 64, 80]),
                     "scale": r.choice([0.1, dim ** -0.5, 0.4]), "rot": rot(r.choice([dim, even(2, dim)]))}
            if r.random() < 0.8:
                mixer["mask"] = {"size": r.randint(1, 40), "keep_first": r.choice([0, 0, 1, 2, 5, 18])}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Delilorn", "vocab": r.randint(50, 400), "width": width,
            "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])}, "layers": layers}

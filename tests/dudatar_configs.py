"""Tiny Dudatar configurations for the tests; they differ from one another in every size, in the
order of the layers and in which options are there at all."""
from __future__ import annotations


def _rot(dims, base):
    return {"dims": dims, "base": base}


DUDATAR_TINY = {
    # a looped group from the first layer on (three passes), value sizes unlike key sizes, two
    # key/value heads, a layer without a feed-forward, rotary on all of the left key and on part
    # of the right one
    "X": {
        "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 0.4,
        "loop": {"start": 0, "stop": 2, "times": 3},
        "layers": [
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 96}, "mixer": {
                "left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.5, "rot": _rot(16, 1e4)},
                "right": {"heads": 2, "dim": 32, "vdim": 16, "decay": [0.9, 0.99], "rot": _rot(8, 100.0)}}},
            {"type": "gla", "mlp": None, "mixer": {"heads": 2, "dim": 16, "vdim": 32, "tau": 4.0, "rank": 8}},
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 128}, "mixer": {
                "left": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "rot": _rot(0, 1e4)},
                "right": {"heads": 1, "dim": 16, "vdim": 64, "decay": [0.97], "rot": _rot(16, 5e3)}}},
        ]},
    # no loop and no soft cap; gated layers first and last; tau 1; sizes that are no power of two
    "Y": {
        "vocab": 301, "width": 96, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "gla", "mlp": {"kind": "dense", "ff": 160}, "mixer": {"heads": 3, "dim": 20, "vdim": 24, "tau": 1.0, "rank": 12}},
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 72}, "mixer": {
                "left": {"heads": 2, "kv_heads": 1, "dim": 48, "vdim": 48, "scale": 0.3, "rot": _rot(24, 2e5)},
                "right": {"heads": 3, "dim": 16, "vdim": 32, "decay": [0.5, 0.95, 0.999], "rot": _rot(16, 3e6)}}},
            {"type": "gla", "mlp": {"kind": "dense", "ff": 160}, "mixer": {"heads": 1, "dim": 32, "vdim": 64, "tau": 8.0, "rank": 4}},
        ]},
    # head sizes of 64 (the tensor-core attention kernels), a loop of one pass in the middle, a
    # loop that ends with the last layer is "W" below
    "Z": {
        "vocab": 384, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 0.8,
        "loop": {"start": 1, "stop": 3, "times": 2},
        "layers": [
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 192}, "mixer": {
                "left": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.25, "rot": _rot(32, 1e4)},
                "right": {"heads": 2, "dim": 64, "vdim": 128, "decay": [0.96875, 0.998], "rot": _rot(64, 1e4)}}},
            {"type": "gla", "mlp": {"kind": "dense", "ff": 192}, "mixer": {"heads": 2, "dim": 64, "vdim": 64, "tau": 12.0, "rank": 24}},
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 256}, "mixer": {
                "left": {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 32, "scale": 0.125, "rot": _rot(64, 1e6)},
                "right": {"heads": 4, "dim": 32, "vdim": 32, "decay": [0.9, 0.99, 0.999, 0.9999], "rot": _rot(16, 1e4)}}},
            {"type": "gla", "mlp": None, "mixer": {"heads": 4, "dim": 32, "vdim": 32, "tau": 2.0, "rank": 8}},
        ]},
}


def dudatar_config_dict(name: str) -> dict:
    import copy
    return dict(copy.deepcopy(DUDATAR_TINY[name]), architecture="Dudatar")


def dudatar_config(name: str):
    from tinyserve_b200.config import config_from_dict
    return config_from_dict(dudatar_config_dict(name))


def make_dudatar_dir(folder, name: str, seed: int = 0) -> str:
    from tinyserve_b200.weights import write_random_model
    return write_random_model(dudatar_config(name), str(folder), seed=seed)


def random_dudatar_config_dict(seed: int) -> dict:
    """A configuration drawn from a seed: sizes that are no power of two and no multiple of 16
    among them, any order of layer kinds, a loop anywhere or none, layers without feed-forward."""
    import random
    r = random.Random(seed)
    even = lambda lo, hi: 2 * r.randint(lo // 2, hi // 2)
    width = 8 * r.randint(4, 14)

    def rot(dim):
        return _rot(r.choice([0, dim, even(2, dim)]), r.choice([100.0, 1e4, 7e5]))

    def layer():
        mlp = None if r.random() < 0.25 else {"kind": "dense", "ff": 8 * r.randint(3, 20)}
        if r.random() < 0.5:
            dim = r.choice([4, 8, 12, 20, 24, 36, 40, 64])
            return {"type": "gla", "mlp": mlp, "mixer": {"heads": r.randint(1, 5), "dim": dim, "vdim": r.choice([6, 10, 16, 24, 30, 48, 72]),
                                                        "tau": r.choice([1.0, 2.5, 16.0]), "rank": r.choice([3, 8, 12, 16])}}
        kv = r.randint(1, 3)
        ldim = even(8, 72)
        rdim = r.choice([4, 8, 12, 20, 24, 36, 40, 64])
        heads = r.randint(1, 4)
        return {"type": "parallel", "mlp": mlp, "mixer": {
            "left": {"heads": kv * r.randint(1, 3), "kv_heads": kv, "dim": ldim, "vdim": r.choice([8, 16, 24, 40, 64, 80]),
                     "scale": r.choice([0.1, ldim ** -0.5, 0.4]), "rot": rot(ldim)},
            "right": {"heads": heads, "dim": rdim, "vdim": r.choice([6, 10, 16, 24, 30, 48, 72]),
                      "decay": [round(1.0 - 2.0 ** -r.uniform(1, 9), 6) for _ in range(heads)], "rot": rot(rdim)}}}

    layers = [layer() for _ in range(r.randint(1, 4))]
    raw = {"architecture": "Dudatar", "vocab": r.randint(50, 400), "width": width, "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])},
           "layers": layers}
    if r.random() < 0.7:
        start = r.randint(0, len(layers) - 1)
        raw["loop"] = {"start": start, "stop": r.randint(start + 1, len(layers)), "times": r.randint(1, 3)}
    if r.random() < 0.7:
        raw["logit_softcap"] = r.choice([0.3, 1.0, 25.0])
    return raw

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

"""Dudatar: a decoder whose blocks run their mixer and their feed-forward side by side on one
layer norm, with two kinds of mixer (gated linear attention; softmax attention and retention
side by side), a group of layers that runs several times with the same weights (the embedding
is mixed into the stream again before every pass), and soft-capped logits.

config.json: ``architecture`` "Dudatar"; ``vocab``, ``width``; ``norm.eps``; ``logit_softcap``;
``layers``: a list of {"type": "gla" | "parallel", "mixer": {...}, "mlp": {"kind": "dense",
"ff": n} | null}; ``loop``: {"start", "stop", "times"} or absent.  A "gla" mixer gives heads,
dim, vdim, tau; a "parallel" mixer gives ``left`` (heads, kv_heads, dim, vdim, scale, rot) and
``right`` (heads, dim, vdim, decay, rot); ``rot`` is {"base", "dims"}.  The rank of the decay
projection of a "gla" mixer is the row count of its first factor in the checkpoint (or
``mixer.rank`` where there is no checkpoint to look at).

Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.in``, ``loop.step``, and per layer
``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``: the tensor itself carries the name
(no ".weight"), a bias is ".b"."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import ClassVar

from .model_config import ConfigError, LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec

LAYER_TYPES = ("gla", "parallel")


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


def _positive_int(d, key, where):
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d, key, where):
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class DudatarConfig(ModelConfig):
    architecture: ClassVar[str] = "Dudatar"
    #: ``from_dict`` wants the shapes of the checkpoint's tensors where there is a checkpoint
    reads_tensor_shapes: ClassVar[bool] = True

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    logit_softcap: float = 0.0
    layers: tuple = ()               # the config's layer entries, ranks filled in
    loop: dict = field(default_factory=dict)     # {} or {"start", "stop", "times"}

    @classmethod
    def from_dict(cls, raw: dict, tensor_shapes: dict | None = None) -> "DudatarConfig":
        layers = copy.deepcopy(_need(raw, "layers", "the model"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {LAYER_TYPES}")
            mixer = _need(layer, "mixer", where)
            if kind == "gla":
                for key in ("heads", "dim", "vdim"):
                    _positive_int(mixer, key, where + ".mixer")
                if not _number(mixer, "tau", where + ".mixer") > 0:
                    raise ConfigError(f"config.json: {where}.mixer.tau must be positive")
                if "rank" not in mixer:
                    shape = (tensor_shapes or {}).get(f"l{i}.mix.a1")
                    if shape is None:
                        raise ConfigError(f"config.json: {where}.mixer gives no 'rank' and no checkpoint tensor "
                                          f"'l{i}.mix.a1' shows it")
                    mixer["rank"] = int(shape[0])
            else:
                left, right = _need(mixer, "left", where + ".mixer"), _need(mixer, "right", where + ".mixer")
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(left, key, where + ".mixer.left")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config.json: {where}.mixer.left: heads is no multiple of kv_heads")
                _number(left, "scale", where + ".mixer.left")
                for key in ("heads", "dim", "vdim"):
                    _positive_int(right, key, where + ".mixer.right")
                decay = _need(right, "decay", where + ".mixer.right")
                if not isinstance(decay, list) or len(decay) != right["heads"]:
                    raise ConfigError(f"config.json: {where}.mixer.right.decay must list one decay per head")
                for side, name in ((left, "left"), (right, "right")):
                    rot = _need(side, "rot", f"{where}.mixer.{name}")
                    dims = _need(rot, "dims", f"{where}.mixer.{name}.rot")
                    _number(rot, "base", f"{where}.mixer.{name}.rot")
                    if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > side["dim"]:
                        raise ConfigError(f"config.json: {where}.mixer.{name}.rot.dims {dims!r} must be even and at most dim")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not 'dense'")
                _positive_int(mlp, "ff", where + ".mlp")
        loop = dict(raw.get("loop") or {})
        if loop:
            start, stop, times = (_need(loop, k, "loop") for k in ("start", "stop", "times"))
            if not (isinstance(start, int) and isinstance(stop, int) and isinstance(times, int)
                    and 0 <= start <= stop <= len(layers) and times >= 1):
                raise ConfigError(f"config.json: loop {loop!r} does not fit {len(layers)} layers")
            loop = {"start": start, "stop": stop, "times": times}
        norm = _need(raw, "norm", "the model")
        eps = _number(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        cap = raw.get("logit_softcap")
        return cls(vocab=_positive_int(raw, "vocab", "the model"), width=_positive_int(raw, "width", "the model"),
                   norm_eps=eps, logit_softcap=float(cap) if cap else 0.0, layers=tuple(layers), loop=loop)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop:
            out["loop"] = dict(self.loop)
        return out

    # ------------------------------------------------------------------ parts
    @staticmethod
    def _rotary(rot: dict):
        if not rot["dims"]:
            return None
        return PartSpec("rotary", {"rotary_dim": rot["dims"], "theta": float(rot["base"]), "pairing": "half"})

    def _mixer(self, layer: dict) -> PartSpec:
        m, w, eps = layer["mixer"], self.width, self.norm_eps
        bare = {"q": "q", "k": "k", "v": "v", "o": "o"}
        if layer["type"] == "gla":
            return PartSpec("gated_linear_attention", {
                "hidden_size": w, "num_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                "tau": float(m["tau"]), "decay_rank": m["rank"], "eps": eps,
                "names": dict(bare, g="g", decay_down="a1", decay_up="a2", norm="norm")})
        left, right = m["left"], m["right"]
        attention = PartSpec("attention", {
            "hidden_size": w, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "value_dim": left["vdim"], "position": self._rotary(left["rot"]), "scale": float(left["scale"]),
            "unit_norm_eps": eps, "head_gate": True, "names": dict(bare, gate="g")})
        retention = PartSpec("retention", {
            "hidden_size": w, "num_heads": right["heads"], "key_dim": right["dim"], "value_dim": right["vdim"],
            "decay": tuple(float(d) for d in right["decay"]), "eps": eps, "position": self._rotary(right["rot"]),
            "names": dict(bare, g="g")})
        return PartSpec("side_by_side", {"hidden_size": w, "eps": eps,
                                         "branches": (("left", attention), ("right", retention))})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("layernorm", {"eps": self.norm_eps})
        names = {"mixer": "mix", "ffn": "mlp", "input_norm": "norm1"}
        layers = []
        for layer in self.layers:
            ffn = None
            if layer.get("mlp") is not None:
                ffn = PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": layer["mlp"]["ff"],
                                             "activation": "gelu_tanh",
                                             "names": {"gate": "gate", "up": "up", "down": "down"}})
            layers.append(LayerSpec(self._mixer(layer), ffn, norm, arrangement="parallel", names=names))
        # the run order: the layers before the group, the group `times` times (every pass with a
        # cache and a state of its own, the embedding mixed in again before its first layer), the rest
        n = len(layers)
        start, stop, times = (self.loop.get("start", 0), self.loop.get("stop", 0), self.loop.get("times", 1)) \
            if self.loop else (0, 0, 1)
        order, entry = [], 0
        runs = [(i, None) for i in range(start)]
        for t in range(times if stop > start else 0):
            runs += [(i, t if i == start else None) for i in range(start, stop)]
        runs += [(i, None) for i in range(stop if stop > start else start, n)]
        for i, t in runs:
            order.append(LayerCall(i, entry, True, before=(("loop", t),) if t is not None else ()))
            entry += 1
        stream_ops = ()
        if self.loop and stop > start:
            stream_ops = (("loop", PartSpec("input_injection", {"hidden_size": self.width, "times": times})),)
        return ModelSpec(
            self.vocab, self.width, tuple(layers), tuple(order), norm, tie_word_embeddings=False, weight_prefix="",
            names={"embed": "embed", "layers": "l{i}", "final_norm": "final.norm", "lm_head": "head"},
            logit_softcap=self.logit_softcap, stream_ops=stream_ops,
            name_rules=((r"\.weight$", ""), (r"\.bias$", ".b")))

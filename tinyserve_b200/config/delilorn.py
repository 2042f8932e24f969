"""Delilorn: a decoder whose blocks norm every sub-layer's input and output (RMS norms whose
weights are stored around zero), with three kinds of mixer in any order (lightning attention: a
matrix state with one decay per head; latent attention: keys and values expanded from one cached
latent per token, a sink in the softmax, optionally another layer's cache; grouped-query
attention over a window beside the first tokens of the sequence, rotary frequencies optionally
stretched for long contexts) and a mixture of experts as feed-forward.  The logits come from the
embedding table.

config.json: ``architecture`` "Delilorn"; ``vocab``, ``width``; ``norm.eps``; ``layers``: a list
of {"type": "lightning" | "latent_attention" | "attention", "mixer": {...}, "mlp": {"kind": "moe",
"expert": {"ff"}, "router": {"experts", "top"}} | null}.  Mixers: lightning gives heads, dim,
vdim, decay (one per head); latent_attention heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
rot {base, dims} and optionally kv_from (the layer whose cache it reads); attention heads,
kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, low, high, original} or none} and
mask {size, keep_first} (absent: every earlier token is visible).

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1``, ``norm1b``, ``norm2``,
``norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<k>.{up,down}``: the tensor itself
carries the name (no ".weight")."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import ClassVar

from .dudatar import _need, _number, _positive_int
from .model_config import ConfigError, LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec

LAYER_TYPES = ("lightning", "latent_attention", "attention")


def _rot(mixer: dict, where: str, most: int, exact: bool = False):
    """The checked ``rot`` entry of a mixer, or None where it has none (nothing is rotated)."""
    rot = mixer.get("rot")
    if rot is None:
        return None
    dims = _need(rot, "dims", where + ".rot")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > most or (exact and dims != most):
        raise ConfigError(f"config.json: {where}.rot.dims {dims!r} must be even and "
                          f"{'equal to' if exact else 'at most'} {most}")
    if not _number(rot, "base", where + ".rot") > 0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive")
    scaling = rot.get("scaling")
    if scaling is not None:
        for key in ("factor", "low", "high", "original"):
            _number(scaling, key, where + ".rot.scaling")
        if not (scaling["factor"] > 0 and scaling["low"] > 0 and scaling["high"] > scaling["low"] and scaling["original"] > 0):
            raise ConfigError(f"config.json: {where}.rot.scaling {scaling!r}: factor, low, original positive, high above low")
    return rot


@dataclass(frozen=True)
class DelilornConfig(ModelConfig):
    architecture: ClassVar[str] = "Delilorn"

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    layers: tuple = ()               # the config's layer entries, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "DelilornConfig":
        layers = copy.deepcopy(_need(raw, "layers", "the model"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {LAYER_TYPES}")
            mixer = _need(layer, "mixer", where)
            at = where + ".mixer"
            for key in ("heads", "dim", "vdim"):
                _positive_int(mixer, key, at)
            if kind == "lightning":
                decay = _need(mixer, "decay", at)
                if not isinstance(decay, list) or len(decay) != mixer["heads"] or \
                        any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                    raise ConfigError(f"config.json: {at}.decay must list one decay per head")
            elif kind == "latent_attention":
                source = mixer.get("kv_from")
                if isinstance(source, int) and not isinstance(source, bool) and 0 <= source < i \
                        and layers[source]["type"] == "latent_attention":
                    # what the cache row is made of is the writer's to say; a reader may leave it out
                    for key in ("kv_rank", "rot_dim", "rot"):
                        if key not in mixer and key in layers[source]["mixer"]:
                            mixer[key] = copy.deepcopy(layers[source]["mixer"][key])
                for key in ("q_rank", "kv_rank"):
                    _positive_int(mixer, key, at)
                rot_dim = mixer.get("rot_dim", 0)
                if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0 or rot_dim % 2:
                    raise ConfigError(f"config.json: {at}.rot_dim {rot_dim!r} must be even and not negative")
                mixer["rot_dim"] = rot_dim
                _number(mixer, "scale", at)
                rot = _rot(mixer, at, rot_dim)
                if rot_dim and (rot is None or rot["dims"] != rot_dim):
                    raise ConfigError(f"config.json: {at}: the rotated part of {rot_dim} is rotated as a whole (rot.dims)")
                source = mixer.get("kv_from")
                if source is not None:
                    if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                        raise ConfigError(f"config.json: {at}.kv_from {source!r} must name an earlier layer")
                    other = layers[source]
                    if other["type"] != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {at}.kv_from names layer {source}, which keeps no latent of its own")
                    if any(other["mixer"].get(k) != mixer.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        raise ConfigError(f"config.json: {at}.kv_from: layer {source} differs in kv_rank, rot_dim or rot")
            else:
                mixer.setdefault("kv_heads", mixer["heads"])        # (left out: every query head has its own)
                kv_heads = _positive_int(mixer, "kv_heads", at)
                if mixer["heads"] % kv_heads:
                    raise ConfigError(f"config.json: {at}: heads is no multiple of kv_heads")
                _number(mixer, "scale", at)
                _rot(mixer, at, mixer["dim"])
                mask = mixer.get("mask")
                if mask is not None:
                    _positive_int(mask, "size", at + ".mask")
                    keep = mask.get("keep_first", 0)
                    if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
                        raise ConfigError(f"config.json: {at}.mask.keep_first {keep!r} must be an integer, not negative")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not 'moe'")
                _positive_int(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                router = _need(mlp, "router", where + ".mlp")
                experts = _positive_int(router, "experts", where + ".mlp.router")
                if _positive_int(router, "top", where + ".mlp.router") > experts:
                    raise ConfigError(f"config.json: {where}.mlp.router: top exceeds experts")
        norm = _need(raw, "norm", "the model")
        eps = _number(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cls(vocab=_positive_int(raw, "vocab", "the model"), width=_positive_int(raw, "width", "the model"),
                   norm_eps=eps, layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}

    # ------------------------------------------------------------------ parts
    @staticmethod
    def _rotary(rot):
        if not rot or not rot["dims"]:
            return None
        return PartSpec("rotary", {"rotary_dim": rot["dims"], "theta": float(rot["base"]), "pairing": "half",
                                   "scaling": dict(rot["scaling"]) if rot.get("scaling") else None})

    def _mixer(self, layer: dict) -> PartSpec:
        m, w, eps = layer["mixer"], self.width, self.norm_eps
        if layer["type"] == "lightning":
            return PartSpec("lightning", {
                "hidden_size": w, "num_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                "decay": tuple(float(d) for d in m["decay"]), "eps": eps,
                "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}})
        if layer["type"] == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": w, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]),
                "eps": eps, "position": self._rotary(m.get("rot")), "own_kv": m.get("kv_from") is None})
        mask = m.get("mask") or {}
        return PartSpec("attention", {
            "hidden_size": w, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "position": self._rotary(m.get("rot")), "scale": float(m["scale"]),
            "window": mask.get("size", 0), "keep_first": mask.get("keep_first", 0),
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"eps": self.norm_eps, "offset": 1.0})
        names = {"mixer": "mix", "ffn": "mlp", "input_norm": "norm1", "mixer_out_norm": "norm1b",
                 "post_mixer_norm": "norm2", "ffn_out_norm": "norm2b"}
        layers, order = [], []
        entry_of = {}                       # layer -> the cache entry its mixer reads
        for i, layer in enumerate(self.layers):
            ffn = None
            if layer.get("mlp") is not None:
                mlp = layer["mlp"]
                ffn = PartSpec("moe", {"hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"],
                                       "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                                       "activation": "relu_squared"})
            layers.append(LayerSpec(self._mixer(layer), ffn, norm, arrangement="sandwich", names=names))
            source = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
            entry_of[i] = entry_of[source] if source is not None else i
            order.append(LayerCall(i, entry_of[i], writes_cache=source is None))
        # a layer without a feed-forward has no use for the two norms around one, should a checkpoint hold them
        unread = tuple(rf"l{i}\.norm2b?" for i, layer in enumerate(self.layers) if layer.get("mlp") is None)
        return ModelSpec(
            self.vocab, self.width, tuple(layers), tuple(order), norm, tie_word_embeddings=True, weight_prefix="",
            names={"embed": "embed", "layers": "l{i}", "final_norm": "final.norm"},
            name_rules=((r"\.weight$", ""),), unread_names=unread)

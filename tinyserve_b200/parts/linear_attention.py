"""Mixers with a matrix state instead of a cache: per request and head

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,

S of key size x value size in 32-bit, kept in the request's state slot between steps and zero
for a request that starts.  What the two kinds share (fused projection, state, output norm over
the value size, silu gate, output projection) is ``MatrixStateMixer``; they differ in a_t:

* ``Retention``: one constant decay per head (a list), rotary positions on q and k, k times
  key_dim^(-1/2), no weight on the output norm.
* ``GatedLinearAttention``: one decay per key channel and token, a = sigmoid(z)^(1 / tau) with
  z = W2 (W1 h) + b a low-rank projection of the mixer's input, q times key_dim^(-1/2), a weight
  of value size on the output norm (one for all heads).

* ``Lightning``: one constant decay per head (a list), silu on q, k and v, no positions and no
  factor; the heads of a token are normed together with one weight over all of them and multiplied
  by sigmoid (not silu) of the gate.

Everything behind the projections is 32-bit (angles, decays, state, output norm):
csrc/linear_attention.cu.  The decay logits z leave their product in 32-bit."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, ParamSpec, Source, StateSpec, build_position_encoding, register_mixer

DEFAULT_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "g_proj", "o": "o_proj",
                 "decay_down": "a1", "decay_up": "a2", "norm": "norm"}


class MatrixStateMixer(Mixer):
    tree_name = "mixer"
    capturable = True
    accepts_scaled_rows = True

    def __init__(self, hidden_size, num_heads, key_dim, value_dim, eps, names=None):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.value_dim, self.eps = key_dim, value_dim, float(eps)
        if not ops.linear_attention_supports(key_dim) or not 0 < value_dim <= ops.LINEAR_ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"linear attention: key size {key_dim} or value size {value_dim} is not supported")
        self.qk_size, self.v_size = num_heads * key_dim, num_heads * value_dim

    def _projection_rows(self):
        qk, v, nm = self.qk_size, self.v_size, self.names
        return [(nm["q"], qk), (nm["k"], qk), (nm["v"], v), (nm["g"], v)]

    def param_specs(self):
        sources, at = [], 0
        for name, rows in self._projection_rows():
            sources.append(Source(f"{name}.weight", at, at + rows))
            at += rows
        return {
            "in_proj.weight": ParamSpec((at, self.hidden_size), sources=tuple(sources)),
            "o_proj.weight": ParamSpec((self.hidden_size, self.v_size),
                                       sources=(Source(f"{self.names['o']}.weight", 0, self.hidden_size),)),
        }

    def state_spec(self):
        return StateSpec((self.num_heads, self.key_dim, self.value_dim), "float32")

    def _split(self, h):
        proj = ops.materialize(ops.linear(h, self.w["in_proj.weight"]))
        qk, v = self.qk_size, self.v_size
        return proj, proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + v], proj[:, 2 * qk + v:2 * qk + 2 * v]


class Retention(MatrixStateMixer):
    def __init__(self, hidden_size, num_heads, key_dim, value_dim, decay, eps, position=None, names=None):
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, names)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != num_heads:
            raise ValueError(f"retention: {len(self.decay_values)} decays for {num_heads} heads")
        self.position = build_position_encoding(position) if position is not None else None
        self.decay = None

    def children(self):
        return {"position": self.position} if self.position is not None else {}

    def prepare(self, runtime):
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def forward(self, h, ctx, call):
        _, q, k, v, g = self._split(h)
        out = ops.linear_attention(q, k, v, g, ctx.state(call.state), ctx, self.num_heads, self.key_dim,
                                   self.value_dim, ctx.dtype, decay=self.decay, rotary=self.position,
                                   k_scale=self.key_dim ** -0.5, eps=self.eps)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


class GatedLinearAttention(MatrixStateMixer):
    def __init__(self, hidden_size, num_heads, key_dim, value_dim, tau, decay_rank, eps, names=None):
        self.decay_rank = int(decay_rank)
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, names)
        self.tau = float(tau)
        if not self.tau > 0 or self.decay_rank <= 0:
            raise ValueError("gated linear attention: tau and the rank of the decay projection must be positive")

    def _projection_rows(self):
        # the first factor of the decay projection reads the same input: it rides with q, k, v and the gate
        return super()._projection_rows() + [(self.names["decay_down"], self.decay_rank)]

    def param_specs(self):
        specs = super().param_specs()
        nm = self.names
        specs["decay_up.weight"] = ParamSpec((self.qk_size, self.decay_rank),
                                             sources=(Source(f"{nm['decay_up']}.weight", 0, self.qk_size),))
        # drawn like a matrix in the random-weights mode: a bias of zeros would hide a fault
        specs["decay_up.bias"] = ParamSpec((self.qk_size,), role="vector", init="normal",
                                           sources=(Source(f"{nm['decay_up']}.bias", 0, self.qk_size),))
        specs["norm.weight"] = ParamSpec((self.value_dim,), role="vector", init="norm_weight",
                                         sources=(Source(f"{nm['norm']}.weight", 0, self.value_dim),))
        return specs

    def forward(self, h, ctx, call):
        proj, q, k, v, g = self._split(h)
        low = proj[:, 2 * self.qk_size + 2 * self.v_size:]
        z = ops.linear(low, self.w["decay_up.weight"], self.w["decay_up.bias"], out_float32=True)
        out = ops.linear_attention(q, k, v, g, ctx.state(call.state), ctx, self.num_heads, self.key_dim,
                                   self.value_dim, ctx.dtype, decay_logits=z, tau=self.tau,
                                   q_scale=self.key_dim ** -0.5, norm_weight=self.w["norm.weight"], eps=self.eps)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


class Lightning(MatrixStateMixer):
    def __init__(self, hidden_size, num_heads, key_dim, value_dim, decay, eps, names=None):
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, names)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != num_heads:
            raise ValueError(f"lightning: {len(self.decay_values)} decays for {num_heads} heads")
        self.decay = None

    def param_specs(self):
        specs = super().param_specs()
        specs["norm.weight"] = ParamSpec((self.v_size,), role="vector", init="norm_weight",
                                         sources=(Source(f"{self.names['norm']}.weight", 0, self.v_size),))
        return specs

    def prepare(self, runtime):
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def forward(self, h, ctx, call):
        _, q, k, v, g = self._split(h)
        out = ops.linear_attention(q, k, v, g, ctx.state(call.state), ctx, self.num_heads, self.key_dim,
                                   self.value_dim, ctx.dtype, decay=self.decay, norm_weight=self.w["norm.weight"],
                                   eps=self.eps, input_activation="silu", gate_activation="sigmoid", joint_norm=True)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


register_mixer("retention", Retention)
register_mixer("lightning", Lightning)
register_mixer("gated_linear_attention", GatedLinearAttention)

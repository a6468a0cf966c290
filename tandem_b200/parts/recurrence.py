"""Recurrences with per-request state as mixers: linear attention with a fixed decay per head
(``DecayRecurrence``) and the selective state-space layer whose decay comes from the token
(``SelectiveRecurrence``); both run the same scan kernel.

Linear attention with a fixed decay per head:

S <- decay_h S + k v^T and o = S^T q per head, the state [heads, key_dim, value_dim] in float32 in
the cache manager's state slots (zero when a request is admitted, carried from step to step).  What
surrounds the recurrence is chosen by :class:`~tandem_b200.config.plan.DecayRecurrenceSpec`: an
activation on q, k and v, a rotary encoding of q and k, a factor on k, how o is normalised, and
the activation of the output gate.  One fused projection (rows [q | k | v | g]) with a float32 result.
"""

from __future__ import annotations

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import DecayRecurrenceSpec, ParamSpec, SelectiveRecurrenceSpec, WeightSource
from tandem_b200.kernels import deferred, ops
from tandem_b200.kernels import recurrence as kernels
from tandem_b200.parts.base import Mixer, StateNeed, StepContext

_SUFFIX = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}


def _name(spec, local: str) -> str:
    return f"{spec.prefix}.{dict(spec.names).get(local, _SUFFIX[local])}"


class DecayRecurrence(Mixer):
    capturable = True  # forward only launches kernels; requests and their state rows are read from device arrays
    takes_deferred = True

    @staticmethod
    def params(spec: DecayRecurrenceSpec) -> dict:
        qk, v, H = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.hidden_size
        out = {
            "qkvg": ParamSpec((2 * qk + 2 * v, H), (WeightSource(_name(spec, "q"), 0, qk), WeightSource(_name(spec, "k"), qk, qk),
                                                    WeightSource(_name(spec, "v"), 2 * qk, v),
                                                    WeightSource(_name(spec, "g"), 2 * qk + v, v))),
            "o": ParamSpec((H, v), (WeightSource(_name(spec, "o")),)),
        }
        if spec.output_norm == "all_heads":
            out["norm"] = ParamSpec((v,), (WeightSource(_name(spec, "norm")),), role="vector")
        return out

    @staticmethod
    def state_need(spec: DecayRecurrenceSpec) -> StateNeed:
        return StateNeed((spec.num_heads, spec.key_dim, spec.value_dim), torch.float32)

    def __init__(self, spec: DecayRecurrenceSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if len(spec.decay) != spec.num_heads:
            raise ConfigError(f"{len(spec.decay)} decays for {spec.num_heads} heads")
        if spec.output_norm not in ("per_head", "all_heads"):
            raise ConfigError(f"no output norm {spec.output_norm!r} (per_head or all_heads)")
        if spec.gate not in ("silu", "sigmoid") or spec.activation not in ("none", "silu"):
            raise ConfigError(f"gate {spec.gate!r} / activation {spec.activation!r}: the gate is silu or sigmoid, the "
                              "activation none or silu")
        if spec.rotary_dim % 2 or not 0 <= spec.rotary_dim <= spec.key_dim:
            raise ConfigError(f"rotary_dim {spec.rotary_dim} must be even and at most the key size {spec.key_dim}")
        self.spec = spec
        self.qkvg, self.o, self.norm = weights["qkvg"], weights["o"], weights.get("norm")
        self.decay = torch.tensor(spec.decay, dtype=torch.float64).to(torch.float32).to(device)
        self.freq = None
        if spec.rotary_dim:
            i = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
            self.freq = (float(spec.rotary_base) ** (-2.0 * i / spec.rotary_dim)).to(torch.float32).to(device)

    def forward(self, x, ctx: StepContext, defer: bool = False):
        s = self.spec
        x = deferred.tensor(x)
        proj = ops.linear(x, self.qkvg, out_dtype=torch.float32)
        kernels.prepare(proj, ctx.positions, self.freq, s.num_heads, s.key_dim, s.value_dim, s.activation, s.key_scale)
        o = kernels.scan(proj, ctx.cu_seqlens, ctx.state_slots, ctx.num_seqs, ctx.state(self), self.decay, s.num_heads,
                         s.key_dim, s.value_dim)
        gate = proj[:, 2 * s.num_heads * s.key_dim + s.num_heads * s.value_dim:]
        y = kernels.finish(o, gate, self.norm, s.num_heads, s.value_dim, s.output_norm == "per_head", s.gate, s.norm_eps,
                           ctx.dtype)
        out = ops.linear(y, self.o, out_dtype=torch.float32)
        if defer:
            return deferred.Unsummed(out, None, ctx.dtype)
        return out if ctx.dtype == torch.float32 else ops.bias_act(out, None, "none", ctx.dtype)


class SelectiveRecurrence(Mixer):
    """A state-space recurrence whose decay and step size come from the token (see
    :class:`~tandem_b200.config.plan.SelectiveRecurrenceSpec`).  One projection with a float32 result;
    one kernel runs the causal convolution (its earlier inputs from the request's state), SiLU, the
    softplus of the step size and the decay; the scan is the package's recurrence kernel with a decay per
    token and q and k shared by groups of heads; one kernel adds the skip term, gates, normalises in
    equal parts and rounds.  A request's state row holds S [H, N, P] and behind it the convolution's
    last inputs [taps - 1, channels], both float32."""

    capturable = True  # forward only launches kernels; requests and their state rows are read from device arrays
    _SUFFIX = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
               "norm": "norm", "o": "o"}

    @classmethod
    def _name(cls, spec, local: str) -> str:
        return f"{spec.prefix}.{dict(spec.names).get(local, cls._SUFFIX[local])}"

    @staticmethod
    def sizes(spec: SelectiveRecurrenceSpec) -> tuple:
        """(inner, columns of B and C together, convolution channels)."""
        inner, gn2 = spec.num_heads * spec.value_dim, 2 * spec.groups * spec.state_dim
        return inner, gn2, inner + gn2

    @classmethod
    def params(cls, spec: SelectiveRecurrenceSpec) -> dict:
        inner, gn2, channels = cls.sizes(spec)
        H = spec.num_heads

        def vector(local: str, *shape) -> ParamSpec:
            return ParamSpec(tuple(shape), (WeightSource(cls._name(spec, local)),), role="vector")

        return {
            "in": ParamSpec((inner + channels + H, spec.hidden_size), (WeightSource(cls._name(spec, "in")),)),
            "conv": vector("conv", channels, spec.conv_taps), "conv_bias": vector("conv_bias", channels),
            "dt_bias": vector("dt_bias", H), "a_log": vector("a_log", H), "skip": vector("skip", H),
            "norm": vector("norm", inner),
            "o": ParamSpec((spec.hidden_size, inner), (WeightSource(cls._name(spec, "o")),)),
        }

    @classmethod
    def state_need(cls, spec: SelectiveRecurrenceSpec) -> StateNeed:
        inner, _, channels = cls.sizes(spec)
        return StateNeed((inner * spec.state_dim + (spec.conv_taps - 1) * channels,), torch.float32)

    def __init__(self, spec: SelectiveRecurrenceSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.groups <= 0 or spec.num_heads % spec.groups:
            raise ConfigError(f"{spec.num_heads} heads cannot share {spec.groups} groups of B and C")
        if spec.norm_groups <= 0 or (spec.num_heads * spec.value_dim) % spec.norm_groups:
            raise ConfigError(f"{spec.norm_groups} parts do not divide a row of {spec.num_heads * spec.value_dim}")
        if spec.conv_taps <= 0:
            raise ConfigError("the convolution needs at least the current token's tap")
        self.spec = spec
        self.w = weights

    def forward(self, x, ctx: StepContext, defer: bool = False):
        s, w = self.spec, self.w
        inner, gn2, channels = self.sizes(s)
        x = deferred.tensor(x)
        proj = ops.linear(x, w["in"], out_dtype=torch.float32)
        state = ctx.state(self)
        conv_offset = inner * s.state_dim
        rows, decay = kernels.selective_prepare(proj, w["conv"], w["conv_bias"], w["dt_bias"], w["a_log"], state, conv_offset, ctx,
                                                s.num_heads, s.value_dim, gn2, s.conv_taps)
        kernels.conv_state_update(proj, inner, state, conv_offset, ctx, channels, s.conv_taps)
        # rows = [x | B | C | dt x]: q = C, k = B, v = dt x
        o = kernels.scan_general(rows, ctx.cu_seqlens, ctx.state_slots, ctx.num_seqs, state, None, decay, s.num_heads, s.groups,
                                 s.state_dim, s.value_dim, inner + gn2 // 2, inner, inner + gn2)
        y = kernels.selective_finish(o, rows, proj, w["skip"], w["norm"], s.num_heads, s.value_dim, s.norm_groups, s.norm_eps,
                                     ctx.dtype)
        return ops.linear(y, w["o"], out_dtype=torch.float32)

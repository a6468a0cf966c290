"""Linear attention with a fixed decay per head, as a mixer with per-request state.

S <- decay_h S + k v^T and o = S^T q per head, the state [heads, key_dim, value_dim] in float32 in
the cache manager's state slots (zero when a request is admitted, carried from step to step).  What
surrounds the recurrence is chosen by :class:`~tandem_b200.config.plan.DecayRecurrenceSpec`: an
activation on q, k and v, a rotary encoding of q and k, a factor on k, how o is normalised, and
the activation of the output gate.  One fused projection (rows [q | k | v | g]) with a float32 result.
"""

from __future__ import annotations

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import DecayRecurrenceSpec, ParamSpec, WeightSource
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

"""Gated feed-forward (SwiGLU): down(act(gate(x)) * up(x)) with gate and up as one product
(12vivi/tandem python/tandem/layers/mlp.py:23-44; rows [gate | up] as python/tandem/models/loader.py:52-53
stacks them), and the plain two-layer feed-forward down(act(up(x) + b) ) + b with optional biases."""

from __future__ import annotations

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import DenseMLPSpec, GatedMLPSpec, ParamSpec, WeightSource
from tandem_b200.kernels import deferred, ops
from tandem_b200.parts.base import FeedForward, StepContext


class GatedMLP(FeedForward):
    takes_deferred = True  # x may be a norm whose scale is pending; with ``defer`` the last product may stay pending

    @staticmethod
    def params(spec: GatedMLPSpec) -> dict:
        H, I, p = spec.hidden_size, spec.intermediate_size, spec.prefix
        return {
            "gate_up": ParamSpec((2 * I, H), (WeightSource(f"{p}.gate_proj.weight", 0, I),
                                              WeightSource(f"{p}.up_proj.weight", I, I))),
            "down": ParamSpec((H, I), (WeightSource(f"{p}.down_proj.weight"),)),
        }

    def __init__(self, spec: GatedMLPSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.activation != "silu":
            raise ConfigError(f"gated_mlp has no activation {spec.activation!r} (only silu)")
        self.gate_up = weights["gate_up"]
        self.down = weights["down"]

    def forward(self, x, ctx: StepContext, defer: bool = False):
        return ops.linear(ops.gated_linear(x, self.gate_up), self.down, defer=defer)


class DenseMLP(FeedForward):
    """down(act(up(x) + up_bias)) + down_bias.  The first product comes back in float32, bias and
    activation are one kernel that rounds once; the second may come back with its bias not yet added."""

    takes_deferred = True
    _SUFFIX = {"up": "up", "down": "down", "up_bias": "up.b", "down_bias": "down.b"}

    @classmethod
    def _name(cls, spec, local: str) -> str:
        return f"{spec.prefix}.{dict(spec.names).get(local, cls._SUFFIX[local])}"

    @classmethod
    def params(cls, spec: DenseMLPSpec) -> dict:
        H, I = spec.hidden_size, spec.intermediate_size
        out = {"up": ParamSpec((I, H), (WeightSource(cls._name(spec, "up")),)),
               "down": ParamSpec((H, I), (WeightSource(cls._name(spec, "down")),))}
        if spec.bias:
            out["up_bias"] = ParamSpec((I,), (WeightSource(cls._name(spec, "up_bias")),), role="vector")
            out["down_bias"] = ParamSpec((H,), (WeightSource(cls._name(spec, "down_bias")),), role="vector")
        return out

    def __init__(self, spec: DenseMLPSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.activation not in ("gelu_tanh", "silu", "none"):
            raise ConfigError(f"dense_mlp has no activation {spec.activation!r} (gelu_tanh, silu or none)")
        self.activation = spec.activation
        self.up, self.down = weights["up"], weights["down"]
        self.up_bias, self.down_bias = weights.get("up_bias"), weights.get("down_bias")

    def forward(self, x, ctx: StepContext, defer: bool = False):
        x = deferred.tensor(x)
        a = ops.bias_act(ops.linear(x, self.up, out_dtype=torch.float32), self.up_bias, self.activation, ctx.dtype)
        y = ops.linear(a, self.down, out_dtype=torch.float32)
        if defer:
            return deferred.Unsummed(y, self.down_bias, ctx.dtype)
        return ops.bias_act(y, self.down_bias, "none", ctx.dtype)

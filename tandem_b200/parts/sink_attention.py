"""Grouped-query attention with optional projection biases, unit-norm q and k, capped scores, a
learned bias by distance, a window that keeps the first tokens, a softmax sink and value mixing
across layers.  Every option is a field of :class:`~tandem_b200.config.plan.SinkAttentionSpec`;
the mixer does not know which model it serves.

One fused projection (rows [q | k | v]) with a float32 result; one kernel adds the biases,
normalises q and k, mixes and stores k and v; one kernel attends over the paged cache (the tokens
of the step included, so a portion sees itself through the cache): one warp per token and head
in float32 and wherever the others do not take the shape, query tiles on the tensor cores for
bfloat16 steps that bring prompt portions, a token's keys cut over several blocks for bfloat16
steps of single tokens.  The output projection comes
back with its bias not yet added (``deferred.Unsummed``) when the arrangement asks for that.
"""

from __future__ import annotations

import torch

from tandem_b200.cache.manager import KVNeed
from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import ParamSpec, SinkAttentionSpec, WeightSource
from tandem_b200.kernels import deferred, ops
from tandem_b200.kernels import sink_attention as kernels
from tandem_b200.parts.base import Mixer, StepContext

_SUFFIX = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
           "rel": "rel", "sink": "sink", "vmix": "vmix"}


def _name(spec, local: str) -> str:
    return f"{spec.prefix}.{dict(spec.names).get(local, _SUFFIX[local])}"


class SinkAttention(Mixer):
    capturable = True  # forward only launches kernels and reads the batch from device arrays
    takes_deferred = True

    @staticmethod
    def params(spec: SinkAttentionSpec) -> dict:
        q, k, v, H = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.num_kv_heads * spec.value_dim, spec.hidden_size
        out = {
            "qkv": ParamSpec((q + k + v, H), (WeightSource(_name(spec, "q"), 0, q), WeightSource(_name(spec, "k"), q, k),
                                              WeightSource(_name(spec, "v"), q + k, v))),
            "o": ParamSpec((H, spec.num_heads * spec.value_dim), (WeightSource(_name(spec, "o")),)),
        }
        if spec.bias:
            out["qkv_bias"] = ParamSpec((q + k + v,), (WeightSource(_name(spec, "q_bias"), 0, q),
                                                       WeightSource(_name(spec, "k_bias"), q, k),
                                                       WeightSource(_name(spec, "v_bias"), q + k, v)), role="vector")
            out["o_bias"] = ParamSpec((H,), (WeightSource(_name(spec, "o_bias")),), role="vector")
        if spec.distance_bias is not None:
            out["rel"] = ParamSpec((spec.distance_bias.buckets, spec.num_heads), (WeightSource(_name(spec, "rel")),), role="vector")
        if spec.sink:
            out["sink"] = ParamSpec((spec.num_heads,), (WeightSource(_name(spec, "sink")),), role="vector")
        if spec.value_mix is not None:
            out["vmix"] = ParamSpec((), (WeightSource(_name(spec, "vmix")),), role="vector")
        return out

    @staticmethod
    def kv_need(spec: SinkAttentionSpec) -> KVNeed:
        return KVNeed(spec.num_kv_heads, spec.head_dim, spec.window, value_dim=spec.value_dim,
                      keep_first=spec.keep_first if spec.window else 0)

    def __init__(self, spec: SinkAttentionSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ConfigError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} kv heads")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError(f"a window of {spec.window} keys shows a token nothing")
        self.spec = spec
        self.qkv, self.o = weights["qkv"], weights["o"]
        self.qkv_bias, self.o_bias = weights.get("qkv_bias"), weights.get("o_bias")
        self.sink = weights.get("sink")
        self.vmix = weights.get("vmix")
        self.bias_by_distance = None
        if spec.distance_bias is not None:
            b = spec.distance_bias
            if b.buckets < 2 or b.max_distance <= b.buckets // 2:
                raise ConfigError(f"a distance bias of {b.buckets} buckets needs a largest distance beyond {b.buckets // 2}, "
                                  f"got {b.max_distance}")
            self.bias_by_distance = kernels.expand_distance_bias(weights["rel"], b.bucket, b.max_distance)

    def _tiles_key(self):
        return ("sink_attention_tiles", self.spec.num_heads // self.spec.num_kv_heads)

    def step_arrays(self, ctx: StepContext, out: dict) -> None:
        """Steps that bring prompt portions run the tensor-core kernel where it takes the shape: its
        query tiles are cut here, once per step for all layers with as many query heads per kv head."""
        s, key = self.spec, self._tiles_key()
        cols = (s.num_heads + s.num_kv_heads) * s.head_dim + s.num_kv_heads * s.value_dim
        if key in out or ctx.max_new < 2 or \
                not kernels.tiles_apply(ctx.dtype, s.head_dim, s.value_dim, s.num_heads // s.num_kv_heads, cols):
            return
        out[key] = kernels.plan_tiles(ctx.host_starts, ctx.host_lens, s.num_heads // s.num_kv_heads)

    def step_array_capacity(self, bucket: int, max_model_len: int, page_size: int, out: dict) -> None:
        """Steps of single tokens (the ones CUDA graphs capture) need no arrays: they run the kernel of one
        warp per token and head, which reads the batch from the context's device arrays."""

    def forward(self, x, ctx: StepContext, defer: bool = False):
        s = self.spec
        x = deferred.tensor(x)
        qkv = ops.linear(x, self.qkv, out_dtype=torch.float32)
        kv = ctx.kv(self)
        other = None
        if s.value_mix is not None:
            key = ("value_mix", s.value_mix)
            if s.value_mix_first:
                ctx.scratch[key] = qkv[:, (s.num_heads + s.num_kv_heads) * s.head_dim:]  # its v columns, once the biases are in
            else:
                other = ctx.scratch.get(key)
                if other is None:
                    raise RuntimeError(f"values of {s.value_mix!r} are mixed in before the layer that makes them has run")
        kernels.prepare(qkv, self.qkv_bias, other, self.vmix if other is not None else None, kv, s.num_heads, s.num_kv_heads,
                        s.head_dim, s.value_dim, s.unit_norm, s.norm_eps)
        tiles = ctx.extras.get(self._tiles_key())
        cols = qkv.shape[1]
        if tiles is not None and kernels.tiles_apply(kv.k.dtype, s.head_dim, s.value_dim, s.num_heads // s.num_kv_heads, cols):
            o = kernels.attend_tiles(qkv, kv, tiles, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.window,
                                     s.keep_first, s.scale, s.softcap, self.bias_by_distance, self.sink)
        elif ctx.max_new == 1 and kernels.split_applies(kv.k.dtype, s.head_dim, s.value_dim, s.num_heads // s.num_kv_heads, cols):
            o = kernels.attend_split(qkv, kv, ctx, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.window, s.keep_first,
                                     s.scale, s.softcap, self.bias_by_distance, self.sink)
        else:
            o = kernels.attend(qkv, kv, ctx, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.window, s.keep_first,
                               s.scale, s.softcap, self.bias_by_distance, self.sink)
        y = ops.linear(o, self.o, out_dtype=torch.float32)
        if defer:
            return deferred.Unsummed(y, self.o_bias, ctx.dtype)
        return ops.bias_act(y, self.o_bias, "none", ctx.dtype)

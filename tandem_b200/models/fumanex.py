"""Fumanex: configuration -> model plan, and its random-weight recipe.

Every layer is a "parallel" arrangement: one RMSNorm (``l<i>.norm1``) whose output both the mixer
(``l<i>.mix.*``) and the dense feed-forward (``l<i>.mlp.*``) read.  The three kinds of mixer map
onto two parts of the package: "attention" -> ``sink_attention`` with all of its options on;
"retention" and "lightning" -> ``decay_recurrence`` in two dressings (rotary q/k, scaled k, heads
normalised one by one, SiLU gate; or SiLU on q/k/v, one weighted norm over all heads, sigmoid gate).
The embedding is scaled, the logits are scaled, and there is no table of positions.
"""

from __future__ import annotations

from typing import Iterator

import torch

from tandem_b200.config.fumanex_config import NO_POSITION_LIMIT, FumanexConfig
from tandem_b200.config.plan import (
    DecayRecurrenceSpec,
    DenseMLPSpec,
    DistanceBiasSpec,
    EmbeddingSpec,
    HeadSpec,
    LayerSpec,
    ModelPlan,
    NormSpec,
    RunStep,
    SinkAttentionSpec,
)
from tandem_b200.registry import Architecture, register_architecture


def mixer_spec(cfg: FumanexConfig, i: int, first_mixing: int):
    L, m, p = cfg.layers[i], cfg.layers[i].mixer, f"l{i}.mix"
    if L.type == "attention":
        return SinkAttentionSpec(
            "sink_attention", prefix=p, hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
            value_dim=m.vdim, scale=m.scale, bias=True, unit_norm=True, norm_eps=cfg.norm_eps, softcap=m.softcap,
            distance_bias=DistanceBiasSpec(m.bias_buckets, m.bias_max), window=m.window,
            keep_first=m.keep_first if m.window else 0, sink=True, value_mix="v_mix" if m.v_mix else None,
            value_mix_first=m.v_mix and i == first_mixing)
    if L.type == "retention":
        return DecayRecurrenceSpec(
            "decay_recurrence", prefix=p, hidden_size=cfg.width, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
            decay=m.decay, activation="none", rotary_dim=m.rot_dims, rotary_base=m.rot_base, key_scale=m.dim ** -0.5,
            output_norm="per_head", gate="silu", norm_eps=cfg.norm_eps)
    return DecayRecurrenceSpec(
        "decay_recurrence", prefix=p, hidden_size=cfg.width, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
        decay=m.decay, activation="silu", key_scale=1.0, output_norm="all_heads", gate="sigmoid", norm_eps=cfg.norm_eps)


def build_plan(cfg: FumanexConfig) -> ModelPlan:
    mixing = [i for i, l in enumerate(cfg.layers) if l.type == "attention" and l.mixer.v_mix]
    first_mixing = mixing[0] if mixing else -1
    layers = []
    for i, L in enumerate(cfg.layers):
        slots = dict(norm=NormSpec("rmsnorm", cfg.width, cfg.norm_eps, f"l{i}.norm1"),
                     mixer=mixer_spec(cfg, i, first_mixing))
        if L.ff is not None:
            slots["feed_forward"] = DenseMLPSpec("dense_mlp", prefix=f"l{i}.mlp", hidden_size=cfg.width,
                                                 intermediate_size=L.ff, activation="gelu_tanh", bias=True)
        layers.append(LayerSpec.of("parallel", **slots))
    return ModelPlan(
        embedding=EmbeddingSpec(cfg.vocab, cfg.width, "embed", scale=cfg.embedding_scale),
        layers=tuple(layers),
        order=tuple(RunStep(i) for i in range(len(layers))),
        final_norm=NormSpec("rmsnorm", cfg.width, cfg.norm_eps, "final.norm"),
        head=HeadSpec(cfg.vocab, cfg.width, "head", scale=cfg.logit_scale),
        max_position=NO_POSITION_LIMIT,
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


def tensor_shapes(cfg: FumanexConfig) -> dict:
    """Checkpoint tensor name -> shape, in file order."""
    W = cfg.width
    shapes: dict = {"embed": (cfg.vocab, W)}
    for i, L in enumerate(cfg.layers):
        m, p = L.mixer, f"l{i}.mix"
        shapes[f"l{i}.norm1"] = (W,)
        if L.type == "attention":
            for name, rows in (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)):
                shapes[f"{p}.{name}"] = (rows, W)
                shapes[f"{p}.{name}.b"] = (rows,)
            shapes[f"{p}.rel"] = (m.bias_buckets, m.heads)
            if m.v_mix:
                shapes[f"{p}.vmix"] = ()
            shapes[f"{p}.sink"] = (m.heads,)
            shapes[f"{p}.o"] = (W, m.heads * m.vdim)
            shapes[f"{p}.o.b"] = (W,)
        else:
            shapes[f"{p}.q"] = (m.heads * m.dim, W)
            shapes[f"{p}.k"] = (m.heads * m.dim, W)
            shapes[f"{p}.v"] = (m.heads * m.vdim, W)
            shapes[f"{p}.g"] = (m.heads * m.vdim, W)
            shapes[f"{p}.o"] = (W, m.heads * m.vdim)
            if L.type == "lightning":
                shapes[f"{p}.norm"] = (m.heads * m.vdim,)
        if L.ff is not None:
            shapes[f"l{i}.mlp.up"] = (L.ff, W)
            shapes[f"l{i}.mlp.up.b"] = (L.ff,)
            shapes[f"l{i}.mlp.down"] = (W, L.ff)
            shapes[f"l{i}.mlp.down.b"] = (W,)
    shapes["final.norm"] = (W,)
    shapes["head"] = (cfg.vocab, W)
    return shapes


def random_weights(cfg: FumanexConfig, seed: int, device: str = "cpu", dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_spread: float = 0.1) -> Iterator[tuple]:
    """Seeded random tensors by checkpoint name, each from a generator of its own: matrices and the
    embedding N(0, std) (the embedding N(0, 1 / embedding scale), so the stream starts near unit size),
    norm weights 1 + U(-spread, spread), biases, sinks and distance biases N(0, 0.5), mixing shares U(0.2, 0.8)."""
    for index, (name, shape) in enumerate(tensor_shapes(cfg).items()):
        g = torch.Generator(device=device).manual_seed((seed * 1_000_003 + index) % (2**63 - 1))
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "vmix":
            t = 0.2 + 0.6 * torch.rand(shape, generator=g, device=device, dtype=torch.float32)
        elif leaf in ("norm1", "norm"):
            t = 1.0 + norm_spread * (2.0 * torch.rand(shape, generator=g, device=device, dtype=torch.float32) - 1.0)
        elif leaf in ("b", "sink", "rel"):
            t = torch.empty(shape, device=device, dtype=torch.float32).normal_(0.0, 0.5, generator=g)
        elif name == "embed":
            t = torch.empty(shape, device=device, dtype=torch.float32).normal_(0.0, 1.0 / max(cfg.embedding_scale, 1e-6), generator=g)
        else:
            t = torch.empty(shape, device=device, dtype=torch.float32).normal_(0.0, std, generator=g)
        yield name, t.to(dtype)


register_architecture(Architecture("Fumanex", FumanexConfig, build_plan, random_weights,
                                    complete=FumanexConfig.with_checkpoint_shapes))

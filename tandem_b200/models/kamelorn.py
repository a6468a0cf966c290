"""Kamelorn: configuration -> model plan, and its random-weight recipe.

Every layer is a "connected" arrangement: norm, mixer and the link that ties the mixer to the
residual (``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.hc1.*``), then the same for the feed-forward
(``l<i>.norm2``, ``l<i>.mlp.*``, ``l<i>.hc2.*``) where the layer has one.  The two kinds of mixer
map onto two parts of the package: "mamba2" -> ``selective_recurrence``, "latent_attention" ->
``latent_attention``; the feed-forwards onto ``gated_mlp`` (dense) and ``routed_mlp`` (experts).
With ``streams`` in the file the residual is that many streams and every link has learned
coefficients; without it the links are the plain sum x <- x + residual_mult * y.  A looped span
of layers appears in the plan's running order once per pass, each pass with a cache of its own.
The embedding is scaled and there is no table of positions.
"""

from __future__ import annotations

from typing import Iterator

import torch

from tandem_b200.config.kamelorn_config import NO_POSITION_LIMIT, KamelornConfig
from tandem_b200.config.plan import (
    EmbeddingSpec,
    GatedMLPSpec,
    HeadSpec,
    LatentAttentionSpec,
    LayerSpec,
    ModelPlan,
    NormSpec,
    RoutedMLPSpec,
    RunStep,
    SelectiveRecurrenceSpec,
    StreamLinkSpec,
)
from tandem_b200.registry import Architecture, register_architecture


def mixer_spec(cfg: KamelornConfig, i: int):
    L, m, p = cfg.layers[i], cfg.layers[i].mixer, f"l{i}.mix"
    if L.type == "mamba2":
        return SelectiveRecurrenceSpec(
            "selective_recurrence", prefix=p, hidden_size=cfg.width, num_heads=m.heads, value_dim=m.vdim, state_dim=m.state,
            groups=m.groups, conv_taps=m.conv, norm_groups=m.norm_groups, norm_eps=cfg.norm_eps)
    return LatentAttentionSpec(
        "latent_attention", prefix=p, hidden_size=cfg.width, num_heads=m.heads, head_dim=m.dim, rotary_dim=m.rot_dim,
        rotated_dims=m.rot_dims, rotary_base=m.rot_base, value_dim=m.vdim, latent_dim=m.kv_rank, scale=m.scale,
        norm_eps=cfg.norm_eps, gate="sigmoid")


def feed_forward_spec(cfg: KamelornConfig, i: int):
    mlp, p = cfg.layers[i].mlp, f"l{i}.mlp"
    if mlp.kind == "dense":
        return GatedMLPSpec("gated_mlp", prefix=p, hidden_size=cfg.width, intermediate_size=mlp.ff, activation="silu",
                            names=(("gate", "gate"), ("up", "up"), ("down", "down")), float32_output=True)
    return RoutedMLPSpec("routed_mlp", prefix=p, hidden_size=cfg.width, intermediate_size=mlp.ff, num_experts=mlp.experts,
                         top_k=mlp.top, score="sigmoid", normalize=True, route_scale=mlp.route_scale, activation="silu")


def build_plan(cfg: KamelornConfig) -> ModelPlan:
    streams = cfg.streams or 1
    layers = []
    for i, L in enumerate(cfg.layers):
        def link(q: int) -> StreamLinkSpec:
            return StreamLinkSpec("stream_link", streams=streams, mult=cfg.residual_mult,
                                  prefix=f"l{i}.hc{q}" if cfg.streams is not None else None)

        slots = dict(mixer_norm=NormSpec("rmsnorm", cfg.width, cfg.norm_eps, f"l{i}.norm1"), mixer=mixer_spec(cfg, i),
                     mixer_link=link(1))
        if L.mlp is not None:
            slots.update(feed_forward_norm=NormSpec("rmsnorm", cfg.width, cfg.norm_eps, f"l{i}.norm2"),
                         feed_forward=feed_forward_spec(cfg, i), feed_forward_link=link(2))
        layers.append(LayerSpec.of("connected", **slots))
    return ModelPlan(
        embedding=EmbeddingSpec(cfg.vocab, cfg.width, "embed", scale=cfg.embedding_scale, copies=streams),
        layers=tuple(layers),
        order=tuple(RunStep(i) for i in cfg.run_order()),
        final_norm=NormSpec("rmsnorm", cfg.width, cfg.norm_eps, "final.norm"),
        head=HeadSpec(cfg.vocab, cfg.width, "head"),
        max_position=NO_POSITION_LIMIT,
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


def tensor_shapes(cfg: KamelornConfig) -> dict:
    """Checkpoint tensor name -> shape, in file order."""
    W = cfg.width
    shapes: dict = {"embed": (cfg.vocab, W)}
    for i, L in enumerate(cfg.layers):
        m, p = L.mixer, f"l{i}.mix"
        shapes[f"l{i}.norm1"] = (W,)
        if L.mlp is not None:
            shapes[f"l{i}.norm2"] = (W,)
        if L.type == "mamba2":
            inner, channels = m.heads * m.vdim, m.heads * m.vdim + 2 * m.groups * m.state
            shapes[f"{p}.in"] = (inner + channels + m.heads, W)
            shapes[f"{p}.conv"] = (channels, m.conv)
            shapes[f"{p}.conv.b"] = (channels,)
            for name in ("dt_bias", "A_log", "D"):
                shapes[f"{p}.{name}"] = (m.heads,)
            shapes[f"{p}.norm"] = (inner,)
            shapes[f"{p}.o"] = (W, inner)
        else:
            shapes[f"{p}.q"] = (m.heads * (m.dim + m.rot_dim), W)
            shapes[f"{p}.dkv"] = (m.kv_rank + m.rot_dim, W)
            shapes[f"{p}.dkv.norm"] = (m.kv_rank,)
            shapes[f"{p}.uk"] = (m.heads * m.dim, m.kv_rank)
            shapes[f"{p}.uv"] = (m.heads * m.vdim, m.kv_rank)
            shapes[f"{p}.g"] = (m.heads * m.vdim, W)
            shapes[f"{p}.o"] = (W, m.heads * m.vdim)
        if L.mlp is not None and L.mlp.kind == "dense":
            shapes[f"l{i}.mlp.gate"] = (L.mlp.ff, W)
            shapes[f"l{i}.mlp.up"] = (L.mlp.ff, W)
            shapes[f"l{i}.mlp.down"] = (W, L.mlp.ff)
        elif L.mlp is not None:
            for e in range(L.mlp.experts):
                shapes[f"l{i}.mlp.e{e}.gate"] = (L.mlp.ff, W)
                shapes[f"l{i}.mlp.e{e}.up"] = (L.mlp.ff, W)
                shapes[f"l{i}.mlp.e{e}.down"] = (W, L.mlp.ff)
            shapes[f"l{i}.mlp.router"] = (L.mlp.experts, W)
        if cfg.streams is not None:
            for q in (1, 2) if L.mlp is not None else (1,):
                shapes[f"l{i}.hc{q}.in"] = (cfg.streams,)
                shapes[f"l{i}.hc{q}.out"] = (cfg.streams,)
                shapes[f"l{i}.hc{q}.mix"] = (cfg.streams, cfg.streams)
    shapes["final.norm"] = (W,)
    shapes["head"] = (cfg.vocab, W)
    return shapes


def random_weights(cfg: KamelornConfig, seed: int, device: str = "cpu", dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_spread: float = 0.1) -> Iterator[tuple]:
    """Seeded random tensors by checkpoint name, each from a generator of its own: matrices N(0, std)
    (the embedding N(0, 1 / embedding scale), so the streams start near unit size; the router N(0, 1.5 / sqrt(width)), so that
    scores spread without saturating), norm weights and D 1 + U(-spread, spread), convolution taps N(0, 0.4) with biases N(0, 0.1),
    dt_bias U(-4, -1), A_log U(-1, 1.5), stream reads 1 / streams + N(0, 0.1), stream writes 1 + N(0, 0.2), stream
    mixing the identity + N(0, 0.1)."""
    for index, (name, shape) in enumerate(tensor_shapes(cfg).items()):
        g = torch.Generator(device=device).manual_seed((seed * 1_000_003 + index) % (2**63 - 1))

        def normal(mean: float, sd: float) -> torch.Tensor:
            return torch.empty(shape, device=device, dtype=torch.float32).normal_(mean, sd, generator=g)

        def uniform(lo: float, hi: float) -> torch.Tensor:
            return lo + (hi - lo) * torch.rand(shape, generator=g, device=device, dtype=torch.float32)

        parts = name.split(".")
        leaf = parts[-1]
        if leaf in ("norm1", "norm2", "D") or name == "final.norm" or name.endswith(".mix.norm") or name.endswith("dkv.norm"):
            t = uniform(1.0 - norm_spread, 1.0 + norm_spread)
        elif name.endswith(".conv.b"):
            t = normal(0.0, 0.1)
        elif leaf == "conv":
            t = normal(0.0, 0.4)
        elif leaf == "dt_bias":
            t = uniform(-4.0, -1.0)
        elif leaf == "A_log":
            t = uniform(-1.0, 1.5)
        elif len(parts) == 3 and parts[1].startswith("hc"):
            s = cfg.streams or 1
            t = normal(1.0 / s, 0.1) if leaf == "in" else normal(1.0, 0.2) if leaf == "out" else \
                torch.eye(s, device=device, dtype=torch.float32) + normal(0.0, 0.1)
        elif leaf == "router":
            t = normal(0.0, 1.5 / cfg.width ** 0.5)
        elif name == "embed":
            t = normal(0.0, 1.0 / max(cfg.embedding_scale, 1e-6))
        else:
            t = normal(0.0, std)
        yield name, t.to(dtype)


register_architecture(Architecture("Kamelorn", KamelornConfig, build_plan, random_weights))

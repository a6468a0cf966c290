"""Kamelorn on the CPU: reading config.json, the plan it becomes (parts, links, the looped span in the
running order), what each mixer asks of the cache manager, the checkpoint's tensor names, and the
plain implementation's pieces against closed forms."""

import json
import math

import pytest
import torch

import plain_kamelorn as plain
from tandem_b200.config.kamelorn_config import KamelornConfig
from tandem_b200.config.model_config import ConfigError
from tandem_b200.models.kamelorn import build_plan, random_weights, tensor_shapes
from tandem_b200.registry import part, resolve_architecture

CFG = dict(
    architecture="Kamelorn", vocab=300, width=72, embedding=dict(scale=3.0), norm=dict(eps=1e-4), residual_mult=0.6, streams=2,
    loop=dict(start=1, stop=3, times=3),
    layers=[
        dict(type="latent_attention", mixer=dict(heads=5, dim=12, rot_dim=6, vdim=10, kv_rank=28, scale=0.2, rot=dict(dims=6, base=777.0)),
             mlp=None),
        dict(type="mamba2", mixer=dict(heads=6, vdim=4, state=10, groups=3, conv=4, norm_groups=2), mlp=dict(kind="dense", ff=50)),
        dict(type="mamba2", mixer=dict(heads=2, vdim=16, state=8, groups=1, conv=2, norm_groups=1),
             mlp=dict(kind="moe", expert=dict(ff=20), router=dict(experts=7, top=3, scale=2.0))),
        dict(type="latent_attention", mixer=dict(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, scale=1.0, rot=dict(dims=8, base=1e4)),
             mlp=dict(kind="dense", ff=30)),
    ])


def test_the_registry_finds_the_design_and_the_file_round_trips():
    arch = resolve_architecture(CFG)
    assert arch.name == "Kamelorn"
    cfg = arch.config_class.from_dict(CFG)
    assert cfg.to_dict() == CFG
    assert KamelornConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert cfg.run_order() == [0, 1, 2, 1, 2, 1, 2, 3]


def test_the_plan_names_parts_not_models():
    plan = build_plan(KamelornConfig.from_dict(CFG))
    assert [layer.slot("mixer").kind for layer in plan.layers] == ["latent_attention", "selective_recurrence", "selective_recurrence",
                                                                   "latent_attention"]
    assert [layer.block for layer in plan.layers] == ["connected"] * 4
    assert [name for name, _, _ in plan.layers[0].parts] == ["mixer_norm", "mixer", "mixer_link"]
    assert plan.layers[1].slot("feed_forward").kind == "gated_mlp" and plan.layers[2].slot("feed_forward").kind == "routed_mlp"
    routed = plan.layers[2].slot("feed_forward")
    assert (routed.num_experts, routed.top_k, routed.route_scale, routed.score, routed.normalize) == (7, 3, 2.0, "sigmoid", True)
    link = plan.layers[2].slot("feed_forward_link")
    assert (link.streams, link.mult, link.prefix) == (2, 0.6, "l2.hc2")
    assert [run.layer for run in plan.order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert plan.embedding.scale == 3.0 and plan.embedding.copies == 2 and plan.head.scale == 1.0


def test_without_streams_the_links_are_the_plain_sum():
    cfg = {k: v for k, v in CFG.items() if k not in ("streams", "loop")}
    typed = KamelornConfig.from_dict(cfg)
    plan = build_plan(typed)
    link = plan.layers[0].slot("mixer_link")
    assert (link.streams, link.prefix, link.mult) == (1, None, 0.6) and plan.embedding.copies == 1
    assert part("connection", "stream_link").params(link) == {}
    assert not any(".hc" in name for name in tensor_shapes(typed))
    assert [run.layer for run in plan.order] == [0, 1, 2, 3]


def test_what_the_mixers_ask_of_the_cache_manager():
    plan = build_plan(KamelornConfig.from_dict(CFG))
    latent, mamba = plan.layers[0].slot("mixer"), plan.layers[1].slot("mixer")
    need = part("mixer", latent.kind).kv_need(latent)
    assert (need.num_kv_heads, need.head_dim, need.value_dim, need.window) == (1, 28 + 6, 28, None)
    assert part("mixer", latent.kind).state_need(latent) is None
    assert part("mixer", mamba.kind).kv_need(mamba) is None
    state = part("mixer", mamba.kind).state_need(mamba)
    assert state.shape == (6 * 4 * 10 + 3 * (6 * 4 + 2 * 3 * 10),) and state.dtype == torch.float32


def test_tensor_names_and_shapes():
    cfg = KamelornConfig.from_dict(CFG)
    shapes = tensor_shapes(cfg)
    assert shapes["l1.mix.in"] == (2 * 24 + 2 * 30 + 6, 72) and shapes["l1.mix.conv"] == (24 + 60, 4) and shapes["l1.mix.conv.b"] == (84,)
    assert shapes["l0.mix.q"] == (5 * 18, 72) and shapes["l0.mix.dkv"] == (34, 72) and shapes["l0.mix.uk"] == (60, 28)
    assert shapes["l2.mlp.e6.down"] == (72, 20) and shapes["l2.mlp.router"] == (7, 72) and "l2.mlp.e7.gate" not in shapes
    assert "l0.hc2.in" not in shapes and "l0.norm2" not in shapes and shapes["l3.hc2.mix"] == (2, 2)
    assert {name: tuple(t.shape) for name, t in random_weights(cfg, 1)} == {k: tuple(v) for k, v in shapes.items()}
    plan = build_plan(cfg)
    wanted = set()
    for layer in plan.layers:
        for _, family, spec in layer.parts:
            for ps in part(family, spec.kind).params(spec).values():
                wanted.update(src.name for src in ps.sources)
    assert wanted | {"embed", "final.norm", "head"} == set(shapes)


@pytest.mark.parametrize("bad, match", [
    (dict(layers=[dict(type="attention", mixer={}, mlp=None)]), "attention"),
    (dict(layers=[dict(type="mamba2", mixer=dict(heads=4, vdim=4, state=4, groups=3, conv=2), mlp=None)]), "groups"),
    (dict(layers=[dict(type="mamba2", mixer=dict(heads=3, vdim=5, state=4, conv=2, norm_groups=2), mlp=None)]), "norm_groups"),
    (dict(layers=[dict(type="mamba2", mixer=dict(heads=2, vdim=4, state=4, conv=2), mlp=dict(kind="routed", ff=8))]), "routed"),
    (dict(layers=[dict(type="mamba2", mixer=dict(heads=2, vdim=4, state=4, conv=2),
                       mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=2, top=3)))]), "top"),
    (dict(layers=[dict(type="latent_attention", mixer=dict(heads=2, dim=4, rot_dim=4, vdim=4, kv_rank=8, scale=1.0, rot=dict(dims=6, base=10.0)),
                       mlp=None)]), "rot.dims"),
    (dict(loop=dict(start=2, stop=9, times=2)), "loop"),
    (dict(width=None), "width"),
])
def test_what_the_engine_does_not_have_is_refused(bad, match):
    with pytest.raises(ConfigError, match=match):
        KamelornConfig.from_dict(dict(CFG, **bad))


# ----------------------------------------------------------------------------- the plain implementation's pieces
def test_the_plain_convolution_and_scan_against_closed_forms():
    u = torch.arange(12, dtype=torch.float64).view(6, 2) + 1
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)  # channel 0: the current token; channel 1: two back
    out = plain.causal_conv(u, taps, torch.tensor([0.5, 0.0], dtype=torch.float64))
    assert torch.equal(out[:, 0], u[:, 0] + 0.5)
    assert torch.equal(out[:, 1], torch.cat([torch.zeros(2, dtype=torch.float64), u[:4, 1]]))
    # one head, one state row, constant inputs: S_t is a geometric series
    T, dt, rate = 7, 0.3, math.exp(0.2)
    ones = torch.ones(T, 1, 1, dtype=torch.float64)
    y = plain.selective_scan(2 * ones, ones, ones, torch.full((T, 1), dt, dtype=torch.float64), torch.tensor([0.2], dtype=torch.float64),
                             torch.tensor([0.5], dtype=torch.float64))
    a = math.exp(-rate * dt)
    for t in range(T):
        assert abs(float(y[t, 0, 0]) - (dt * 2 * (1 - a ** (t + 1)) / (1 - a) + 0.5 * 2)) < 1e-12


def test_the_plain_router_and_links():
    w = {"p.router": torch.tensor([[1.0], [3.0], [2.0], [-1.0]], dtype=torch.float64)}
    for e in range(4):
        w[f"p.e{e}.gate"] = torch.full((2, 1), 1.0 + e, dtype=torch.float64)
        w[f"p.e{e}.up"] = torch.ones(2, 1, dtype=torch.float64)
        w[f"p.e{e}.down"] = torch.ones(1, 2, dtype=torch.float64)
    h = torch.tensor([[1.0]], dtype=torch.float64)
    got = plain.routed_ff(h, w, "p", dict(router=dict(experts=4, top=2, scale=1.5)))
    s = torch.sigmoid(torch.tensor([3.0, 2.0], dtype=torch.float64))
    weights = s / s.sum() * 1.5
    each = [2 * (g / (1 + math.exp(-g))) for g in (2.0, 3.0)]  # experts 1 and 2
    assert abs(float(got) - float(weights[0] * each[0] + weights[1] * each[1])) < 1e-12
    X = torch.tensor([[[1.0, 2.0], [10.0, 20.0]]], dtype=torch.float64)  # one token, two streams of width two
    hc = {"h.in": torch.tensor([0.5, 2.0], dtype=torch.float64), "h.out": torch.tensor([1.0, -1.0], dtype=torch.float64),
          "h.mix": torch.tensor([[1.0, 3.0], [0.0, 1.0]], dtype=torch.float64)}
    assert torch.equal(plain.read_streams(X, hc, "h"), torch.tensor([[20.5, 41.0]], dtype=torch.float64))
    new = plain.connect(X, torch.tensor([[1.0, 1.0]], dtype=torch.float64), hc, "h", 0.5)
    assert torch.equal(new, torch.tensor([[[1.5, 2.5], [12.5, 25.5]]], dtype=torch.float64))  # stream 1 <- 3 X_0 + X_1 - 0.5 y

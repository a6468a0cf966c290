"""Fumanex on the CPU: reading config.json, the plan it becomes, sizes that only the checkpoint's
tensors give, the distance buckets, and the cache manager's handling of kept first tokens."""

import json

import pytest

import plain_fumanex as plain
from tandem_b200.cache.manager import CacheManager, KVNeed
from tandem_b200.config.fumanex_config import FumanexConfig
from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import DistanceBiasSpec
from tandem_b200.models.fumanex import build_plan, tensor_shapes
from tandem_b200.registry import resolve_architecture

CFG = dict(
    architecture="Fumanex", vocab=300, width=72, embedding=dict(scale=3.0), logit_scale=0.5, norm=dict(eps=1e-4),
    layers=[
        dict(type="retention", mixer=dict(heads=3, dim=12, vdim=20, decay=[0.9, 0.95, 0.99], rot=dict(dims=6, base=777.0)), mlp=None),
        dict(type="attention", mixer=dict(heads=6, kv_heads=3, dim=12, vdim=10, scale=0.2, softcap=9.0, bias_max=77, v_mix=True,
                                          mask=dict(size=19, keep_first=2)), mlp=dict(kind="dense", ff=50)),
        dict(type="lightning", mixer=dict(heads=2, dim=6, vdim=8, decay=[0.5, 0.75]), mlp=dict(kind="dense", ff=30)),
        dict(type="attention", mixer=dict(heads=3, kv_heads=3, dim=8, vdim=10, scale=1.0, bias_max=30, v_mix=True), mlp=None),
    ])


def test_the_registry_finds_the_design_and_the_file_round_trips():
    arch = resolve_architecture(CFG)
    assert arch.name == "Fumanex"
    cfg = arch.config_class.from_dict(CFG)
    assert FumanexConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert cfg.layers[1].mixer.window == 19 and cfg.layers[3].mixer.window is None and cfg.layers[3].mixer.softcap is None


def test_the_plan_names_parts_not_models():
    plan = build_plan(FumanexConfig.from_dict(CFG))
    kinds = [layer.slot("mixer").kind for layer in plan.layers]
    assert kinds == ["decay_recurrence", "sink_attention", "decay_recurrence", "sink_attention"]
    assert [layer.block for layer in plan.layers] == ["parallel"] * 4
    ret, att, lig, att2 = (layer.slot("mixer") for layer in plan.layers)
    assert (ret.rotary_dim, ret.key_scale, ret.output_norm, ret.gate, ret.activation) == (6, 12 ** -0.5, "per_head", "silu", "none")
    assert (lig.rotary_dim, lig.key_scale, lig.output_norm, lig.gate, lig.activation) == (0, 1.0, "all_heads", "sigmoid", "silu")
    assert att.value_mix_first and not att2.value_mix_first and att2.window is None and att2.keep_first == 0
    assert [name for name, _, _ in plan.layers[0].parts] == ["norm", "mixer"]
    assert plan.embedding.scale == 3.0 and plan.head.scale == 0.5


def test_table_rows_come_from_the_tensor():
    cfg = FumanexConfig.from_dict(CFG)
    shapes = dict(tensor_shapes(cfg))
    shapes["l1.mix.rel"] = (14, 6)
    done = cfg.with_checkpoint_shapes(shapes)
    assert done.layers[1].mixer.bias_buckets == 14 and done.layers[3].mixer.bias_buckets == cfg.layers[3].mixer.bias_buckets
    assert build_plan(done).layers[1].slot("mixer").distance_bias == DistanceBiasSpec(14, 77)


@pytest.mark.parametrize("bad, match", [
    (dict(layers=[dict(type="mamba", mixer={}, mlp=None)]), "mamba"),
    (dict(layers=[dict(type="lightning", mixer=dict(heads=2, dim=4, vdim=4, decay=[0.5]), mlp=None)]), "decay"),
    (dict(layers=[dict(type="lightning", mixer=dict(heads=1, dim=4, vdim=4, decay=[0.5]), mlp=dict(kind="routed", ff=8))]), "routed"),
    (dict(layers=[dict(type="attention", mixer=dict(heads=5, kv_heads=2, dim=4, vdim=4, scale=1.0, bias_max=9), mlp=None)]), "multiple"),
    (dict(width=None), "width"),
])
def test_what_the_engine_does_not_have_is_refused(bad, match):
    with pytest.raises(ConfigError, match=match):
        FumanexConfig.from_dict(dict(CFG, **bad))


@pytest.mark.parametrize("rows, far", [(32, 120), (16, 64), (10, 50), (4, 9), (7, 300)])
def test_buckets(rows, far):
    spec = DistanceBiasSpec(rows, far)
    got = [spec.bucket(n) for n in range(2 * far)]
    assert got == [plain.distance_bucket(n, rows, far) for n in range(2 * far)]
    assert got[: rows // 2] == list(range(rows // 2)) and got[far] == rows - 1 and len(set(got[far:])) == 1
    assert all(a <= b for a, b in zip(got, got[1:]))


def test_pages_of_kept_first_tokens_are_not_given_back():
    m = CacheManager([KVNeed(2, 16, window=10, value_dim=8, keep_first=5), KVNeed(2, 16, window=10), KVNeed(2, 16, None)],
                     page_size=4, num_pages=40, max_requests=2)
    assert len(m.groups) == 3
    m.begin("a")
    assert m.grow("a", 64)
    m.commit("a", 64)
    assert m.grow("a", 65)  # the next query stands at 64: keys 55 .. 64 and, in the first group, 0 .. 4
    kept, plain_window, everything = (m.table(g, "a") for g in range(3))
    assert [p >= 0 for p in kept[:4]] == [True, True, False, False]  # tokens 0 .. 4 live in pages 0 and 1
    assert all(p < 0 for p in kept[2:13]) and all(p >= 0 for p in kept[13:])
    assert all(p < 0 for p in plain_window[:13]) and all(p >= 0 for p in everything)
    assert m.pages_to_grow("a", 66) == [0, 0, 0]
    m.check()
    m.end("a")
    assert m.all_free()

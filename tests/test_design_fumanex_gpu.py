"""Fumanex in the engine against the plain implementation (``plain_fumanex``): each mixer alone,
whole prompts against decoding and against portions, mixed batches on small pools, window and
kept-token edges made visible by the weights, long decoding, other sizes, greedy generation
through ``LLMEngine``.  Every test builds its own tiny model with random weights."""

import json
import math
import os
import random

import numpy as np
import pytest
import torch

import plain_fumanex as plain
import replay_cases as rc

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- tiny models
def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=12, keep_first=3, v_mix=True, softcap=20.0, bias_max=40,
                    scale=0.3, ff=40):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, bias_max=bias_max, v_mix=v_mix)
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = dict(size=window, keep_first=keep_first)
    return dict(type="attention", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def retention_layer(heads=2, dim=16, vdim=8, rot_dims=8, base=500.0, decay=None, ff=40):
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=decay or [1.0 - 2.0 ** -(3 + i) for i in range(heads)])
    if rot_dims:
        m["rot"] = dict(dims=rot_dims, base=base)
    return dict(type="retention", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def lightning_layer(heads=3, dim=8, vdim=16, decay=None, ff=40):
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=decay or [math.exp(-0.5 / (i + 1)) for i in range(heads)])
    return dict(type="lightning", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def model_config(layers, width=48, vocab=211, embedding_scale=6.0, logit_scale=0.5, eps=1e-5):
    return dict(architecture="Fumanex", vocab=vocab, width=width, embedding=dict(scale=embedding_scale), logit_scale=logit_scale,
                norm=dict(eps=eps), layers=layers)


# the first two attention layers have sizes that the tensor-core kernel takes (bfloat16, steps with portions), the third has not
HYBRID = model_config([attention_layer(vdim=32), lightning_layer(), attention_layer(vdim=32, window=70, keep_first=1), retention_layer(),
                       attention_layer(dim=8, vdim=24, v_mix=False), lightning_layer(ff=None)])


def make_folder(tmp_path, cfg, seed=3, edits=None, buckets=None, name="m") -> str:
    """A model folder with bfloat16-representable random weights; ``edits``: tensor name -> function
    that changes the float32 tensor in place; ``buckets``: rows of the distance-bias tables."""
    from safetensors.torch import save_file

    from tandem_b200.config.fumanex_config import FumanexConfig
    from tandem_b200.models.fumanex import random_weights

    cfg = json.loads(json.dumps(cfg))
    if buckets is not None:
        for layer in cfg["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["bias_buckets"] = buckets
    typed = FumanexConfig.from_dict(cfg)
    tensors = {}
    for tensor_name, t in random_weights(typed, seed, "cpu", torch.float32, std=0.08):
        if edits and tensor_name in edits:
            edits[tensor_name](t)
        tensors[tensor_name] = t.to(torch.bfloat16).contiguous()
    folder = os.path.join(str(tmp_path), name)
    os.makedirs(folder, exist_ok=True)
    for layer in cfg["layers"]:  # the file a user is given names no table size: the tensor's shape does
        layer["mixer"].pop("bias_buckets", None)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


def tokens(seed, n, vocab):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_steps(folder, dtype, steps, page_size=4, pool_tokens=None, max_requests=4, log=None):
    """The steps through the engine's step function; request id -> [positions, vocab] float64."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.kernels import ops

    decoder, _ = load_model(folder, dtype, "cuda:0")
    need = pool_tokens if pool_tokens is not None else rc.tokens_needed(steps, round_to=max(16, page_size))
    ex = build_executor(decoder, page_size=page_size, num_pages=-(-need // page_size), max_requests=max_requests)
    if log is not None:
        log.append(rc.PageLog(ex.manager))
    out = {}
    for st in steps:
        logits = ex.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]], end=st["end"])
        if logits.shape[0]:
            out[st["step"]] = logits.cpu().double().numpy()
        ex.manager.check()
    ops.check_status(ex.device)
    assert ex.manager.all_free()
    return {rid: torch.from_numpy(np.stack(rows)) for rid, rows in rc.collect(steps, out).items()}


def distance(got, ref):
    """Largest error of a position: root mean square over the vocabulary of the difference (mean
    taken off), over the root mean square of the reference's logits."""
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / r.pow(2).mean().sqrt()).max())


LIMIT = {"float32": 2e-5, "bfloat16": 4e-2}


def reference(folder, requests):
    cfg, w = plain.read_folder(folder)
    return {rid: plain.forward(cfg, w, t) for rid, t in requests.items()}


# ----------------------------------------------------------------------------- each mechanism alone
ALONE = {
    "attention": [attention_layer(v_mix=False)],
    "attention_mixing": [attention_layer(ff=None), attention_layer(window=5, keep_first=0)],
    "attention_tensor_cores": [attention_layer(heads=6, kv_heads=2, dim=32, vdim=16, window=9, keep_first=2, v_mix=False)],
    "attention_tensor_cores_full": [attention_layer(heads=2, kv_heads=2, dim=64, vdim=64, window=None, v_mix=False, softcap=None)],
    "attention_full": [attention_layer(window=None, softcap=None, kv_heads=4, dim=24, vdim=24, v_mix=False)],
    "retention": [retention_layer()],
    "retention_whole_head_rotates": [retention_layer(dim=8, rot_dims=8, vdim=40)],
    "retention_no_rotation": [retention_layer(rot_dims=0, ff=None)],
    "lightning": [lightning_layer()],
    "lightning_wide": [lightning_layer(heads=1, dim=40, vdim=72, decay=[0.97])],
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mixer_alone(tmp_path, name, dtype):
    folder = make_folder(tmp_path, model_config(ALONE[name]))
    requests = {"a": tokens(1, 45, 211), "b": tokens(2, 1, 211)}
    ref = reference(folder, requests)
    got = run_steps(folder, dtype, rc.whole(requests))
    for rid in requests:
        assert distance(got[rid], ref[rid]) < LIMIT[dtype], (name, rid)


def test_the_stream_after_every_layer_is_the_plain_one(tmp_path):
    """The float32 residual stream, layer by layer (read behind each layer's arrangement)."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry

    folder = make_folder(tmp_path, HYBRID)
    toks = tokens(5, 30, 211)
    cfg, w = plain.read_folder(folder)
    _, layers = plain.forward(cfg, w, toks, return_layers=True)
    decoder, _ = load_model(folder, "float32", "cuda:0")
    ex = build_executor(decoder, page_size=8, num_pages=8, max_requests=2)
    seen = []
    for layer in decoder.layers:
        inner = layer.block.forward

        def spy(l, x, residual, ctx, inner=inner):
            out = inner(l, x, residual, ctx)
            assert out is None  # everything is in the stream
            seen.append(residual.detach().cpu().double().clone())
            return out

        layer.block.forward = spy
    ex.step([StepEntry("a", toks, [0])], end=["a"])
    assert len(seen) == len(layers)
    for i, (g, r) in enumerate(zip(seen, layers)):
        assert (g - r).abs().max() < 2e-4 * max(1.0, float(r.abs().max())), i


# ----------------------------------------------------------------------------- schedules
@pytest.fixture(scope="module")
def hybrid(tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("hybrid"), HYBRID)
    requests = {"a": tokens(11, 97, 211), "b": tokens(12, 33, 211), "c": tokens(13, 64, 211), "d": tokens(14, 2, 211),
                "e": tokens(15, 50, 211), "f": tokens(16, 1, 211)}
    return folder, requests, reference(folder, requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [1, 4, 16])
def test_prefill_against_token_by_token_decoding(hybrid, dtype, page_size):
    folder, requests, ref = hybrid
    whole = run_steps(folder, dtype, rc.whole(requests), page_size)
    tail = run_steps(folder, dtype, rc.tail_one_by_one(requests, tail=40), page_size)
    for rid in requests:
        assert distance(whole[rid], ref[rid]) < LIMIT[dtype], rid
        assert distance(tail[rid], ref[rid]) < LIMIT[dtype], rid
        if dtype == "float32":  # every kernel sums in an order that does not depend on the cut
            assert torch.equal(whole[rid], tail[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(hybrid, dtype):
    folder, requests, ref = hybrid
    whole = run_steps(folder, dtype, rc.whole(requests), 4) if dtype == "float32" else None
    for sizes in ((2,), (3, 2, 7, 2, 19, 2), (16, 2, 5)):
        got = run_steps(folder, dtype, rc.changing_portions(requests, sizes=sizes), 4)
        for rid in requests:
            assert distance(got[rid], ref[rid]) < LIMIT[dtype], (sizes, rid)
            if whole is not None:
                assert torch.equal(got[rid], whole[rid]), (sizes, rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_on_a_small_pool(hybrid, dtype):
    """Up to three live requests, portions beside single tokens; the pool holds only what is live, the state
    tensor has three rows: pages and slots go to new holders while other requests are being read."""
    folder, requests, ref = hybrid
    steps = rc.mixed(requests, live=3, portion=9, decode_after=0.5)
    log = []
    got = run_steps(folder, dtype, steps, page_size=4, pool_tokens=rc.tokens_needed(steps, round_to=4), max_requests=3, log=log)
    assert log[0].pages_reused > 0 and log[0].reused_beside_live > 0
    alone = run_steps(folder, dtype, rc.whole(requests), 4) if dtype == "float32" else None
    for rid in requests:
        assert distance(got[rid], ref[rid]) < LIMIT[dtype], rid
        if alone is not None:
            assert torch.equal(got[rid], alone[rid]), rid


def test_a_state_slot_that_is_used_again_starts_from_zero(tmp_path):
    folder = make_folder(tmp_path, model_config([lightning_layer(), retention_layer()]))
    requests = {"first": tokens(1, 40, 211), "second": tokens(2, 25, 211)}
    ref = reference(folder, requests)
    got = run_steps(folder, "float32", rc.tail_one_by_one(requests, tail=5), page_size=8, max_requests=1)
    for rid in requests:
        assert distance(got[rid], ref[rid]) < LIMIT["float32"], rid


def test_long_decoding(tmp_path):
    """Three hundred tokens one by one: the window passes over decoded tokens page after page, the kept first
    tokens stay, the states are carried."""
    cfg = model_config([attention_layer(window=21, keep_first=5), retention_layer(decay=[0.9995, 0.9]), lightning_layer()])
    folder = make_folder(tmp_path, cfg)
    requests = {"a": tokens(21, 330, 211)}
    ref = reference(folder, requests)
    for dtype in ("float32", "bfloat16"):
        got = run_steps(folder, dtype, rc.tail_one_by_one(requests, tail=300), page_size=8, pool_tokens=21 + 5 + 3 * 8 + 16)
        assert distance(got["a"], ref["a"]) < LIMIT[dtype], dtype


# ----------------------------------------------------------------------------- edges made visible
def loud_rows(rows):
    def edit(t):
        t.mul_(0.1)
        for r in rows:
            t[r] += 12.0
    return edit


@pytest.mark.parametrize("regime", ["whole", "tail", "portions"])
def test_the_last_key_inside_the_window_and_the_kept_tokens_stand_out(tmp_path, regime):
    """The distance bias is made loud at the window's last distance and in the last row (far keys): a
    window one key short, or kept tokens that are dropped, change the result by much.  The window (10) and
    the kept tokens (3) straddle the pages of 4."""
    window, keep, rows, far = 10, 3, 12, 30
    layer = attention_layer(window=window, keep_first=keep, bias_max=far, v_mix=False, ff=None)
    inside = plain.distance_bucket(window - 1, rows, far)
    folder = make_folder(tmp_path, model_config([layer]), buckets=rows,
                         edits={"l0.mix.rel": loud_rows([inside, rows - 1]), "l0.mix.sink": lambda t: t.fill_(-3.0)})
    requests = {"a": tokens(31, 70, 211), "b": tokens(32, 41, 211)}
    ref = reference(folder, requests)
    steps = {"whole": rc.whole, "tail": lambda r: rc.tail_one_by_one(r, 35), "portions": lambda r: rc.changing_portions(r, (3, 2, 5))}[regime](requests)
    for dtype in ("float32", "bfloat16"):
        got = run_steps(folder, dtype, steps, page_size=4)
        for rid in requests:
            assert distance(got[rid], ref[rid]) < LIMIT[dtype], (dtype, rid)
    # the oracle itself tells the neighbours apart: one key more or less in the window is another model
    cfg, w = plain.read_folder(folder)
    for other in (dict(size=window - 1, keep_first=keep), dict(size=window + 1, keep_first=keep), dict(size=window, keep_first=keep - 1),
                  dict(size=window, keep_first=keep + 1)):
        changed = json.loads(json.dumps(cfg))
        changed["layers"][0]["mixer"]["mask"] = other
        assert distance(plain.forward(changed, w, requests["a"]), ref["a"]) > 0.05, other


def test_a_loud_sink_silences_the_values(tmp_path):
    layer = attention_layer(v_mix=False, ff=None)
    quiet = make_folder(tmp_path, model_config([layer]), name="quiet")
    loud = make_folder(tmp_path, model_config([layer]), name="loud", edits={"l0.mix.sink": lambda t: t.fill_(25.0)})
    requests = {"a": tokens(41, 30, 211)}
    for folder in (quiet, loud):
        ref = reference(folder, requests)
        got = run_steps(folder, "float32", rc.tail_one_by_one(requests, 8), page_size=4)
        assert distance(got["a"], ref["a"]) < LIMIT["float32"]
    assert distance(reference(loud, requests)["a"], reference(quiet, requests)["a"]) > 0.05


class FakeContext:
    def __init__(self, positions, seq_of_token):
        self.positions, self.seq_of_token = positions, seq_of_token


def attend_one_sequence(q, k, v, page_size, cuts, dtype, tiles=False, **options):
    """The attention kernels alone: one sequence written to a paged cache (pages in scrambled order)
    portion by portion, every portion attending through the cache.  q [T, H, dk], k [T, G, dk], v [T, G, dv]."""
    from tandem_b200.kernels import sink_attention as kernels
    from tandem_b200.parts.base import KVView

    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    pages = -(-T // page_size)
    order = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(0))[:pages].to(torch.int32)
    kc = torch.zeros((pages + 3, G, page_size, dk), dtype=dtype, device="cuda")
    vc = torch.zeros((pages + 3, G, page_size, dv), dtype=dtype, device="cuda")
    table = order.view(1, -1).cuda()
    out, at = [], 0
    for n in cuts:
        pos = torch.arange(at, at + n, dtype=torch.int32)
        slots = (order[(pos // page_size).long()] * page_size + pos % page_size).to(torch.int32).cuda()
        qkv = torch.cat([q[at: at + n].reshape(n, -1), k[at: at + n].reshape(n, -1), v[at: at + n].reshape(n, -1)], -1).float().cuda().contiguous()
        view = KVView(kc, vc, table, slots, page_size, True)
        kernels.prepare(qkv, None, None, None, view, H, G, dk, dv, False, 0.0)
        ctx = FakeContext(pos.cuda(), torch.zeros(n, dtype=torch.int32, device="cuda"))
        rest = (options.get("window"), options.get("keep_first", 0), options.get("scale", 1.0), options.get("softcap"),
                options.get("bias"), options.get("sink"))
        if tiles and n == 1 and kernels.split_applies(dtype, dk, dv, H // G, qkv.shape[1]):  # single tokens: the split kernel
            out.append(kernels.attend_split(qkv, view, ctx, H, G, dk, dv, *rest).float().cpu())
        elif tiles:
            assert kernels.tiles_apply(dtype, dk, dv, H // G, qkv.shape[1])
            plan = torch.tensor(kernels.plan_tiles([at], [n], H // G), dtype=torch.int32, device="cuda")
            out.append(kernels.attend_tiles(qkv, view, plan, H, G, dk, dv, *rest).float().cpu())
        else:
            out.append(kernels.attend(qkv, view, ctx, H, G, dk, dv, *rest).float().cpu())
        at += n
    return torch.cat(out).view(T, H, dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv", [(64, 64), (16, 128), (40, 24)])
def test_one_far_key_among_hundreds(dtype, dk, dv):
    """No window: the query of the last tokens points at one key 600 back; kept tokens beyond a window likewise."""
    g = torch.Generator().manual_seed(7)
    T, H, G = 700, 4, 2
    q, k, v = (torch.randn(T, n, d, generator=g).to(dtype).double() for n, d in ((H, dk), (G, dk), (G, dv)))
    k[83] = 0.0
    k[83, :, 0] = 6.0
    k[2, :, 1] = 6.0
    q[650:, :, 0] = 6.0  # looks for key 83
    q[400:420, :, 1] = 6.0  # looks for key 2, a kept one
    for options in (dict(), dict(window=64, keep_first=3), dict(window=64, keep_first=2), dict(window=617, keep_first=0)):
        ref = plain.sink_softmax_attention(q, k, v, 0.5, None, None, 0, options.get("window"), options.get("keep_first", 0), None)
        for cuts in ([T], [512, 100] + [1] * 88, [37] * 18 + [34]):
            got = attend_one_sequence(q, k, v, 16, cuts, dtype, scale=0.5, **options).double()
            assert (got - ref).abs().max() < (1e-4 if dtype == torch.float32 else 3e-2), (options, cuts[:3])
            if dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0:
                got = attend_one_sequence(q, k, v, 16, cuts, dtype, tiles=True, scale=0.5, **options).double()
                assert (got - ref).abs().max() < 3e-2, ("tensor cores", options, cuts[:3])
    seen = plain.sink_softmax_attention(q, k, v, 0.5, None, None, 0, None, 0, None)
    hidden = plain.sink_softmax_attention(q, k, v, 0.5, None, None, 0, 64, 2, None)
    assert (seen[690] - hidden[690]).abs().max() > 0.1 and (seen[410] - hidden[410]).abs().max() > 0.1


def test_cap_bias_and_sink_in_the_kernel():
    g = torch.Generator().manual_seed(9)
    T, H, G, dk, dv = 90, 6, 3, 32, 16
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=torch.float64) for n, d in ((H, dk), (G, dk), (G, dv)))
    q *= 3.0  # scores far beyond the cap
    rel = torch.randn(10, H, generator=g, dtype=torch.float64) * 2
    sink = torch.randn(H, generator=g, dtype=torch.float64) * 3
    by_distance = rel[torch.tensor([plain.distance_bucket(n, 10, 50) for n in range(51)])].float().cuda().contiguous()
    ref = plain.sink_softmax_attention(q, k, v, 0.4, 5.0, rel, 50, 33, 4, sink)
    got = attend_one_sequence(q, k, v, 8, [50, 2, 1, 1, 36], torch.float32, scale=0.4, softcap=5.0, window=33, keep_first=4,
                              bias=by_distance, sink=sink.float().cuda()).double()
    assert (got - ref).abs().max() < 1e-4
    uncapped = plain.sink_softmax_attention(q, k, v, 0.4, None, rel, 50, 33, 4, sink)
    assert (uncapped - ref).abs().max() > 0.05
    for page_size, cuts in ((8, [50, 2, 1, 1, 36]), (1, [90]), (32, [3] * 30)):  # the same on the tensor cores, from bfloat16 inputs
        qb, kb, vb = (t.to(torch.bfloat16).double() for t in (q, k, v))
        ref16 = plain.sink_softmax_attention(qb, kb, vb, 0.4, 5.0, rel, 50, 33, 4, sink)
        got = attend_one_sequence(qb, kb, vb, page_size, cuts, torch.bfloat16, tiles=True, scale=0.4, softcap=5.0, window=33, keep_first=4,
                                  bias=by_distance, sink=sink.float().cuda()).double()
        assert (got - ref16).abs().max() < 3e-2, (page_size, cuts[:2])


@pytest.mark.parametrize("dk,dv,H", [(32, 64, 4), (20, 8, 3), (96, 33, 1), (128, 128, 2), (544, 16, 1), (6, 70, 2)])
def test_the_recurrence_kernel_alone(dk, dv, H):
    """Two requests of unequal length in one launch, then their continuation from the stored state; a third
    request takes over a row of the state tensor that was in use."""
    from tandem_b200.kernels import recurrence as kernels

    g = torch.Generator().manual_seed(dk)
    lens = [37, 5]
    decay = [1.0 - 0.3 / (i + 1) for i in range(H)]
    state = torch.randn(4, H, dk, dv, generator=g).cuda()  # rows hold leftovers: the engine zeroes a row at admission
    state[1].zero_()
    state[3].zero_()
    cols = 2 * H * dk + H * dv
    seqs = [torch.randn(n, cols + 5, generator=g) * 0.5 for n in lens]
    refs = [plain.decay_recurrence(s[:, : H * dk].double().view(-1, H, dk), s[:, H * dk: 2 * H * dk].double().view(-1, H, dk),
                                   s[:, 2 * H * dk: cols].double().view(-1, H, dv), decay) for s in seqs]
    slots = torch.tensor([3, 1], dtype=torch.int32).cuda()
    dec = torch.tensor(decay, dtype=torch.float32).cuda()
    outs, at = [[], []], [0, 0]
    for cut in ((20, 3), (1, 1), (16, 1)):
        proj = torch.cat([seqs[i][at[i]: at[i] + cut[i]] for i in range(2)]).cuda().contiguous()
        at = [at[i] + cut[i] for i in range(2)]
        cu = torch.tensor([0, cut[0], cut[0] + cut[1]], dtype=torch.int32).cuda()
        o = kernels.scan(proj, cu, slots, 2, state, dec, H, dk, dv).cpu().double().view(-1, H, dv)
        outs[0].append(o[: cut[0]])
        outs[1].append(o[cut[0]:])
    for got, ref in zip(outs, refs):
        assert (torch.cat(got) - ref).abs().max() < 1e-4 * max(1.0, float(ref.abs().max()))


# ----------------------------------------------------------------------------- other sizes
def random_model(rng: random.Random) -> dict:
    width = rng.choice([24, 40, 56, 66, 100])
    layers = []
    for _ in range(rng.randint(1, 5)):
        kind = rng.choice(["attention", "attention", "retention", "lightning"])
        ff = rng.choice([None, 2 * rng.randint(5, 40), 8 * rng.randint(2, 12)])
        if kind == "attention":
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 64])
            layers.append(attention_layer(heads=kv * rng.choice([1, 2, 4]), kv_heads=kv, dim=dim, vdim=rng.choice([8, 16, 40, 64]),
                                          window=rng.choice([None, 1, 2, 7, 16, 33]), keep_first=rng.choice([0, 1, 4, 9]),
                                          v_mix=rng.random() < 0.6, softcap=rng.choice([None, 3.0, 50.0]),
                                          bias_max=rng.choice([20, 64, 300]), scale=rng.choice([dim ** -0.5 * 4, 0.5, 1.0]), ff=ff))
        elif kind == "retention":
            dim = rng.choice([4, 8, 16, 34, 64])
            layers.append(retention_layer(heads=rng.randint(1, 4), dim=dim, vdim=rng.choice([4, 8, 33, 64]),
                                          rot_dims=rng.choice([0, 2, dim // 2 * 2, dim // 4 * 2]), base=rng.choice([50.0, 1e4, 1e6]), ff=ff))
        else:
            layers.append(lightning_layer(heads=rng.randint(1, 4), dim=rng.choice([4, 8, 16, 36]), vdim=rng.choice([8, 16, 30, 64]), ff=ff))
    mixing = [l["mixer"] for l in layers if l["type"] == "attention" and l["mixer"]["v_mix"]]
    for m in mixing[1:]:  # layers that mix one another's values agree in their shape
        m["kv_heads"], m["vdim"] = mixing[0]["kv_heads"], mixing[0]["vdim"]
        m["heads"] = m["kv_heads"] * max(1, m["heads"] // m["kv_heads"])
    return model_config(layers, width=width, vocab=rng.randint(50, 400), embedding_scale=rng.choice([1.0, 7.5]),
                        logit_scale=rng.choice([1.0, 0.125]), eps=rng.choice([1e-6, 1e-5, 1e-3]))


@pytest.mark.parametrize("seed", range(12))
def test_random_models_and_schedules(tmp_path, seed):
    rng = random.Random(100 + seed)
    cfg = random_model(rng)
    folder = make_folder(tmp_path, cfg, seed=seed, buckets=rng.choice([4, 10, 16, 32]))
    requests = {f"r{i}": tokens(seed * 10 + i, rng.randint(1, 90), cfg["vocab"]) for i in range(rng.randint(2, 5))}
    ref = reference(folder, requests)
    page_size = rng.choice([1, 2, 8, 16, 32])
    regime = rng.choice(["mixed", "portions", "tail"])
    steps = {"mixed": lambda: rc.mixed(requests, live=rng.randint(2, 4), portion=rng.randint(2, 20), decode_after=rng.choice([0.4, 0.8])),
             "portions": lambda: rc.changing_portions(requests, sizes=tuple(rng.randint(2, 17) for _ in range(7))),
             "tail": lambda: rc.tail_one_by_one(requests, tail=rng.randint(1, 30))}[regime]()
    for dtype in ("float32", "bfloat16"):
        got = run_steps(folder, dtype, steps, page_size, pool_tokens=rc.tokens_needed(steps, round_to=max(page_size, 4)))
        for rid in requests:
            assert distance(got[rid], ref[rid]) < LIMIT[dtype], (cfg, page_size, regime, dtype, rid)


# ----------------------------------------------------------------------------- through the engine's entry point
@pytest.mark.parametrize("options", [dict(), dict(cuda_graph=False, overlap_schedule=False), dict(max_num_batched_tokens=16, max_num_seqs=2)])
def test_greedy_generation_through_the_engine(tmp_path, options):
    from tandem_b200.engine.llm_engine import LLM
    from tandem_b200.sampling.params import SamplingParams

    folder = make_folder(tmp_path, HYBRID)
    prompts = [tokens(51, 23, 211), tokens(52, 5, 211), tokens(53, 40, 211)]
    cfg, w = plain.read_folder(folder)
    llm = LLM(folder, dtype="float32", block_size=4, num_kv_blocks=64, **options)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        seq = list(prompt)
        for produced in out.output_token_ids:
            logits = plain.forward(cfg, w, seq)[-1]
            best = int(logits.argmax())
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) > 1e-3:  # a tie within rounding may go either way
                assert produced == best, (len(seq) - len(prompt))
            seq.append(produced)
        assert len(out.output_token_ids) == 12
    assert llm.engine.cache.all_free()

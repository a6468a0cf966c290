"""A plain, slow implementation of the Fumanex design in PyTorch on the CPU (float64 by default),
written from the design's equations: one function per mechanism, whole sequences at once, no
cache, no batching, no kernels.  It shares no code with ``tandem_b200``; the tests compare the
engine with it.

Notation: x [T, W] the residual stream of one sequence, positions 0 .. T-1; a weight ``w[name]``
is stored [out, in] and applied as x @ w.T.
"""

from __future__ import annotations

import json
import math
import os

import torch


def read_folder(folder: str, dtype=torch.float64):
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for name in f.keys():
            w[name] = f.get_tensor(name).to(dtype)
    return cfg, w


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the distance-bias table for distance n: one row per distance below rows // 2, then
    rows spaced evenly in log(distance) up to ``far``; the last row takes the rest."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def visible(T: int, window, keep_first: int):
    """[T, T] bool: query i sees key j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen &= (i - j < window) | (j < keep_first)
    return seen


def rotate_half(x, positions, dims: int, base: float):
    """x [T, heads, dim]: dim i of the first ``dims`` is paired with i + dims / 2; the pair (u, v) at
    position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2 i / dims)."""
    if not dims:
        return x
    half = dims // 2
    f = float(base) ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :].to(x.dtype), a.sin()[:, None, :].to(x.dtype)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- mechanisms
def sink_softmax_attention(q, k, v, scale, softcap, rel, far, window, keep_first, sink):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv].  score = cap(scale q.k) + rel[bucket];
    the softmax denominator also holds exp(sink_h).  ``rel`` [rows, H] or None, ``sink`` [H] or None."""
    T, H, _ = q.shape
    G = k.shape[1]
    seen = visible(T, window, keep_first)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    if rel is not None:
        dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0)
        rows = torch.tensor([distance_bucket(n, rel.shape[0], far) for n in range(T)])[dist]
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        if rel is not None:
            s = s + rel[:, h][rows]
        s = s.masked_fill(~seen, -math.inf)
        top = s.max(-1).values
        if sink is not None:
            top = torch.maximum(top, sink[h])
        e = torch.exp(s - top[:, None])
        denominator = e.sum(-1)
        if sink is not None:
            denominator = denominator + torch.exp(sink[h] - top)
        out[:, h] = (e / denominator[:, None]) @ v[:, g]
    return out


def decay_recurrence(q, k, v, decay):
    """q, k [T, H, dk], v [T, H, dv]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=q.dtype)
    d = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    o = []
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        o.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(o)


def attention_mixer(w, p, m, h, eps, shared):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    if m.get("v_mix"):
        if "first_values" in shared:
            share = w[p + "vmix"]
            v = (1.0 - share) * v + share * shared["first_values"]
        else:
            shared["first_values"] = v
    mask = m.get("mask") or {}
    o = sink_softmax_attention(q, k, v, m["scale"], m.get("softcap"), w[p + "rel"], m["bias_max"], mask.get("size"),
                               mask.get("keep_first", 0), w[p + "sink"])
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def retention_mixer(w, p, m, h, eps, shared):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    rot = m.get("rot") or {}
    positions = torch.arange(T)
    q = rotate_half(q, positions, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_half(k, positions, rot.get("dims", 0), rot.get("base", 1.0)) * dk ** -0.5
    o = unit_rms(decay_recurrence(q, k, v, m["decay"]), eps).reshape(T, H * dv)
    return (o * torch.nn.functional.silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def lightning_mixer(w, p, m, h, eps, shared):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w[p + "q"].T).view(T, H, dk)
    k = silu(h @ w[p + "k"].T).view(T, H, dk)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    o = decay_recurrence(q, k, v, m["decay"]).reshape(T, H * dv)
    o = unit_rms(o, eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_feed_forward(w, p, h):
    return gelu_tanh(h @ w[p + "up"].T + w[p + "up.b"]) @ w[p + "down"].T + w[p + "down.b"]


MIXERS = {"attention": attention_mixer, "retention": retention_mixer, "lightning": lightning_mixer}


def forward(cfg: dict, w: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    shared, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        h = unit_rms(x, eps) * w[f"l{i}.norm1"]
        y = MIXERS[layer["type"]](w, f"l{i}.mix.", layer["mixer"], h, eps, shared)
        if layer.get("mlp"):
            y = y + dense_feed_forward(w, f"l{i}.mlp.", h)
        x = x + y
        after.append(x)
    logits = (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(after)) if return_layers else logits

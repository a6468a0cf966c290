"""A plain, slow implementation of the Kamelorn design in PyTorch on the CPU (float64 by default),
written from the design's equations: one function per mechanism, whole sequences at once, no
cache, no batching, no kernels.  It shares no code with ``tandem_b200``; the tests compare the
engine with it.

Notation: a sequence has T tokens at positions 0 .. T-1; X [T, s, W] are the s residual streams
(s = 1 without hyper-connections); a weight ``w[name]`` is stored [out, in] and applied as x @ w.T.
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


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


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
def causal_conv(u, taps, bias):
    """u [T, C], taps [C, K] (column K-1 weighs the current token), zeros in front of the sequence."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = bias[None, :].expand(T, C).clone()
    for j in range(K):
        out = out + padded[j: j + T] * taps[:, j][None, :]
    return out


def selective_scan(x, B, C, dt, a_log, D):
    """x [T, H, P], B and C [T, G, N], dt [T, H] (after softplus), a_log and D [H].  Head h reads group
    h // (H / G).  S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T; y_t = S_t^T C_t + D x_t."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros(T, H, P, dtype=x.dtype)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(N, P, dtype=x.dtype)
        rate = torch.exp(a_log[h])
        for t in range(T):
            S = torch.exp(-rate * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def mamba2_mixer(h, w, p, m, eps):
    """h [T, W] -> [T, W].  ``m``: the mixer's sizes (heads, vdim, state, groups, conv, norm_groups)."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[f"{p}.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner: inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[f"{p}.dt_bias"][None, :])
    y = selective_scan(x, B, C, dt, w[f"{p}.A_log"], w[f"{p}.D"]).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[f"{p}.norm"][None, :]
    return y @ w[f"{p}.o"].T


def latent_attention_mixer(h, w, p, m, eps, positions=None):
    """h [T, W] -> [T, W].  Keys and values are expanded from a latent of ``kv_rank`` numbers a token;
    one rotated key part of ``rot_dim`` numbers is shared by all heads."""
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w[f"{p}.q"].T).reshape(T, H, d + r)
    q_flat, q_rot = q[..., :d], rotate_half(q[..., d:], positions, m["rot"]["dims"], m["rot"]["base"])
    dkv = h @ w[f"{p}.dkv"].T
    c = unit_rms(dkv[:, :R], eps) * w[f"{p}.dkv.norm"][None, :]
    k_rot = rotate_half(dkv[:, None, R:], positions, m["rot"]["dims"], m["rot"]["base"])[:, 0]
    k_flat = (c @ w[f"{p}.uk"].T).reshape(T, H, d)
    v = (c @ w[f"{p}.uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_flat, k_flat) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    scores = scores.masked_fill((j > i)[None], -math.inf)
    o = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_ff(h, w, p, mlp):
    """Sigmoid scores, the ``top`` largest chosen, their scores divided by their sum (+ 1e-20), times
    ``scale``; the output is the weighted sum of the chosen experts' outputs."""
    r = mlp["router"]
    s = torch.sigmoid(h @ w[f"{p}.router"].T)
    val, idx = torch.topk(s, r["top"], dim=-1)
    weight = val / (val.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    out = torch.zeros(h.shape[0], w[f"{p}.e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for k in range(r["top"]):
            e = int(idx[t, k])
            out[t] += weight[t, k] * gated_ff(h[t: t + 1], w[f"{p}.e{e}.gate"], w[f"{p}.e{e}.up"], w[f"{p}.e{e}.down"])[0]
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return gated_ff(h, w[f"{p}.gate"], w[f"{p}.up"], w[f"{p}.down"])
    return routed_ff(h, w, p, mlp)


def connect(X, y, w, name, mult):
    """Hyper-connection write: X'_t = sum_s mix[s, t] X_s + mult * out[t] * y  (all from the old streams)."""
    if name is None:
        return X + mult * y[:, None, :]
    return torch.einsum("st,isw->itw", w[f"{name}.mix"], X) + mult * w[f"{name}.out"][None, :, None] * y[:, None, :]


def read_streams(X, w, name):
    return X[:, 0] if name is None else torch.einsum("s,isw->iw", w[f"{name}.in"], X)


def run_order(cfg) -> list:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def forward(cfg, w, tokens, keep_layers: bool = False):
    """Logits [T, vocab] for one sequence (and, with ``keep_layers``, the summed streams after every layer run)."""
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    streams = cfg.get("streams")
    x0 = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    X = x0[:, None, :].repeat(1, streams or 1, 1)
    after = []
    for i in run_order(cfg):
        L, p = cfg["layers"][i], f"l{i}"
        hc = (lambda q: f"{p}.hc{q}") if streams else (lambda q: None)
        u = unit_rms(read_streams(X, w, hc(1)), eps) * w[f"{p}.norm1"][None, :]
        if L["type"] == "mamba2":
            y = mamba2_mixer(u, w, f"{p}.mix", L["mixer"], eps)
        else:
            y = latent_attention_mixer(u, w, f"{p}.mix", L["mixer"], eps)
        X = connect(X, y, w, hc(1), mult)
        if L.get("mlp") is not None:
            u = unit_rms(read_streams(X, w, hc(2)), eps) * w[f"{p}.norm2"][None, :]
            X = connect(X, feed_forward(u, w, f"{p}.mlp", L["mlp"]), w, hc(2), mult)
        after.append(X.sum(1))
    x = unit_rms(X.sum(1), eps) * w["final.norm"][None, :]
    logits = x @ w["head"].T
    return (logits, torch.stack(after)) if keep_layers else logits

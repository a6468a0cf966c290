"""Entry points of ``csrc/decay_recurrence.cu``: linear attention with a fixed decay per head,
S <- decay S + k v^T, o = S^T q, with the state of every live request in a float32 tensor."""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

_ACT = {"none": 0, "silu": 1, "sigmoid": 2}


def prepare(proj: torch.Tensor, positions: torch.Tensor, freq: Optional[torch.Tensor], num_heads: int, key_dim: int,
            value_dim: int, activation: str, key_scale: float) -> None:
    """In place on the float32 projection [T, >= 2 H dk + H dv] = [q | k | v | ...]: ``activation``
    ("none" | "silu") on q, k and v; rotate_half rotary encoding of the first 2 len(freq) dims of each q
    and k head with angle position * freq[i]; then k times ``key_scale``."""
    ops._need(proj, "proj", torch.float32)
    ops._need(positions, "positions", torch.int32)
    if activation not in ("none", "silu"):
        raise ops.KernelError(f"no activation {activation!r} for q, k and v (none or silu)")
    T, cols = proj.shape
    if cols < 2 * num_heads * key_dim + num_heads * value_dim:
        raise ops.KernelError(f"the projection has {cols} columns, q, k and v need {2 * num_heads * key_dim + num_heads * value_dim}")
    rd = 0
    if freq is not None:
        ops._need(freq, "freq", torch.float32)
        rd = 2 * freq.numel()
    if rd == 0 and activation == "none" and key_scale == 1.0:
        return
    lib = load_library("decay_recurrence")
    ops._check(lib.tb_decay_recurrence_prep(ops._stream(), ops._ptr(proj), proj.stride(0), ops._ptr(positions), ops._ptr(freq), T,
                                            num_heads, key_dim, value_dim, rd, _ACT[activation], ctypes.c_float(key_scale)),
               "decay_recurrence_prep")


def scan(proj: torch.Tensor, cu_seqlens: torch.Tensor, state_slots: torch.Tensor, num_requests: int, state: torch.Tensor,
         decay: torch.Tensor, num_heads: int, key_dim: int, value_dim: int) -> torch.Tensor:
    """Runs every request's tokens (rows cu_seqlens[b] .. cu_seqlens[b + 1] of ``proj``) through the
    recurrence from ``state[state_slots[b]]`` [H, dk, dv] and leaves the new state there.  Returns o
    float32 [T, H dv]."""
    ops._need(proj, "proj", torch.float32)
    ops._need(cu_seqlens, "cu_seqlens", torch.int32)
    ops._need(state_slots, "state_slots", torch.int32)
    ops._need(state, "state", torch.float32)
    ops._need(decay, "decay", torch.float32)
    if tuple(state.shape[1:]) != (num_heads, key_dim, value_dim) or decay.numel() != num_heads:
        raise ops.KernelError(f"state {tuple(state.shape)} / {decay.numel()} decays do not fit {num_heads} heads of "
                              f"{key_dim} x {value_dim}")
    if cu_seqlens.numel() < num_requests + 1 or state_slots.numel() < num_requests:
        raise ops.KernelError("cu_seqlens or state_slots are shorter than the number of requests")
    out = torch.empty((proj.shape[0], num_heads * value_dim), dtype=torch.float32, device=proj.device)
    lib = load_library("decay_recurrence")
    ops._check(lib.tb_decay_recurrence_scan(ops._stream(), ops._ptr(proj), proj.stride(0), ops._ptr(cu_seqlens),
                                            ops._ptr(state_slots), ops._ptr(state), ops._ptr(decay), ops._ptr(out), num_requests,
                                            num_heads, key_dim, value_dim), "decay_recurrence_scan")
    return out


def finish(o: torch.Tensor, gate: Optional[torch.Tensor], weight: Optional[torch.Tensor], num_heads: int, value_dim: int,
           per_head: bool, gate_activation: str, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """o [T, H dv] float32 divided by its root mean square (``per_head``: each head by its own, no
    weight; else all heads together, times ``weight`` [H dv]), times act(gate) (float32 rows of H dv
    values, any row stride), rounded to ``out_dtype``."""
    ops._need(o, "o", torch.float32)
    T = o.shape[0]
    stride = 0
    if gate is not None:
        ops._need(gate, "gate", torch.float32, contiguous=False)
        if gate.shape != o.shape or gate.stride(1) != 1:
            raise ops.KernelError(f"gate {tuple(gate.shape)} does not fit o {tuple(o.shape)}")
        stride = gate.stride(0)
    if weight is not None:
        ops._need(weight, "weight", torch.float32)
        if weight.numel() != num_heads * value_dim:
            raise ops.KernelError(f"norm weight has {weight.numel()} elements, rows have {num_heads * value_dim}")
    y = torch.empty((T, num_heads * value_dim), dtype=out_dtype, device=o.device)
    lib = load_library("decay_recurrence")
    ops._check(lib.tb_decay_recurrence_post(ops._stream(), ops._ptr(o), ops._ptr(gate), stride, ops._ptr(weight), ops._ptr(y), T,
                                            num_heads, value_dim, 0 if per_head else 1, _ACT[gate_activation], ctypes.c_float(eps),
                                            ops._code(out_dtype)), "decay_recurrence_post")
    return y

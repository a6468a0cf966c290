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


# ----------------------------------------------------------------------------- selective recurrences
def scan_general(rows: torch.Tensor, cu_seqlens: torch.Tensor, state_slots: torch.Tensor, num_requests: int, state: torch.Tensor,
                 decay: Optional[torch.Tensor], decay_tok: Optional[torch.Tensor], num_heads: int, qk_heads: int, key_dim: int,
                 value_dim: int, q_off: int, k_off: int, v_off: int) -> torch.Tensor:
    """The scan with its layout as arguments: ``rows`` float32 [T, cols] holds ``qk_heads`` sets of q from
    column ``q_off`` and of k from ``k_off`` (``key_dim`` numbers each; head h reads set h // (H / qk_heads))
    and H values of ``value_dim`` numbers from ``v_off``; ``state`` float32 [slots, >= H dk dv] holds a
    request's S [H, dk, dv] at the front of its row; ``decay`` [H] (None: 1) is the fixed decay, ``decay_tok``
    [T, H] one per token that takes its place.  Returns o float32 [T, H dv]."""
    ops._need(rows, "rows", torch.float32)
    ops._need(cu_seqlens, "cu_seqlens", torch.int32)
    ops._need(state_slots, "state_slots", torch.int32)
    ops._need(state, "state", torch.float32)
    per_slot = state[0].numel()
    if per_slot < num_heads * key_dim * value_dim:
        raise ops.KernelError(f"a state row of {per_slot} numbers does not hold {num_heads} x {key_dim} x {value_dim}")
    if decay is not None:
        ops._need(decay, "decay", torch.float32)
    if decay_tok is not None:
        ops._need(decay_tok, "decay_tok", torch.float32)
        if tuple(decay_tok.shape) != (rows.shape[0], num_heads):
            raise ops.KernelError(f"decays per token have shape {tuple(decay_tok.shape)}, expected {(rows.shape[0], num_heads)}")
    if max(q_off, k_off) + qk_heads * key_dim > rows.shape[1] or v_off + num_heads * value_dim > rows.shape[1]:
        raise ops.KernelError("q, k or v lie beyond the row")
    if cu_seqlens.numel() < num_requests + 1 or state_slots.numel() < num_requests:
        raise ops.KernelError("cu_seqlens or state_slots are shorter than the number of requests")
    out = torch.empty((rows.shape[0], num_heads * value_dim), dtype=torch.float32, device=rows.device)
    lib = load_library("decay_recurrence")
    ops._check(lib.tb_recurrence_scan(ops._stream(), ops._ptr(rows), rows.stride(0), ops._ptr(cu_seqlens), ops._ptr(state_slots),
                                      ops._ptr(state), ctypes.c_longlong(per_slot), ops._ptr(decay), ops._ptr(decay_tok),
                                      ops._ptr(out), num_requests, num_heads, qk_heads, key_dim, value_dim, q_off, k_off, v_off),
               "recurrence_scan")
    return out


def selective_prepare(proj: torch.Tensor, taps: torch.Tensor, conv_bias: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                      state: torch.Tensor, conv_offset: int, ctx, num_heads: int, value_dim: int, group_cols: int,
                      num_taps: int) -> tuple:
    """From the float32 projection [T, >= 2 H P + GN2 + H] = [z | x | B | C | dt] to the scan's rows
    float32 [T, 2 H P + GN2] = [x | B | C | dt x] (x, B, C after the causal convolution and SiLU) and the decays
    float32 [T, H] = exp(-exp(A_log) softplus(dt + dt_bias)).  The inputs in front of the step's first token
    come from ``state`` [slots, n], where a request keeps its last ``num_taps - 1`` inputs from ``conv_offset`` on."""
    ops._need(proj, "proj", torch.float32)
    ops._need(state, "state", torch.float32)
    inner, C = num_heads * value_dim, num_heads * value_dim + group_cols
    T = proj.shape[0]
    if proj.shape[1] < inner + C + num_heads:
        raise ops.KernelError(f"the projection has {proj.shape[1]} columns, the layer needs {inner + C + num_heads}")
    for t, n, size in ((taps, "taps", C * num_taps), (conv_bias, "conv_bias", C), (dt_bias, "dt_bias", num_heads), (a_log, "A_log", num_heads)):
        ops._need(t, n, torch.float32)
        if t.numel() != size:
            raise ops.KernelError(f"{n} has {t.numel()} elements, expected {size}")
    per_slot = state[0].numel()
    if conv_offset + (num_taps - 1) * C > per_slot:
        raise ops.KernelError("the convolution's inputs do not fit into the state row")
    rows = torch.empty((T, 2 * inner + group_cols), dtype=torch.float32, device=proj.device)
    decay = torch.empty((T, num_heads), dtype=torch.float32, device=proj.device)
    steps = torch.empty((T, num_heads), dtype=torch.float32, device=proj.device)
    lib = load_library("decay_recurrence")
    conv_state = ctypes.c_void_p(state.data_ptr() + 4 * conv_offset)
    ops._check(lib.tb_selective_prep(ops._stream(), ops._ptr(proj), proj.stride(0), ops._ptr(taps), ops._ptr(conv_bias),
                                     ops._ptr(dt_bias), ops._ptr(a_log), conv_state, ctypes.c_longlong(per_slot),
                                     ops._ptr(ctx.seq_of_token), ops._ptr(ctx.positions), ops._ptr(ctx.seq_starts),
                                     ops._ptr(ctx.state_slots), ops._ptr(rows), ops._ptr(decay), ops._ptr(steps), T, num_heads,
                                     value_dim, group_cols, num_taps), "selective_prep")
    ops.launches += 1  # two kernels
    return rows, decay


def conv_state_update(proj: torch.Tensor, first_col: int, state: torch.Tensor, conv_offset: int, ctx, channels: int,
                      num_taps: int) -> None:
    """Leaves, for every request of the step, its newest ``num_taps - 1`` convolution inputs (columns
    ``first_col`` .. + channels of ``proj``; older ones from the state itself) in its state row."""
    if num_taps <= 1:
        return
    lib = load_library("decay_recurrence")
    conv_state = ctypes.c_void_p(state.data_ptr() + 4 * conv_offset)
    ops._check(lib.tb_conv_state_update(ops._stream(), ops._ptr(proj), proj.stride(0), first_col, conv_state,
                                        ctypes.c_longlong(state[0].numel()), ops._ptr(ctx.cu_seqlens), ops._ptr(ctx.state_slots),
                                        ctx.num_seqs, channels, num_taps), "conv_state_update")


def selective_finish(o: torch.Tensor, rows: torch.Tensor, proj: torch.Tensor, skip: torch.Tensor, weight: torch.Tensor,
                     num_heads: int, value_dim: int, parts: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """(o + skip_h x) * SiLU(z), divided by its root mean square in ``parts`` equal parts of the row, times
    ``weight`` [H P], rounded to ``out_dtype``.  x: the first H P columns of ``rows``; z: the first H P of ``proj``."""
    ops._need(o, "o", torch.float32)
    ops._need(skip, "skip", torch.float32)
    ops._need(weight, "weight", torch.float32)
    inner = num_heads * value_dim
    if weight.numel() != inner or skip.numel() != num_heads or inner % parts:
        raise ops.KernelError(f"norm weight {weight.numel()} / skip {skip.numel()} / {parts} parts do not fit {num_heads} x {value_dim}")
    y = torch.empty((o.shape[0], inner), dtype=out_dtype, device=o.device)
    lib = load_library("decay_recurrence")
    ops._check(lib.tb_selective_post(ops._stream(), ops._ptr(o), ops._ptr(rows), rows.stride(0), ops._ptr(proj), proj.stride(0),
                                     ops._ptr(skip), ops._ptr(weight), ops._ptr(y), o.shape[0], num_heads, value_dim, parts,
                                     ctypes.c_float(eps), ops._code(out_dtype)), "selective_post")
    return y

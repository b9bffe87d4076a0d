"""Launchers of csrc/ssm.cu: the short causal convolution and the recurrence of a state-space mixer."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream, want_f32, want_int32
from .elementwise import ctypes_ptr

_LIB = "ssm"
MAX_STATE = 256      # csrc/ssm.cu SSM_MAX_STATE
MAX_TAPS = 8         # csrc/ssm.cu SSM_MAX_TAPS


def conv_silu(proj: torch.Tensor, off: int, weight: torch.Tensor, bias: Optional[torch.Tensor], kept: torch.Tensor,
              out: torch.Tensor, seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """out[t, c] = silu(bias[c] + sum_k weight[c, k] * u[t - (taps-1-k), c]) with u = proj[:, off:off+C] inside a
    sequence and zeros before its start.  kept float32 [max_slots, taps-1, C] (rows may be strided): every
    sequence's last taps-1 inputs, read for a run's first tokens and renewed after the convolution."""
    want_f32(proj, "the projection")
    want_f32(out, "the convolution's output")
    want_f32(kept, "the kept inputs")
    T, C = out.shape
    taps = weight.shape[1]
    if weight.shape[0] != C or kept.shape[1:] != (taps - 1, C) or kept.stride(2) != 1 or kept.stride(1) != C:
        raise KernelError("conv_silu: weight, kept inputs and output do not fit together")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_conv_silu(ptr(proj), c_int(proj.shape[1]), c_int(off), ptr(weight), ptr(bias), c_int(code(weight.dtype)),
                                 ctypes_ptr(kept), c_longlong(kept.stride(0)), ptr(out), c_int(T), c_int(C), c_int(taps),
                                 ptr(seq_of_token), ptr(cu_seqlens), ptr(slots), c_int(cu_seqlens.shape[0] - 1), stream()),
          kernels=2 if taps > 1 else 1)
    return out


def ssm_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_off: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             d_skip: torch.Tensor, state: torch.Tensor, y: torch.Tensor, heads: int, vdim: int, n_state: int,
             groups: int, cu_seqlens: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """The recurrence over every sequence's run of new tokens.  xbc float32 [T, heads*vdim + 2*groups*n_state]
    (x | B | C after convolution and silu); the raw step sizes are proj[:, dt_off:dt_off+heads];
    state float32 [max_slots, heads, vdim, n_state] (a head's state column by column; rows may be strided); y float32 [T, heads*vdim]."""
    for t, what in ((xbc, "x, B and C"), (proj, "the projection"), (state, "the state"), (y, "the output")):
        want_f32(t, what)
    if not (dt_bias.dtype == a_log.dtype == d_skip.dtype):
        raise KernelError("ssm_scan: the per-head constants must share a dtype")
    if tuple(state.shape[1:]) != (heads, vdim, n_state) or not state[0].is_contiguous():
        raise KernelError("ssm_scan: the state must be [slots, heads, vdim, state] with dense rows")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_ssm_scan(ptr(xbc), c_int(xbc.shape[1]), ptr(proj), c_int(proj.shape[1]), c_int(dt_off), ptr(dt_bias),
                                ptr(a_log), ptr(d_skip), c_int(code(dt_bias.dtype)), ctypes_ptr(state),
                                c_longlong(state.stride(0)), ptr(y), c_int(cu_seqlens.shape[0] - 1), c_int(heads), c_int(vdim),
                                c_int(n_state), c_int(groups), ptr(cu_seqlens), ptr(slots), stream()))
    return y


def gated_group_norm(y: torch.Tensor, proj: torch.Tensor, z_off: int, weight: torch.Tensor, norm_groups: int, eps: float,
                     out: torch.Tensor) -> torch.Tensor:
    """out = rms_in_groups(y * silu(z)) * weight with z = proj[:, z_off:z_off+inner]: the gate first, then each of
    the norm_groups equal parts of a row divided by its own root mean square."""
    want_f32(y, "the recurrence's output")
    want_f32(proj, "the projection")
    T, inner = y.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_gated_group_norm(ptr(y), ptr(proj), c_int(proj.shape[1]), c_int(z_off), ptr(weight),
                                        c_int(code(weight.dtype)), ptr(out), c_int(code(out.dtype)), c_int(T), c_int(inner),
                                        c_int(norm_groups), c_float(eps), stream()))
    return out

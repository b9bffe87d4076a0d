"""A state-space mixer with a scalar decay per head (Mamba-2).

With inner = heads * vdim, N = state, G = groups, the input projection's rows are [z: inner | x: inner | B: G*N |
C: G*N | dt: heads].  x, B and C pass a causal convolution per channel (`taps` taps, the last on the current token,
zeros before a sequence's start) and silu.  Per head a (using group a // (heads / groups)):

    dt  = softplus(dt + dt_bias_a)
    S  <- exp(-exp(A_log_a) dt) S + dt B x^T        S is [N, vdim], zero at a sequence's start
    y   = S^T C + D_a x

then y * silu(z), an RMS norm in `norm_groups` equal parts with a weight, and the output projection.  A sequence's
state is S of every head (stored column by column, [vdim, N]) and the convolution's last taps-1 inputs, both
float32, in one row of the cache's state area.  The projection leaves the library's product as float32 and everything up to the gated norm stays float32.
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ssm as KS
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import LayerCache, Mixer, StateNeed, StepContext, register_mixer


class Mamba2Mixer(Mixer):
    def __init__(self, prefix: str, hidden: int, heads: int, vdim: int, state: int, groups: int, taps: int,
                 norm_groups: int, eps: float):
        if heads < 1 or vdim < 1 or groups < 1 or heads % groups:
            raise ValueError(f"state-space mixer '{prefix}': {heads} heads in {groups} groups")
        if not 1 <= state <= KS.MAX_STATE or not 1 <= taps <= KS.MAX_TAPS:
            raise ValueError(f"state-space mixer '{prefix}': state {state} (1..{KS.MAX_STATE}), taps {taps} (1..{KS.MAX_TAPS})")
        if norm_groups < 1 or (heads * vdim) % norm_groups:
            raise ValueError(f"state-space mixer '{prefix}': {heads * vdim} elements in {norm_groups} norm groups")
        self.prefix, self.hidden = prefix, int(hidden)
        self.heads, self.vdim, self.n_state, self.groups = int(heads), int(vdim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps = int(taps), int(norm_groups), float(eps)
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state                 # what the convolution sees
        self.proj_rows = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        self.kept_size = (self.taps - 1) * self.channels
        self.w_in = self.w_conv = self.b_conv = self.dt_bias = self.a_log = self.d_skip = self.w_norm = self.w_o = None

    def weight_specs(self) -> List[WeightSpec]:
        p = self.prefix
        return [WeightSpec(p + "in", (self.proj_rows, self.hidden)), WeightSpec(p + "conv", (self.channels, self.taps)),
                WeightSpec(p + "conv.b", (self.channels,)), WeightSpec(p + "dt_bias", (self.heads,)),
                WeightSpec(p + "A_log", (self.heads,)), WeightSpec(p + "D", (self.heads,), init="one_plus_normal"),
                WeightSpec(p + "norm", (self.inner,), init="one_plus_normal"), WeightSpec(p + "o", (self.hidden, self.inner))]

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        self.w_in, self.w_o = store.get(p + "in"), store.get(p + "o")
        self.w_conv, self.b_conv = store.get(p + "conv"), store.get(p + "conv.b")
        # what enters the recurrence is float32
        self.dt_bias, self.a_log, self.d_skip = (store.get(p + n).float().contiguous() for n in ("dt_bias", "A_log", "D"))
        self.w_norm = store.get(p + "norm")

    def kernels(self) -> List[str]:
        return ["ssm"]

    def state_need(self) -> StateNeed:
        return StateNeed((self.kept_size + self.heads * self.n_state * self.vdim,), torch.float32)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        state = 4.0 * self.heads * self.n_state * self.vdim
        return {"matmul": (wb(self.w_in) + wb(self.w_o), 2.0 * n_tokens * self.hidden * (self.proj_rows + self.inner)),
                "other": (2.0 * state, 6.0 * n_tokens * self.heads * self.n_state * self.vdim)}

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T, dev = xn.shape[0], xn.device
        st = cache.state                                                       # [max_slots, kept | S]
        kept = st[:, :self.kept_size].unflatten(1, (self.taps - 1, self.channels))
        S = st[:, self.kept_size:].unflatten(1, (self.heads, self.vdim, self.n_state))     # column by column
        proj = linear(xn, self.w_in, out_dtype=torch.float32)                  # [T, z | x | B | C | dt]
        xbc = torch.empty((T, self.channels), dtype=torch.float32, device=dev)
        KS.conv_silu(proj, self.inner, self.w_conv, self.b_conv, kept, xbc, ctx.seq_of_token, ctx.cu_seqlens, ctx.slots)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        KS.ssm_scan(xbc, proj, 2 * self.inner + 2 * self.groups * self.n_state, self.dt_bias, self.a_log, self.d_skip, S, y,
                    self.heads, self.vdim, self.n_state, self.groups, ctx.cu_seqlens, ctx.slots)
        g = torch.empty((T, self.inner), dtype=ctx.act_dtype, device=dev)
        KS.gated_group_norm(y, proj, 0, self.w_norm, self.norm_groups, self.eps, g)
        return linear(g, self.w_o, out_dtype=torch.float32)


register_mixer("mamba2", Mamba2Mixer)

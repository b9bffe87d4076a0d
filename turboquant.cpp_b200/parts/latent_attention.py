"""Latent attention: every position caches one low-rank row instead of keys and values per head.

With h the mixer's input, H heads, per head `dim` plain and `rot_dim` rotated query/key dimensions, value size
`vdim` and latent size `kv_rank`:

    q          = W_q h                       [H, dim + rot_dim], head by head as [plain | rotated]
    [d | r]    = W_dkv h                     kv_rank + rot_dim rows
    c          = rms(d) * w                  the latent (RMS norm with a weight)
    kr         = rotate(r)                   one rotated key part that all heads share
    key_a      = [W_uk,a c | kr],  value_a = W_uv,a c
    score      = (q_plain . W_uk,a c + rotate(q_rot) . kr) * scale

Only [c | kr] is cached.  The products with W_uk and W_uv are moved to the query's side: q~_a = W_uk,a^T q_plain
meets c directly, the softmax-weighted sum of the c_j is taken first and W_uv,a applied to it, so one cached row
serves all heads as key and value, in prompts and in decoding alike.  Options: a window (position i sees j with
0 <= i - j < window), a learned sink per head in the softmax's denominator, reading the rows another layer
cached (the layer then has no W_dkv), and queries that go through a latent of their own:

    c_q = rms(W_dq h) * w_q,   q = W_uq c_q        (q_rank > 0; tensors dq, dq.norm, uq instead of q)
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import elementwise as KE
from ..kernels import latent_attention as KL
from ..kernels.linear import batched_linear, linear, product
from ..weights.loader import WeightSpec, WeightStore
from .base import KVNeed, LayerCache, Mixer, StepContext, register_mixer


class LatentAttentionMixer(Mixer):
    PROMPT_MIN_RUN = 32       # steps whose longest run of new tokens is at least this take the matrix-product path
    PROMPT_ROWS = 8192        # (token, head) rows of scores per block of that path

    def __init__(self, prefix: str, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, eps: float, window: int = 0, position=None, own_cache: bool = True,
                 keep_window: Optional[int] = None, sink: bool = True, q_rank: int = 0):
        """position: an encoding with `freq` and `mag` (parts.rotary.ScaledRotaryEncoding) over at most rot_dim
        dimensions, or None.  own_cache False: the layer has no latent projection and reads the rows of the
        schedule entry its own entry names.  keep_window: how long the cache keeps rows (0: all); a layer whose
        rows are read by layers with other windows must keep them for the widest."""
        if heads < 1 or dim < 0 or rot_dim < 0 or dim + rot_dim < 1 or vdim < 1 or kv_rank < 1 or q_rank < 0:
            raise ValueError(f"latent attention '{prefix}': bad sizes")
        if kv_rank + rot_dim > KL.MAX_ROW:
            raise ValueError(f"latent attention '{prefix}': kv_rank + rot_dim = {kv_rank + rot_dim} exceeds {KL.MAX_ROW}")
        if window < 0:
            raise ValueError(f"latent attention '{prefix}': negative window {window}")
        if position is not None and position.dims > rot_dim:
            raise ValueError(f"latent attention '{prefix}': {position.dims} rotated dimensions exceed rot_dim {rot_dim}")
        self.prefix, self.hidden, self.heads = prefix, int(hidden), int(heads)
        self.dim, self.rot_dim, self.vdim, self.kv_rank = int(dim), int(rot_dim), int(vdim), int(kv_rank)
        self.scale, self.eps, self.window = float(scale), float(eps), int(window)
        self.position, self.own_cache, self.has_sink = position, bool(own_cache), bool(sink)
        self.keep_window = self.window if keep_window is None else int(keep_window)
        self.q_dim = self.dim + self.rot_dim
        self.q_rank = int(q_rank)            # 0: queries straight from the input
        self.w_dq = self.w_qnorm = None
        self.w_q = self.w_dkv = self.w_norm = self.w_uk = self.w_uv_t = self.w_o = self.sink = None

    def weight_specs(self) -> List[WeightSpec]:
        p, H = self.prefix, self.heads
        if self.q_rank:
            specs = [WeightSpec(p + "dq", (self.q_rank, self.hidden)),
                     WeightSpec(p + "dq.norm", (self.q_rank,), init="one_plus_normal"),
                     WeightSpec(p + "uq", (H * self.q_dim, self.q_rank))]
        else:
            specs = [WeightSpec(p + "q", (H * self.q_dim, self.hidden))]
        specs += [WeightSpec(p + "uk", (H * self.dim, self.kv_rank)),
                 WeightSpec(p + "uv", (H * self.vdim, self.kv_rank)), WeightSpec(p + "o", (self.hidden, H * self.vdim))]
        if self.own_cache:
            specs += [WeightSpec(p + "dkv", (self.kv_rank + self.rot_dim, self.hidden)),
                      WeightSpec(p + "dkv.norm", (self.kv_rank,), init="one_plus_normal")]
        if self.has_sink:
            specs.append(WeightSpec(p + "sink", (H,)))
        return specs

    def bind(self, store: WeightStore) -> None:
        p, H = self.prefix, self.heads
        self.w_q, self.w_o = store.get(p + ("uq" if self.q_rank else "q")), store.get(p + "o")
        if self.q_rank:
            self.w_dq, self.w_qnorm = store.get(p + "dq"), store.get(p + "dq.norm")
        self.w_uk = store.get(p + "uk").view(H, self.dim, self.kv_rank)                       # q_plain [T, dim] @ [dim, R]
        self.w_uv_t = store.get(p + "uv").view(H, self.vdim, self.kv_rank).transpose(1, 2)    # sums [T, R] @ [R, vdim]
        if self.own_cache:
            self.w_dkv, self.w_norm = store.get(p + "dkv"), store.get(p + "dkv.norm")
        if self.has_sink:
            self.sink = store.get(p + "sink").float().contiguous()
        if self.position is not None:
            self.position.prepare(store.device)

    def kernels(self) -> List[str]:
        return ["latent_attention"] + (["elementwise"] if self.q_rank else [])

    def cache_need(self) -> KVNeed:
        return KVNeed(1, self.kv_rank + self.rot_dim, self.keep_window, planes=1)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        H, R = self.heads, self.kv_rank
        proj = ((self.hidden + H * self.q_dim) * self.q_rank if self.q_rank else self.hidden * H * self.q_dim) \
            + H * self.vdim * self.hidden + H * R * (self.dim + self.vdim)
        if self.own_cache:
            proj += self.hidden * (R + self.rot_dim)
        el = 2 if getattr(self, "run_dtype", None) == torch.bfloat16 else 4
        seen = min(kv_tokens, n_tokens * self.window) if self.window else kv_tokens
        return {"matmul": (sum(wb(w) for w in (self.w_q, self.w_dq, self.w_dkv, self.w_uk, self.w_uv_t, self.w_o)), 2.0 * n_tokens * proj),
                "attn": (float((R + self.rot_dim) * el * seen), 2.0 * H * (2 * R + self.rot_dim) * seen)}

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T, H, R, act = xn.shape[0], self.heads, self.kv_rank, ctx.act_dtype
        if self.q_rank:
            # the queries' latent: projection in float32, RMS norm with its weight, rounded to the activation dtype
            cq = KE.rmsnorm(linear(xn, self.w_dq, out_dtype=torch.float32), self.w_qnorm, self.eps,
                            torch.empty((T, self.q_rank), dtype=act, device=xn.device))
            q = linear(cq, self.w_q, out_dtype=act)
        else:
            q = linear(xn, self.w_q, out_dtype=act)                                    # [T, H * (dim + rot_dim)]
        dkv = linear(xn, self.w_dkv, out_dtype=torch.float32) if self.own_cache else None
        freq, mag = (self.position.freq, self.position.mag) if self.position is not None and self.position.dims else (None, 1.0)
        # norm of the latent, the two rotations and the cache write in one launch
        KL.latent_prepare(q, dkv, self.w_norm, self.eps, freq, mag, ctx.positions, ctx.seq_of_token, cache.page_table,
                          cache.page_size, cache.kv, H, self.dim, self.rot_dim, R)
        q3 = q.view(T, H, self.q_dim)
        runs = (ctx.max_q_len >= self.PROMPT_MIN_RUN and len(ctx.host_q_lens) == ctx.n_seqs
                and len(ctx.host_seq_start) == ctx.n_seqs)
        # the prompt path wants [query in the latent space | rotated part] side by side: the product writes there
        qa = torch.empty((T, H, R + self.rot_dim), dtype=act, device=xn.device) if runs else None
        q_lat = qa[:, :, :R] if runs else torch.empty((T, H, R), dtype=act, device=xn.device)
        if self.dim:
            batched_linear(q3[:, :, :self.dim].transpose(0, 1), self.w_uk, q_lat.transpose(0, 1))
        else:
            q_lat.zero_()
        sums = torch.empty((T, H, R), dtype=act, device=xn.device)
        if runs:
            if self.rot_dim:
                qa[:, :, R:].copy_(q3[:, :, self.dim:])
            self._attend_runs(qa, sums, ctx, cache)
        else:
            self._attend_tokens(q, q_lat, sums, ctx, cache)
        v = torch.empty((T, H, self.vdim), dtype=act, device=xn.device)
        batched_linear(sums.transpose(0, 1), self.w_uv_t, v.transpose(0, 1))
        return linear(v.view(T, H * self.vdim), self.w_o, out_dtype=torch.float32)

    def _attend_tokens(self, q, q_lat, sums, ctx: StepContext, cache: LayerCache) -> None:
        """Every token on its own: the kernel walks its keys (decode steps, short runs).  Reads device tensors of
        the step only, so it runs inside the decode graphs."""
        T, H, R = q_lat.shape
        longest = min(self.window, ctx.max_kv_len) if self.window else ctx.max_kv_len
        n_splits = KL.splits_for(T, H, longest, q.device, KL.tensor_core_form(q.dtype, R, self.rot_dim))
        partial = torch.empty(T * H * n_splits * (R + 2), dtype=torch.float32, device=q.device) if n_splits > 1 else None
        KL.latent_attention(q_lat, q, self.dim, cache.kv, self.sink, ctx.positions, ctx.seq_of_token, cache.page_table,
                            cache.page_size, self.window, self.scale, sums, H, R, self.rot_dim, n_splits, partial)

    def _attend_runs(self, qa, sums, ctx: StepContext, cache: LayerCache) -> None:
        """Long runs of new tokens (prompts): all heads of a block of tokens meet the same cached rows, so scores
        and weighted sums are two matrix products of the library over (token, head) rows, with the mask, the
        scale and the softmax with its sink between them in a kernel of their own (float32 scores in, weights in
        the activation dtype out).  A block's rows are gathered from the pages once.  It walks the step's
        sequences on the host; steps of single tokens never come here."""
        H, R, Dk = self.heads, self.kv_rank, self.kv_rank + self.rot_dim
        act, dev = qa.dtype, qa.device
        block = max(16, self.PROMPT_ROWS // H)
        # one buffer for the gathered rows and one for the weights, sized for the widest block of the step
        longest = max(ctx.host_q_lens)
        most = min(block, longest) + (self.window - 1 if self.window else ctx.max_kv_len)
        most = -(-min(most, ctx.max_kv_len) // 64) * 64
        rows_all = torch.empty((most, Dk), dtype=act, device=dev)
        weights_all = torch.empty(min(block, longest) * H * most, dtype=act, device=dev)
        t0 = 0
        for i, (n, start) in enumerate(zip(ctx.host_q_lens, ctx.host_seq_start)):
            for a in range(0, n, block):
                b = min(n, a + block)
                pos0, k1 = start + a, start + b
                k0 = max(0, pos0 + 1 - self.window) if self.window else 0
                # the library's fast products want dimensions that are multiples of 64 elements: the block's rows are
                # padded with zero rows, which the softmax gives weight 0 (they lie behind the block's last position)
                n_keys = k1 - k0
                n_pad = -(-n_keys // 64) * 64
                rows = rows_all[:n_pad]
                KL.latent_gather(cache.kv, cache.page_table[i], cache.page_size, k0, n_keys, rows[:n_keys])
                if n_pad > n_keys:
                    rows[n_keys:].zero_()
                scores = product(qa[t0 + a:t0 + b].view(-1, Dk), rows.t(), out_dtype=torch.float32)
                weights = weights_all[:scores.shape[0] * n_pad].view(scores.shape[0], n_pad)
                KL.latent_softmax(scores, self.sink, self.scale, self.window, pos0, k0, H, weights)
                product(weights, rows[:, :R], out=sums[t0 + a:t0 + b].view(-1, R))
            t0 += n


register_mixer("latent_attention", LatentAttentionMixer)

"""Launchers of csrc/latent_attention.cu: attention over a cache of one latent row per position."""
from __future__ import annotations

from ctypes import c_float, c_int
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream, want_f32, want_int32

_LIB = "latent_attention"
MAX_ROW = 1024       # csrc/latent_attention.cu LAT_MAX_ROW
HEADS_PER_BLOCK = 4  # csrc/latent_attention.cu LAT_HG


def latent_prepare(q: torch.Tensor, dkv: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor], eps: float,
                   freq: Optional[torch.Tensor], mag: float, positions: torch.Tensor, seq_of_token: torch.Tensor,
                   page_table: Optional[torch.Tensor], page_size: int, cache: Optional[torch.Tensor], heads: int,
                   q_off: int, rot: int, kv_rank: int) -> None:
    """q [T, heads * q_dim] (activation dtype): the `rot` elements from q_off of every head turn in place.
    dkv float32 [T, kv_rank + rot] (or None for a layer that reads another layer's cache): its first kv_rank
    elements are normed (RMS, weight), its last rot turned, and the row is written to the token's place in
    cache [pages, 1, 1, page_size, kv_rank + rot]."""
    T = q.shape[0]
    q_dim = q.shape[1] // heads
    n_pairs = 0 if freq is None else freq.shape[0]
    if dkv is not None:
        want_f32(dkv, "the latent projection")
        if dkv.shape != (T, kv_rank + rot) or cache is None or cache.dtype != q.dtype:
            raise KernelError("latent_prepare: the projection, the cache and the queries do not fit together")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_latent_prepare(
        ptr(q), c_int(code(q.dtype)), ptr(dkv), ptr(norm_weight),
        c_int(code(norm_weight.dtype) if norm_weight is not None else 0), c_float(eps), ptr(freq), c_float(mag),
        ptr(positions), ptr(seq_of_token), ptr(page_table), c_int(page_table.shape[1] if page_table is not None else 0),
        c_int(page_size), ptr(cache) if dkv is not None else None, c_int(T), c_int(heads), c_int(q_dim), c_int(q_off),
        c_int(rot), c_int(n_pairs), c_int(kv_rank), c_int(page_table.shape[0] if page_table is not None else 0),
        c_int(cache.shape[0] if cache is not None else 0), stream()))


def tensor_core_form(dtype: torch.dtype, kv_rank: int, rot: int) -> bool:
    """Whether the launcher takes the tensor-core form of the kernel (csrc/latent_attention.cu: bfloat16, kv_rank a
    multiple of 32 up to 512, kv_rank + rot a multiple of 16; TQ_LATENT_NO_MMA=1 switches it off)."""
    import os
    return (dtype == torch.bfloat16 and kv_rank % 32 == 0 and kv_rank <= 512 and (kv_rank + rot) % 16 == 0
            and os.environ.get("TQ_LATENT_NO_MMA", "") in ("", "0"))


def splits_for(n_tokens: int, heads: int, longest: int, device, tensor_cores: bool = False) -> int:
    """Key ranges per token.  A step of few tokens over long ranges is cut until a block has about 64 keys or the
    launch fills the GPU: three waves of blocks in the CUDA-core form (four heads a block, sixteen keys at a time),
    one wave of two blocks per SM in the tensor-core form (sixteen heads a block, tiles of 32 keys, two blocks'
    shared memory per SM), whose blocks are long enough for a second, partly filled wave to cost more than it
    brings.  Prompts (many tokens) are not cut.  The ranges are joined in range order, so a launch shape gives the
    same bits every time; logits agree across shapes to rounding."""
    blocks = n_tokens * -(-heads // (16 if tensor_cores else HEADS_PER_BLOCK))
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    room = (2 * sms) // blocks if tensor_cores else (3 * sms) // blocks
    return int(max(1, min(64, longest // 64, room)))


def latent_attention(q_lat: torch.Tensor, q: torch.Tensor, q_off: int, cache: torch.Tensor, sink: Optional[torch.Tensor],
                     positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int,
                     window: int, scale: float, out: torch.Tensor, heads: int, kv_rank: int, rot: int,
                     n_splits: int = 1, partial: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q_lat [T, heads, kv_rank]: the queries carried into the latent space; q [T, heads * q_dim]: its `rot`
    elements from q_off of every head meet the rows' last rot elements.  out [T, heads, kv_rank]: the
    softmax-weighted sums of the rows' first kv_rank elements (sink [heads] float32 joins the denominator)."""
    T = q_lat.shape[0]
    if sink is not None:
        want_f32(sink, "sinks")
    want_int32(positions, "positions")
    if cache.dtype != q_lat.dtype or out.dtype != q_lat.dtype or q.dtype != q_lat.dtype:
        raise KernelError("latent_attention: queries, cache and output must share a dtype")
    if n_splits > 1 and (partial is None or partial.numel() < T * heads * n_splits * (kv_rank + 2)):
        raise KernelError("latent_attention: the scratch buffer is too small for the key ranges")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_latent_attention(
        ptr(q_lat), ptr(q), c_int(q.shape[1] // heads), c_int(q_off), ptr(cache), c_int(code(q_lat.dtype)), ptr(sink),
        ptr(positions), ptr(seq_of_token), ptr(page_table), c_int(page_table.shape[1]), c_int(page_size), c_int(window),
        c_float(scale), ptr(out), ptr(partial), c_int(n_splits), c_int(T), c_int(heads), c_int(kv_rank), c_int(rot),
        c_int(page_table.shape[0]), c_int(cache.shape[0]), stream()), kernels=2 if n_splits > 1 else 1)
    return out


def latent_gather(cache: torch.Tensor, table_row: torch.Tensor, page_size: int, k0: int, n: int, out: torch.Tensor) -> torch.Tensor:
    """out[j] = the cached row of position k0 + j of the sequence whose pages table_row lists, j < n."""
    want_int32(table_row, "the page table")
    Dk = cache.shape[-1]
    if tuple(out.shape) != (n, Dk) or out.dtype != cache.dtype:
        raise KernelError("latent_gather: the output must be [n, row] in the cache's dtype")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_latent_gather(ptr(cache), c_int(code(cache.dtype)), ptr(table_row), c_int(table_row.shape[0]),
                                     c_int(page_size), c_int(k0), c_int(n), c_int(Dk), ptr(out), c_int(cache.shape[0]), stream()))
    return out


def latent_softmax(scores: torch.Tensor, sink: Optional[torch.Tensor], scale: float, window: int, pos0: int, k0: int,
                   heads: int, weights: torch.Tensor) -> torch.Tensor:
    """scores float32 [tokens * heads, n_keys] of a run of tokens at positions pos0 … against positions k0 …:
    the softmax of the visible scores (causal, window) times scale, the sink in the denominator; 0 elsewhere."""
    want_f32(scores, "scores")
    rows, n_keys = scores.shape
    if weights.shape != scores.shape:
        raise KernelError("latent_softmax: weights and scores differ in shape")
    lib = load_kernel(_LIB)
    from ctypes import c_longlong
    check(_LIB, lib.tq_latent_softmax(ptr(scores), ptr(sink), c_float(scale), c_int(window), c_int(pos0), c_int(k0),
                                      c_int(n_keys), c_int(heads), ptr(weights), c_int(code(weights.dtype)), c_longlong(rows),
                                      stream()))
    return weights

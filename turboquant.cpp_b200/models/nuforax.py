"""The Nuforax decoder as a list of parts.

Embedding with a scale and a table of token pairs; layers in the order config.json lists them, each a mixer
(latent attention with a window and sinks, or a state-space mixer) and an optional dense feed-forward with the
square of relu, norms on the sub-layers' outputs; final RMS norm; logits from the embedding table itself.  A
latent-attention layer may read the rows an earlier layer cached (`kv_from`) instead of projecting its own.
Tensors: embed, bigram, l<i>.norm1|norm2, l<i>.mix.<name>, l<i>.mlp.up|down, final.norm.
"""
from __future__ import annotations

import torch

from ..config.nuforax import ARCHITECTURE, NuforaxConfig
from ..config.registry import register_architecture
from ..parts import PostNormBlock, make_feed_forward, make_mixer, make_norm, make_position_encoding
from .decoder import DecoderModel, LMHead, PairEmbedding, ScheduleEntry


class NuforaxModel(DecoderModel):
    def __init__(self, cfg: NuforaxConfig, dtype: torch.dtype):
        W = cfg.width
        # how long a layer's cached rows must be kept: for the widest window among the layer and its readers
        keep = {}
        for i, layer in enumerate(cfg.layers):
            if layer.type == "latent_attention":
                src = i if layer.mixer.kv_from is None else layer.mixer.kv_from
                w = layer.mixer.window
                keep[src] = w if src not in keep else (0 if 0 in (w, keep[src]) else max(w, keep[src]))
        blocks, schedule = [], []
        for i, layer in enumerate(cfg.layers):
            p, m = f"l{i}.", layer.mixer
            if layer.type == "latent_attention":
                sc = m.rot_scaling
                position = make_position_encoding(
                    "rotary_scaled", dims=m.rot_dims, base=m.rot_base, factor=sc.factor if sc else None,
                    original=sc.original if sc else 0.0, fast=sc.fast if sc else 0.0, slow=sc.slow if sc else 0.0)
                src = i if m.kv_from is None else m.kv_from
                mixer = make_mixer("latent_attention", prefix=p + "mix.", hidden=W, heads=m.heads, dim=m.dim,
                                   rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale, eps=cfg.eps,
                                   window=m.window, position=position, own_cache=m.kv_from is None,
                                   keep_window=keep[src], sink=True)
                schedule.append(ScheduleEntry(i, cache_of=m.kv_from))
            else:
                mixer = make_mixer("mamba2", prefix=p + "mix.", hidden=W, heads=m.heads, vdim=m.vdim, state=m.state,
                                   groups=m.groups, taps=m.conv, norm_groups=m.norm_groups, eps=cfg.eps)
                schedule.append(ScheduleEntry(i))
            ffn = ffn_norm = None
            if layer.mlp is not None:
                ffn = make_feed_forward("relu2", prefix=p + "mlp.", hidden=W, intermediate=layer.mlp.ff)
                ffn_norm = make_norm("rmsnorm", name=p + "norm2", size=W, eps=cfg.eps)
            blocks.append(PostNormBlock(mixer, make_norm("rmsnorm", name=p + "norm1", size=W, eps=cfg.eps), ffn, ffn_norm))
        pt = cfg.pair_table
        super().__init__(
            cfg, dtype,
            embedding=PairEmbedding("embed", cfg.vocab, W, scale=cfg.embedding_scale,
                                    pair_name="bigram" if pt else None, buckets=pt.buckets if pt else 0,
                                    mul_prev=pt.mul_prev if pt else 0, mul_cur=pt.mul_cur if pt else 0),
            blocks=blocks, schedule=schedule,
            final_norm=make_norm("rmsnorm", name="final.norm", size=W, eps=cfg.eps),
            head=LMHead("embed", cfg.vocab, W))


register_architecture(ARCHITECTURE, NuforaxConfig, NuforaxModel)

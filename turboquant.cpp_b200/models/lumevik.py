"""The Lumevik decoder as a list of parts.

Plain embedding; layers in the order config.json lists them, each a mixer and an optional feed-forward in a
pre-norm block whose norms store their weights around zero; final norm of the same kind; a head of its own.
Mixers: attention without rotation (distance bias, window with kept first positions, a sink of score zero, values
mixed with those of the first such layer), or latent attention without positions whose queries pass a latent too.
Feed-forwards: a gated one with caps (dense), or routed experts of that form with corrected scores, groups and a
shared expert.  Tensors: embed, l<i>.norm1|norm2, l<i>.mix.<name>, l<i>.mlp.<name>, final.norm, head.
"""
from __future__ import annotations

import torch

from ..config.lumevik import ARCHITECTURE, GLU_SLOPE, GLU_UP_OFFSET, ROUTER_WEIGHT_FLOOR, DenseMlpConfig, LumevikConfig
from ..config.registry import register_architecture
from ..kernels.elementwise import Glu
from ..parts import PreNormBlock, make_feed_forward, make_mixer, make_norm
from .decoder import DecoderModel, Embedding, LMHead, ScheduleEntry

MOE_NAMES = {"router": "router", "expert": "e{e}.", "gate": "gate", "up": "up", "down": "down", "shared": "shared.",
             "shared_gate": "shared.sg", "correction": "correction"}
MIXED_VALUES = "values_of_first_mixing_layer"      # the name under which mixing layers share values within a step


class LumevikModel(DecoderModel):
    def __init__(self, cfg: LumevikConfig, dtype: torch.dtype):
        W = cfg.width
        norm = lambda name: make_norm("rmsnorm", name=name, size=W, eps=cfg.eps, around_zero=True)
        glu = lambda limit: Glu(limit=limit, slope=GLU_SLOPE, offset=GLU_UP_OFFSET)
        blocks, first_mixing = [], None
        for i, layer in enumerate(cfg.layers):
            p, m = f"l{i}.", layer.mixer
            if layer.type == "attention":
                if m.v_mix and first_mixing is None:
                    first_mixing = i
                mixer = make_mixer("window_bias_attention", prefix=p + "mix.", hidden=W, heads=m.heads,
                                   kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, window=m.window,
                                   keep_first=m.keep_first, bias_rows=m.bias_rows or -1, bias_far=m.bias_max, sink=True,
                                   mix_values=MIXED_VALUES if m.v_mix else None, mix_first=first_mixing == i)
            else:
                mixer = make_mixer("latent_attention", prefix=p + "mix.", hidden=W, heads=m.heads, dim=m.dim, rot_dim=0,
                                   vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale, eps=cfg.eps, window=0, position=None,
                                   sink=False, q_rank=m.q_rank)
            ffn = ffn_norm = None
            if layer.mlp is not None:
                ffn_norm = norm(p + "norm2")
                if isinstance(layer.mlp, DenseMlpConfig):
                    ffn = make_feed_forward("glu", prefix=p + "mlp.", hidden=W, intermediate=layer.mlp.ff,
                                            glu=glu(layer.mlp.limit))
                else:
                    e = layer.mlp
                    ffn = make_feed_forward("moe", prefix=p + "mlp.", hidden=W, n_experts=e.experts, top_k=e.top,
                                            intermediate=e.ff, norm_topk=True, shared_intermediate=e.shared_ff,
                                            shared_gate=True, glu=glu(e.limit),
                                            shared_glu=glu(e.shared_limit) if e.shared_ff else None, correction=True,
                                            n_groups=e.groups, keep_groups=e.keep_groups,
                                            renorm_floor=ROUTER_WEIGHT_FLOOR, names=MOE_NAMES)
            blocks.append(PreNormBlock(norm(p + "norm1"), mixer, ffn_norm, ffn))
        super().__init__(cfg, dtype, embedding=Embedding("embed", cfg.vocab, W), blocks=blocks,
                         schedule=[ScheduleEntry(i) for i in range(len(blocks))],
                         final_norm=norm("final.norm"), head=LMHead("head", cfg.vocab, W))


register_architecture(ARCHITECTURE, LumevikConfig, LumevikModel)

"""Typed configuration of the Lumevik decoder.

config.json of this design is nested: ``norm`` (eps), ``vocab``, ``width`` and ``layers``, a list in which every entry
names its mixer kind (``type``), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``, or null
for none; ``kind`` dense or moe).  The order and kinds of the layers are data: two models of the design may differ
in all of it.  Every size and constant is read here; the parts get them as parameters.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .reader import ConfigError, KeyReader

ARCHITECTURE = "Lumevik"
# constants the design fixes
GLU_SLOPE = 1.702            # the gate's sigmoid is taken of GLU_SLOPE * gate
GLU_UP_OFFSET = 1.0          # the gated value multiplies (up + GLU_UP_OFFSET)
ROUTER_WEIGHT_FLOOR = 1e-20  # added to the sum of the chosen experts' scores before the division
# limits of the kernels the design's parts launch (csrc/bias_attention.cu BA_MAX_DIM, csrc/latent_attention.cu
# LAT_MAX_ROW), checked when the configuration is read
MAX_HEAD_SIZE = 256
MAX_LATENT_ROW = 1024


def _sub(r: KeyReader, key: str, required: bool = True) -> Optional[KeyReader]:
    r.seen.add(key)
    v = r.raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"{r.where}: required key '{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{r.where}: key '{key}' must be an object, got {v!r}")
    return KeyReader(v, f"{r.where}: {key}")


@dataclass(frozen=True)
class BiasAttentionConfig:
    heads: int
    kv_heads: int
    dim: int              # query/key size per head
    vdim: int             # value size per head
    scale: float
    bias_max: int         # the distance from which all distances share the bias table's last row
    bias_rows: int        # rows of the bias table; 0: as many as the stored tensor has (random weights need the key)
    window: int           # 0: every earlier position is seen
    keep_first: int       # positions at a sequence's start that stay visible beyond the window
    v_mix: bool


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeMlpConfig:
    experts: int
    top: int
    groups: int
    keep_groups: int
    ff: int
    limit: float
    shared_ff: int        # 0: no shared expert
    shared_limit: float


@dataclass(frozen=True)
class LumevikLayer:
    type: str
    mixer: Any
    mlp: Any              # DenseMlpConfig, MoeMlpConfig or None


@dataclass(frozen=True)
class LumevikConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[LumevikLayer, ...]
    raw: Dict[str, Any]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = ARCHITECTURE
    # the design has no longest sequence of its own (no position table)
    max_position_embeddings: int = 1 << 30

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "LumevikConfig":
        r = KeyReader(raw, where)
        width = r.integer("width", minimum=1)
        r.seen.add("layers")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: required key 'layers' must be a non-empty list")
        layers = []
        for i, item in enumerate(layers_raw):
            lw = f"{where}: layers[{i}]"
            lr = KeyReader(item, lw)
            kind = lr.string("type")
            m = _sub(lr, "mixer")
            if kind == "attention":
                mixer = _attention(m)
            elif kind == "latent_attention":
                mixer = _latent(m)
            else:
                raise ConfigError(f"{lw}: unknown layer type '{kind}' (known: attention, latent_attention)")
            ml = _sub(lr, "mlp", required=False)
            layers.append(LumevikLayer(kind, mixer, None if ml is None else _mlp(ml)))
        mixing = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        for m in mixing[1:]:
            if (m.kv_heads, m.vdim) != (mixing[0].kv_heads, mixing[0].vdim):
                raise ConfigError(f"{where}: layers that mix values ('v_mix') must agree in kv_heads and vdim")
        return cls(vocab=r.integer("vocab", minimum=1), width=width, eps=_sub(r, "norm").real("eps", positive=True),
                   layers=tuple(layers), raw=dict(raw), eos_token_ids=tuple(r.token_ids("eos_token_id")))


def _attention(m: KeyReader) -> BiasAttentionConfig:
    heads = m.integer("heads", minimum=1)
    mask = _sub(m, "mask", required=False)
    cfg = BiasAttentionConfig(
        heads=heads, kv_heads=m.integer("kv_heads", default=heads, minimum=1), dim=m.integer("dim", minimum=1),
        vdim=m.integer("vdim", minimum=1), scale=m.real("scale"), bias_max=m.integer("bias_max", minimum=2),
        bias_rows=m.integer("bias_rows", default=0, minimum=0),
        window=mask.integer("size", minimum=1) if mask is not None else 0,
        keep_first=mask.integer("keep_first", default=0, minimum=0) if mask is not None else 0,
        v_mix=m.boolean("v_mix", default=False))
    if cfg.heads % cfg.kv_heads:
        raise ConfigError(f"{m.where}: heads ({cfg.heads}) must be a multiple of kv_heads ({cfg.kv_heads})")
    if max(cfg.dim, cfg.vdim) > MAX_HEAD_SIZE:
        raise ConfigError(f"{m.where}: dim ({cfg.dim}) and vdim ({cfg.vdim}) may not exceed the {MAX_HEAD_SIZE} elements "
                          f"the attention kernels take per key or value")
    return cfg


def _latent(m: KeyReader) -> LatentConfig:
    cfg = LatentConfig(heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1),
                       vdim=m.integer("vdim", minimum=1), kv_rank=m.integer("kv_rank", minimum=1),
                       q_rank=m.integer("q_rank", minimum=1), scale=m.real("scale"))
    if cfg.kv_rank > MAX_LATENT_ROW:
        raise ConfigError(f"{m.where}: kv_rank ({cfg.kv_rank}) exceeds the {MAX_LATENT_ROW} elements the attention "
                          f"kernels take per cached row")
    return cfg


def _mlp(ml: KeyReader):
    kind = ml.string("kind", default="dense")
    if kind == "dense":
        return DenseMlpConfig(ml.integer("ff", minimum=1), ml.real("limit", positive=True))
    if kind != "moe":
        raise ConfigError(f"{ml.where}: unknown feed-forward kind '{kind}' (known: dense, moe)")
    ex, ro = _sub(ml, "expert"), _sub(ml, "router")
    sh = _sub(ml, "shared", required=False)
    gr = _sub(ro, "groups", required=False)
    cfg = MoeMlpConfig(experts=ro.integer("experts", minimum=1), top=ro.integer("top", minimum=1),
                       groups=gr.integer("count", minimum=1) if gr is not None else 1,
                       keep_groups=gr.integer("keep", minimum=1) if gr is not None else 1,
                       ff=ex.integer("ff", minimum=1), limit=ex.real("limit", positive=True),
                       shared_ff=sh.integer("ff", minimum=1) if sh is not None else 0,
                       shared_limit=sh.real("limit", positive=True) if sh is not None else 0.0)
    if cfg.top > cfg.experts:
        raise ConfigError(f"{ro.where}: top ({cfg.top}) exceeds experts ({cfg.experts})")
    if cfg.experts % cfg.groups or cfg.keep_groups > cfg.groups:
        raise ConfigError(f"{ro.where}: {cfg.experts} experts do not form {cfg.groups} equal groups of which "
                          f"{cfg.keep_groups} are kept")
    if cfg.keep_groups * (cfg.experts // cfg.groups) < cfg.top:
        raise ConfigError(f"{ro.where}: {cfg.keep_groups} groups of {cfg.experts // cfg.groups} experts cannot give "
                          f"{cfg.top} choices")
    return cfg

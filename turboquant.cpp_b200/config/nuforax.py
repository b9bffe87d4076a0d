"""Typed configuration of the Nuforax decoder.

config.json of this design is nested: ``embedding`` (scale, optional pair table), ``norm`` (eps), ``vocab``,
``width`` and ``layers``, a list in which every entry names its mixer kind (``type``), the mixer's sizes
(``mixer``) and its feed-forward (``mlp``, or null for none).  The order and kinds of the layers are data: two
models of the design may differ in all of it.  Every size and constant is read here; the parts get them as
parameters.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .reader import ConfigError, KeyReader

ARCHITECTURE = "Nuforax"
# limits of the kernels the design's parts launch (csrc/latent_attention.cu LAT_MAX_ROW, csrc/ssm.cu SSM_MAX_STATE,
# SSM_MAX_TAPS), checked when the configuration is read
MAX_LATENT_ROW = 1024
MAX_SSM_STATE = 256
MAX_CONV_TAPS = 8


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
class RotaryScaling:
    """Frequencies of the slow pairs divided by `factor`, the fast pairs kept, a ramp between."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int              # query/key dimensions per head that are not rotated
    rot_dim: int          # rotated query dimensions per head = size of the key part all heads share
    vdim: int
    kv_rank: int
    scale: float
    window: int           # 0: every earlier position is seen
    rot_dims: int         # how many of the rot_dim dimensions turn
    rot_base: float
    rot_scaling: Optional[RotaryScaling]
    kv_from: Optional[int]


@dataclass(frozen=True)
class Mamba2Config:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class NuforaxLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseMlpConfig]


@dataclass(frozen=True)
class PairTableConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class NuforaxConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    pair_table: Optional[PairTableConfig]
    layers: Tuple[NuforaxLayer, ...]
    raw: Dict[str, Any]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = ARCHITECTURE
    # the design has no longest sequence of its own (angles are computed from the position, no table)
    max_position_embeddings: int = 1 << 30

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "NuforaxConfig":
        r = KeyReader(raw, where)
        width = r.integer("width", minimum=1)
        emb = _sub(r, "embedding", required=False)
        scale, pair = 1.0, None
        if emb is not None:
            scale = emb.real("scale", default=1.0)
            bi = _sub(emb, "bigram", required=False)
            if bi is not None:
                pair = PairTableConfig(bi.integer("buckets", minimum=1), bi.integer("mul_prev"), bi.integer("mul_cur"))
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
            if kind == "latent_attention":
                mixer = _latent(m, i)
            elif kind == "mamba2":
                mixer = _mamba2(m)
            else:
                raise ConfigError(f"{lw}: unknown layer type '{kind}' (known: latent_attention, mamba2)")
            ml = _sub(lr, "mlp", required=False)
            mlp = None
            if ml is not None:
                mk = ml.string("kind", default="dense")
                if mk != "dense":
                    raise ConfigError(f"{ml.where}: unknown feed-forward kind '{mk}' (known: dense)")
                mlp = DenseMlpConfig(ml.integer("ff", minimum=1))
            layers.append(NuforaxLayer(kind, mixer, mlp))
        for i, l in enumerate(layers):
            if l.type == "latent_attention" and l.mixer.kv_from is not None:
                j = l.mixer.kv_from
                if not 0 <= j < i or layers[j].type != "latent_attention" or layers[j].mixer.kv_from is not None:
                    raise ConfigError(f"{where}: layers[{i}]: mixer 'kv_from' names layer {j}, which must be an earlier "
                                      f"latent_attention layer with a projection of its own")
                a, b = l.mixer, layers[j].mixer
                if (a.kv_rank, a.rot_dim) != (b.kv_rank, b.rot_dim):
                    raise ConfigError(f"{where}: layers[{i}] and layer {j}, which its 'kv_from' names, differ in "
                                      f"kv_rank or rot_dim")
        return cls(vocab=r.integer("vocab", minimum=1), width=width, eps=_sub(r, "norm").real("eps", positive=True),
                   embedding_scale=scale, pair_table=pair, layers=tuple(layers), raw=dict(raw),
                   eos_token_ids=tuple(r.token_ids("eos_token_id")))


def _latent(m: KeyReader, index: int) -> LatentAttentionConfig:
    rot_dim = m.integer("rot_dim", minimum=0)
    rot = _sub(m, "rot", required=rot_dim > 0)
    rot_dims, base, scaling = 0, 10000.0, None
    if rot is not None:
        rot_dims = rot.integer("dims", default=rot_dim, minimum=0)
        base = rot.real("base", positive=True)
        sc = _sub(rot, "scaling", required=False)
        if sc is not None:
            scaling = RotaryScaling(sc.real("factor", positive=True), sc.real("original", positive=True),
                                    sc.real("fast", positive=True), sc.real("slow", positive=True))
    if rot_dims % 2 or rot_dims > rot_dim:
        raise ConfigError(f"{m.where}: rot.dims ({rot_dims}) must be even and at most rot_dim ({rot_dim})")
    mask = _sub(m, "mask", required=False)
    window = mask.integer("size", default=0, minimum=0) if mask is not None else 0
    cfg = LatentAttentionConfig(
        heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=0), rot_dim=rot_dim,
        vdim=m.integer("vdim", minimum=1), kv_rank=m.integer("kv_rank", minimum=1), scale=m.real("scale"),
        window=window, rot_dims=rot_dims, rot_base=base, rot_scaling=scaling,
        kv_from=m.integer("kv_from", minimum=0) if m.has("kv_from") else None)
    if cfg.dim + cfg.rot_dim < 1:
        raise ConfigError(f"{m.where}: a head needs at least one query dimension")
    if cfg.kv_rank + cfg.rot_dim > MAX_LATENT_ROW:
        raise ConfigError(f"{m.where}: kv_rank + rot_dim ({cfg.kv_rank + cfg.rot_dim}) exceeds the {MAX_LATENT_ROW} "
                          f"elements the attention kernels take per cached row")
    return cfg


def _mamba2(m: KeyReader) -> Mamba2Config:
    cfg = Mamba2Config(heads=m.integer("heads", minimum=1), vdim=m.integer("vdim", minimum=1),
                       state=m.integer("state", minimum=1), groups=m.integer("groups", default=1, minimum=1),
                       conv=m.integer("conv", minimum=1), norm_groups=m.integer("norm_groups", default=1, minimum=1))
    if cfg.heads % cfg.groups:
        raise ConfigError(f"{m.where}: heads ({cfg.heads}) must be a multiple of groups ({cfg.groups})")
    if (cfg.heads * cfg.vdim) % cfg.norm_groups:
        raise ConfigError(f"{m.where}: heads * vdim ({cfg.heads * cfg.vdim}) must be a multiple of norm_groups "
                          f"({cfg.norm_groups})")
    if cfg.state > MAX_SSM_STATE:
        raise ConfigError(f"{m.where}: state ({cfg.state}) exceeds the {MAX_SSM_STATE} the recurrence kernel takes")
    if cfg.conv > MAX_CONV_TAPS:
        raise ConfigError(f"{m.where}: conv ({cfg.conv}) exceeds the {MAX_CONV_TAPS} taps the convolution kernel takes")
    return cfg

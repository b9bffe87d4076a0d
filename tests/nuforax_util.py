"""Helpers of the Nuforax tests: small configurations, model folders with weights made for the test (written with
a few lines of file code of the tests' own), schedules run through the engine, comparison with the plain model."""
import json
import os
import struct

import numpy as np


def latent(heads=3, dim=16, rot_dim=8, vdim=12, kv_rank=40, window=24, scale=0.5, base=10000.0, dims=None,
           scaling=None, kv_from=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba(heads=4, vdim=12, state=16, groups=2, conv=3, norm_groups=2):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, vocab=97, width=48, eps=1e-5, scale=4.0, bigram=(53, 5, 3)):
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return {"architecture": "Nuforax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": emb,
            "layers": layers}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}

# Four configurations that differ in every size, in the order and kinds of layers, and in the options.
CONFIGS = {
    # attention first, a reader of its rows with a narrower window, a state-space layer with a feed-forward
    "a": config([layer("latent_attention", latent(scaling=YARN), ff=80),
                 layer("latent_attention", latent(window=9, scaling=YARN, kv_from=0), ff=None),
                 layer("mamba2", mamba(), ff=64),
                 layer("latent_attention", latent(heads=5, dim=8, rot_dim=16, vdim=8, kv_rank=24, window=0, dims=12, scale=0.3), ff=56)]),
    # state-space first; one group, one norm group, two taps; a reader with a WIDER window than its source; no
    # pair table, scale 1; sizes that are no multiples of 4 or 32
    "b": config([layer("mamba2", mamba(heads=3, vdim=20, state=33, groups=1, conv=2, norm_groups=1)),
                 layer("latent_attention", latent(heads=2, dim=10, rot_dim=6, vdim=7, kv_rank=30, window=5, scale=1.0), ff=40),
                 layer("latent_attention", latent(heads=2, dim=10, rot_dim=6, vdim=7, kv_rank=30, window=70, scale=1.0, kv_from=1), ff=40),
                 layer("mamba2", mamba(heads=4, vdim=8, state=8, groups=4, conv=1, norm_groups=4), ff=24)],
                vocab=61, width=40, eps=1e-6, scale=1.0, bigram=None),
    # wide rows (more than 256 elements), one head, windows wider than a page, four taps
    "c": config([layer("latent_attention", latent(heads=1, dim=32, rot_dim=32, vdim=32, kv_rank=288, window=130, scale=0.2,
                                                  base=500000.0, scaling={"factor": 8.0, "original": 32, "fast": 16.0, "slow": 2.0}), ff=96),
                 layer("mamba2", mamba(heads=2, vdim=40, state=64, groups=1, conv=4, norm_groups=2)),
                 layer("latent_attention", latent(heads=1, dim=32, rot_dim=32, vdim=32, kv_rank=288, window=65, scale=0.2,
                                                  base=500000.0, scaling={"factor": 8.0, "original": 32, "fast": 16.0, "slow": 2.0}, kv_from=0))],
                vocab=128, width=64, bigram=(31, 1, 1)),
    # a latent of 128 elements (in bfloat16 the tensor-core form with eight warps a block), six heads, a reader with
    # a wider window behind a state-space layer with as many groups as heads
    "d": config([layer("latent_attention", latent(heads=6, dim=24, rot_dim=32, vdim=20, kv_rank=128, window=50, scale=0.25,
                                                  scaling=YARN), ff=100),
                 layer("mamba2", mamba(heads=4, vdim=16, state=32, groups=4, conv=4, norm_groups=1), ff=48),
                 layer("latent_attention", latent(heads=6, dim=24, rot_dim=32, vdim=20, kv_rank=128, window=90, scale=0.25,
                                                  scaling=YARN, kv_from=0))],
                vocab=111, width=72, bigram=(29, 3, 11)),
}


def tensor_shapes(cfg):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    if cfg["embedding"].get("bigram"):
        out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        out[p + "norm1"] = (W,)
        if l["type"] == "latent_attention":
            H = m["heads"]
            out[p + "mix.q"] = (H * (m["dim"] + m["rot_dim"]), W)
            if m.get("kv_from") is None:
                out[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], W)
                out[p + "mix.dkv.norm"] = (m["kv_rank"],)
            out[p + "mix.uk"] = (H * m["dim"], m["kv_rank"])
            out[p + "mix.uv"] = (H * m["vdim"], m["kv_rank"])
            out[p + "mix.sink"] = (H,)
            out[p + "mix.o"] = (W, H * m["vdim"])
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + "mix.in"] = (2 * inner + 2 * gn + m["heads"], W)
            out[p + "mix.conv"] = (inner + 2 * gn, m["conv"])
            out[p + "mix.conv.b"] = (inner + 2 * gn,)
            for n in ("dt_bias", "A_log", "D"):
                out[p + "mix." + n] = (m["heads"],)
            out[p + "mix.norm"] = (inner,)
            out[p + "mix.o"] = (W, inner)
        if l["mlp"] is not None:
            out[p + "norm2"] = (W,)
            out[p + "mlp.up"] = (l["mlp"]["ff"], W)
            out[p + "mlp.down"] = (W, l["mlp"]["ff"])
    return out


def make_weights(cfg, seed, sharp=1.0):
    """Random weights with magnitudes that keep every mechanism visible: projections of unit gain, norms around 1,
    sinks and decays of order 1.  `sharp` scales the query projections (peaked attention)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith("norm1") or name.endswith("norm2") or leaf == "norm" or name == "final.norm":
            w = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf in ("sink", "dt_bias", "A_log", "D", "b"):
            w = rng.standard_normal(shape)
        elif leaf == "conv":
            w = rng.standard_normal(shape) * 0.5
        elif name in ("embed", "bigram"):
            w = rng.standard_normal(shape)
        else:
            w = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf == "q":
                w = w * sharp
        out[name] = w.astype(np.float32)
    return out


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_folder(folder, cfg, weights):
    """config.json and model.safetensors (bfloat16) of a configuration and its weights."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, w in weights.items():
        b = to_bf16_bits(w).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(w.shape), "data_offsets": [at, at + len(b)]}
        blobs.append(b)
        at += len(b)
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))
    return folder


def run_steps(engine, steps, ends):
    """steps: lists of (request, tokens, want); ends: {step index: [requests that end]}.  Returns
    {request: {position: logits row}}."""
    import turboquant_cpp_b200 as tq
    live, pos, logits = {}, {}, {}
    for si, step in enumerate(steps):
        entries = []
        for rid, toks, want in step:
            if rid not in live:
                live[rid] = engine.open()
                pos[rid] = 0
            entries.append(tq.StepEntry(live[rid], list(toks), list(want)))
        out = engine.step(entries)
        out = None if out is None else out.float().cpu().numpy()
        row = 0
        for rid, toks, want in step:
            for w in want:
                logits.setdefault(rid, {})[pos[rid] + w] = out[row]
                row += 1
            pos[rid] += len(toks)
        for rid in ends.get(si, []):
            engine.close(live.pop(rid))
    engine.check_kernels()
    assert not live
    return logits


def spread_error(got, ref):
    """Per row: root mean square of the difference with its mean taken off, relative to the reference's spread."""
    d = np.asarray(got, dtype=np.float64) - ref
    d = d - d.mean(axis=-1, keepdims=True)
    return np.sqrt((d * d).mean(axis=-1)) / np.sqrt(((ref - ref.mean(axis=-1, keepdims=True)) ** 2).mean())


# float32: sums of a few thousand terms in another order than float64.  bfloat16: the plain model rounds nothing, so
# the engine's roundings of activations (2^-9 each) show, amplified where a peaked softmax turns a small change of a
# score into a large change of a weight: most positions stay within a few per cent of the logits' spread, single
# ones reach a tenth of it.  A fault of the logic (a window one token off, a lost state) moves float32 logits by
# 1e-2 and more and is caught there; the bfloat16 runs are about that path's own kernels, where a fault is of order 1.
# Where a sub-layer's output nearly cancels, the norm on it enlarges the rounding before it: single positions of
# single configurations reach 1e-4 in float32 and half the spread in bfloat16, by both attention paths alike.
TOL = {"float32": (2e-5, 3e-4), "bfloat16": (4e-2, 0.6)}      # (nine positions in ten, every position)


def assert_close(got_rows, ref, dtype, what):
    """got_rows {position: row} against the plain logits ref [T, vocab] at those positions."""
    ps = sorted(got_rows)
    e = spread_error(np.stack([got_rows[p] for p in ps]), ref[ps])
    most, every = TOL[dtype]
    assert np.all(np.isfinite(e)), f"{what}: not finite"
    assert e.max() < every, f"{what}: position {ps[int(e.argmax())]} differs by {e.max():.3e} (tolerance {every:.0e})"
    assert np.quantile(e, 0.9) < most, f"{what}: a tenth of the positions differ by more than {np.quantile(e, 0.9):.3e}"
    return float(e.max())

"""A plain, slow implementation of the Nuforax decoder, one function per mechanism, in float64 on the CPU.

It reads a model folder (config.json, model.safetensors) with its own few lines of file parsing and shares no code
with the library.  Every function takes whole sequences and loops over positions where the definition does; nothing
is cached, so the logits of a position are those of the definition itself.

Notation: h is a sub-layer's input [T, width]; rms(v) = v / sqrt(mean(v^2) + eps).
"""
import json
import math
import os
import struct

import numpy as np

F = np.float64


# ---- file reading ---------------------------------------------------------------------------------------------
def read_safetensors(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = data[a:b]
        if meta["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(F)
        elif meta["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F)
        elif meta["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"dtype {meta['dtype']} of '{name}'")
        out[name] = arr.reshape(meta["shape"])
    return out


# ---- small functions --------------------------------------------------------------------------------------------
def rms(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def silu(v):
    return v / (1.0 + np.exp(-v))


def softplus(v):
    return np.logaddexp(0.0, v)


def relu_squared(v):
    return np.maximum(v, 0.0) ** 2


# ---- embedding ------------------------------------------------------------------------------------------------
def embed_tokens(tokens, table, scale, bigram=None, buckets=0, mul_prev=0, mul_cur=0):
    """Row of the table times `scale`, plus a row of the pair table chosen by (previous, current) token; a
    sequence's first token takes the table's last row."""
    x = table[np.asarray(tokens)] * scale
    if bigram is not None:
        for t, tok in enumerate(tokens):
            row = buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets
            x[t] = x[t] + bigram[row]
    return x


# ---- rotation -------------------------------------------------------------------------------------------------
def rotary_frequencies(dims, base, scaling=None):
    """(frequency per pair, factor on cos and sin).  With `scaling` (factor, original, fast, slow) the slow pairs'
    frequencies are divided by factor, the fast ones kept, with a linear ramp between the two pair indices where a
    period of the original context makes `fast` resp. `slow` turns."""
    i = np.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(v, positions, freq, mag):
    """v [T, ..., d]: pairs (2i, 2i+1) of the first 2*len(freq) dimensions turn by position * freq_i; cos and sin
    carry the factor `mag`."""
    out = v.copy()
    n = len(freq)
    for t, p in enumerate(positions):
        a = p * freq
        c, s = np.cos(a) * mag, np.sin(a) * mag
        u, w = v[t, ..., 0:2 * n:2], v[t, ..., 1:2 * n:2]
        out[t, ..., 0:2 * n:2] = u * c - w * s
        out[t, ..., 1:2 * n:2] = w * c + u * s
    return out


# ---- latent attention -----------------------------------------------------------------------------------------
def latent_and_shared_key(h, w_dkv, w_norm, kv_rank, eps, freq, mag):
    """The latent c (normed) and the rotated key part every head shares, for all positions of a sequence."""
    d = h @ w_dkv.T
    c = rms(d[:, :kv_rank], eps) * w_norm
    kr = rotate_interleaved(d[:, kv_rank:], range(h.shape[0]), freq, mag)
    return c, kr


def latent_attention(h, c, kr, w_q, w_uk, w_uv, w_o, sink, heads, dim, rot_dim, vdim, scale, window, freq, mag):
    """Scores of head a: (q_plain . (W_uk c_j) + q_turned . kr_j) * scale over the keys j the window allows; the
    softmax's denominator also holds exp(sink_a)."""
    T = h.shape[0]
    q = (h @ w_q.T).reshape(T, heads, dim + rot_dim)
    q_plain = q[:, :, :dim]
    q_turn = rotate_interleaved(q[:, :, dim:], range(T), freq, mag)
    k_plain = (c @ w_uk.T).reshape(T, heads, dim)
    v = (c @ w_uv.T).reshape(T, heads, vdim)
    out = np.zeros((T, heads, vdim), dtype=F)
    for i in range(T):
        j0 = 0 if window <= 0 else max(0, i - window + 1)
        for a in range(heads):
            s = (k_plain[j0:i + 1, a] @ q_plain[i, a] + kr[j0:i + 1] @ q_turn[i, a]) * scale
            m = max(s.max(), sink[a])
            e = np.exp(s - m)
            out[i, a] = (e @ v[j0:i + 1, a]) / (e.sum() + math.exp(sink[a] - m))
    return out.reshape(T, heads * vdim) @ w_o.T


# ---- state-space mixer ----------------------------------------------------------------------------------------
def causal_conv(u, w, b):
    """u [T, C]; w [C, taps] with the last column on the current position; zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), u], axis=0)
    out = np.zeros_like(u)
    for t in range(T):
        out[t] = (padded[t:t + taps] * w.T).sum(axis=0) + b
    return out


def state_space_scan(x, B, C, dt, a_log, d_skip, heads, vdim, state, groups):
    """Per head a: S <- exp(-exp(a_log_a) dt) S + dt B x^T (S is [state, vdim]); y = S^T C + d_skip_a x."""
    T = x.shape[0]
    x = x.reshape(T, heads, vdim)
    B, C = B.reshape(T, groups, state), C.reshape(T, groups, state)
    y = np.zeros((T, heads, vdim), dtype=F)
    per = heads // groups
    for a in range(heads):
        g = a // per
        S = np.zeros((state, vdim), dtype=F)
        for t in range(T):
            S = math.exp(-math.exp(a_log[a]) * dt[t, a]) * S + dt[t, a] * np.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ C[t, g] + d_skip[a] * x[t, a]
    return y.reshape(T, heads * vdim)


def mamba2_mixer(h, w_in, w_conv, b_conv, dt_bias, a_log, d_skip, w_norm, w_o, heads, vdim, state, groups,
                 norm_groups, eps):
    inner, gn = heads * vdim, groups * state
    p = h @ w_in.T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * gn], p[:, 2 * inner + 2 * gn:]
    xbc = silu(causal_conv(xbc, w_conv, b_conv))
    x, B, C = xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:]
    dt = softplus(dt + dt_bias)
    y = state_space_scan(x, B, C, dt, a_log, d_skip, heads, vdim, state, groups) * silu(z)
    T = h.shape[0]
    y = rms(y.reshape(T, norm_groups, inner // norm_groups), eps).reshape(T, inner) * w_norm
    return y @ w_o.T


# ---- feed-forward ---------------------------------------------------------------------------------------------
def dense_feed_forward(h, w_up, w_down):
    return relu_squared(h @ w_up.T) @ w_down.T


# ---- the model ------------------------------------------------------------------------------------------------
class PlainNuforax:
    def __init__(self, folder):
        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_safetensors(os.path.join(folder, "model.safetensors"))

    def forward(self, tokens, layers_out=None):
        """Logits [T, vocab] of one sequence from its first token; `layers_out`: a list that receives the residual
        stream after every layer."""
        cfg, w = self.cfg, self.w
        eps = float(cfg["norm"]["eps"])
        emb = cfg["embedding"]
        bi = emb.get("bigram")
        x = embed_tokens(list(tokens), w["embed"], float(emb.get("scale", 1.0)),
                         w["bigram"] if bi else None, *( (bi["buckets"], bi["mul_prev"], bi["mul_cur"]) if bi else ()))
        kept = {}
        for l, layer in enumerate(cfg["layers"]):
            p, m = f"l{l}.", layer["mixer"]
            if layer["type"] == "latent_attention":
                rot = m["rot"]
                freq, mag = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
                if m.get("kv_from") is None:
                    kept[l] = latent_and_shared_key(x, w[p + "mix.dkv"], w[p + "mix.dkv.norm"], m["kv_rank"], eps, freq, mag)
                c, kr = kept[l if m.get("kv_from") is None else m["kv_from"]]
                window = int((m.get("mask") or {}).get("size", 0))
                y = latent_attention(x, c, kr, w[p + "mix.q"], w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.o"],
                                     w[p + "mix.sink"], m["heads"], m["dim"], m["rot_dim"], m["vdim"], float(m["scale"]),
                                     window, freq, mag)
            elif layer["type"] == "mamba2":
                y = mamba2_mixer(x, w[p + "mix.in"], w[p + "mix.conv"], w[p + "mix.conv.b"], w[p + "mix.dt_bias"],
                                 w[p + "mix.A_log"], w[p + "mix.D"], w[p + "mix.norm"], w[p + "mix.o"], m["heads"],
                                 m["vdim"], m["state"], m["groups"], m["norm_groups"], eps)
            else:
                raise ValueError(f"layer type '{layer['type']}'")
            x = x + rms(y, eps) * w[p + "norm1"]
            if layer.get("mlp") is not None:
                y = dense_feed_forward(x, w[p + "mlp.up"], w[p + "mlp.down"])
                x = x + rms(y, eps) * w[p + "norm2"]
            if layers_out is not None:
                layers_out.append(x.copy())
        return (rms(x, eps) * w["final.norm"]) @ w["embed"].T

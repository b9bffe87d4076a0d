"""A plain, slow implementation of the Lumevik decoder, one function per mechanism, in float64 on the CPU.

It reads a model folder (config.json, model.safetensors) with its own few lines of file parsing and shares no code
with the library.  Every function takes a whole sequence and loops over positions where the definition does; nothing
is cached, so the logits of a position are those of the definition itself.

Notation: h is a sub-layer's input [T, width]; unit(v) = v / sqrt(mean(v^2) + eps); positions start at 0.
"""
import json
import math
import os
import struct

import numpy as np

F = np.float64
GLU_SLOPE = 1.702          # the gate's sigmoid is taken of GLU_SLOPE * gate
WEIGHT_FLOOR = 1e-20       # added to the sum of the chosen experts' scores before the division


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
def unit(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def norm_around_zero(v, w, eps):
    """The layers' norm: the stored weight is the distance from one."""
    return unit(v, eps) * (1.0 + w)


def norm_plain(v, w, eps):
    return unit(v, eps) * w


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def capped_glu(gate, up, limit):
    """gate capped from above, up capped on both sides; gate * sigmoid(slope * gate) * (up + 1)."""
    g = np.minimum(gate, limit)
    u = np.clip(up, -limit, limit)
    return g * sigmoid(GLU_SLOPE * g) * (u + 1.0)


# ---- distance bias ------------------------------------------------------------------------------------------------
def distance_bucket(n, rows, far):
    """Row of the bias table for distance n >= 0: the first half of the rows one distance each, the second half
    logarithmic steps up to distance `far`, everything beyond in the last row."""
    half = rows // 2
    if n < half:
        return n
    step = math.floor(math.log(n / half) / math.log(far / half) * (rows - half))
    return min(rows - 1, half + step)


def visible(i, j, mask):
    """Whether position i sees position j: the last mask.size positions and the first mask.keep_first; every
    earlier position if there is no mask."""
    if not mask:
        return j <= i
    return j <= i and (i - j < mask["size"] or j < mask.get("keep_first", 0))


# ---- mixers -----------------------------------------------------------------------------------------------------
def biased_attention_core(q, k, v, rel, m):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of one sequence; rel [rows, H] or None.  Per query and head: scores with
    the distance bias over the visible positions, a softmax whose denominator counts one more (a key of score 0
    without a value), the weighted sum of the values."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    out = np.zeros((T, H, dv), dtype=F)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, m.get("mask"))]
        for a in range(H):
            g = a // (H // G)
            s = np.array([q[i, a] @ k[j, g] * m["scale"]
                          + (rel[distance_bucket(i - j, rel.shape[0], m["bias_max"]), a] if rel is not None else 0.0) for j in js])
            e = np.exp(s)
            p = e / (1.0 + e.sum())
            out[i, a] = sum(p[n] * v[j, g] for n, j in enumerate(js))
    return out


def mix_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def biased_attention(h, w, m, v_first=None):
    """Grouped-query attention without rotation: projections, values mixed with those of the first such layer,
    the core above, the output projection.  Returns (output, the values as they would be cached)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = (h @ w["v"].T).reshape(T, G, dv)
    if m.get("v_mix") and v_first is not None:
        v = mix_values(v, v_first, float(w["vmix"]))
    out = biased_attention_core(q, k, v, w["rel"], m)
    return out.reshape(T, H * dv) @ w["o"].T, v


def latent_attention(h, w, m, eps):
    """Queries through a normed latent; keys and values expanded per head from one normed latent per position;
    causal, ordinary softmax, no positions."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, d)
    c = norm_plain(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv), dtype=F)
    for i in range(T):
        for a in range(H):
            s = k[:i + 1, a] @ q[i, a] * m["scale"]
            e = np.exp(s - s.max())
            out[i, a] = (e / e.sum()) @ v[:i + 1, a]
    return out.reshape(T, H * dv) @ w["o"].T


# ---- feed-forwards ------------------------------------------------------------------------------------------------
def dense_ff(h, w, limit):
    return capped_glu(h @ w["gate"].T, h @ w["up"].T, limit) @ w["down"].T


def route(h, w, r, forced=None, margins=None):
    """Per token: (chosen experts, their weights).  Scores are a softmax over all experts; the choice looks at
    score + correction, only inside the groups whose best such value is among the `keep` largest; the weights are
    the chosen experts' plain scores over their sum.  forced [T, top]: these experts instead of the choice (their
    weights are still this model's); margins: receives per token the smallest gap that decided a choice (between
    the last kept and the first dropped group, and between the last chosen and the first dropped expert)."""
    z = h @ w["router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    E, top = r["experts"], r["top"]
    chosen, weights = [], []
    for t in range(h.shape[0]):
        c = s[t] + w["correction"]
        allowed = np.ones(E, dtype=bool)
        groups = r.get("groups")
        gap = np.inf
        if groups:
            n, per = groups["count"], E // groups["count"]
            best = np.array([c[g * per:(g + 1) * per].max() for g in range(n)])
            order = np.argsort(-best, kind="stable")
            kept = order[:groups["keep"]]
            if groups["keep"] < n:
                gap = best[order[groups["keep"] - 1]] - best[order[groups["keep"]]]
            allowed[:] = False
            for g in kept:
                allowed[g * per:(g + 1) * per] = True
        c = np.where(allowed, c, -np.inf)
        order = np.argsort(-c, kind="stable")
        ids = order[:top]
        if top < E and np.isfinite(c[order[top]]):
            gap = min(gap, c[order[top - 1]] - c[order[top]])
        if margins is not None:
            margins.append(gap)
        if forced is not None:
            ids = np.asarray(forced[t])
        chosen.append(ids)
        weights.append(s[t, ids] / (s[t, ids].sum() + WEIGHT_FLOOR))
    return np.array(chosen), np.array(weights)


def expert_ff(h, tensors, prefix, limit):
    w = {n: tensors[prefix + n] for n in ("gate", "up", "down")}
    return dense_ff(h, w, limit)


def moe_ff(h, tensors, prefix, mlp, forced=None, margins=None):
    r = mlp["router"]
    w = {"router": tensors[prefix + "router"], "correction": tensors[prefix + "correction"]}
    ids, wts = route(h, w, r, forced, margins)
    y = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], wts[t]):
            y[t] += a * expert_ff(h[t:t + 1], tensors, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        gate = sigmoid(h @ tensors[prefix + "shared.sg"].T)              # one number per token
        y += gate * expert_ff(h, tensors, prefix + "shared.", mlp["shared"]["limit"])
    return y, ids, wts


# ---- the model --------------------------------------------------------------------------------------------------
class PlainLumevik:
    def __init__(self, folder):
        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        self.t = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.eps = self.cfg["norm"]["eps"]

    def mixer_weights(self, i):
        p = f"l{i}.mix."
        return {n[len(p):]: a for n, a in self.t.items() if n.startswith(p)}

    def forward(self, tokens, streams=None, routing=None, forced=None):
        """Logits [T, vocab] of one sequence; `streams` collects the residual stream after every layer, `routing`
        (experts, weights, margins) of every routed layer, in layer order; forced: per routed layer, in that order,
        the experts [T, top] to take instead of the model's own choice (None, or a shorter list: the layers without
        an entry choose for themselves)."""
        t, cfg, eps = self.t, self.cfg, self.eps
        x = t["embed"][np.asarray(tokens)].astype(F)
        v_first = None
        n_routed = 0
        for i, layer in enumerate(cfg["layers"]):
            p, m = f"l{i}.", layer["mixer"]
            h = norm_around_zero(x, t[p + "norm1"], eps)
            if layer["type"] == "attention":
                y, v = biased_attention(h, self.mixer_weights(i), m, v_first)
                if m.get("v_mix") and v_first is None:
                    v_first = v
            elif layer["type"] == "latent_attention":
                y = latent_attention(h, self.mixer_weights(i), m, eps)
            else:
                raise ValueError(layer["type"])
            x = x + y
            mlp = layer.get("mlp")
            if mlp:
                h = norm_around_zero(x, t[p + "norm2"], eps)
                if mlp["kind"] == "dense":
                    y = dense_ff(h, {n: t[p + "mlp." + n] for n in ("gate", "up", "down")}, mlp["limit"])
                else:
                    margins = []
                    y, ids, wts = moe_ff(h, t, p + "mlp.", mlp, None if forced is None or n_routed >= len(forced) else forced[n_routed], margins)
                    n_routed += 1
                    if routing is not None:
                        routing.append((ids, wts, np.array(margins)))
                x = x + y
            if streams is not None:
                streams.append(x.copy())
        return norm_around_zero(x, t["final.norm"], eps) @ t["head"].T

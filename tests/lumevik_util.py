"""Helpers of the Lumevik tests: small configurations, model folders with weights made for the test, and the
comparison with the plain model, which takes the engine's expert choices where its own were a near-tie."""
import copy

import numpy as np

from nuforax_util import assert_close, run_steps, spread_error, write_folder      # noqa: F401  (file writing, schedules)


def attention(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.25, size=24, keep_first=3, bias_max=40, rows=12, v_mix=True):
    """rows: rows of the layer's bias table; it is no key of the design's config.json (the tensor's shape says it)
    and is taken out before the file is written."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max,
         "v_mix": v_mix, "_rows": rows}
    if size:                  # size 0: no mask, every earlier position is seen
        m["mask"] = {"size": size, "keep_first": keep_first}
    return m


def latent(heads=3, dim=16, vdim=12, kv_rank=40, q_rank=24, scale=0.3):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}


def dense(ff=48, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=8, top=3, groups=(4, 2), ff=16, limit=1.2, shared=(24, 0.8)):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=97, width=48, eps=1e-5):
    return {"architecture": "Lumevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# Configurations that differ in every size, in the order and kinds of layers, and in the options.
CONFIGS = {
    # attention first (it provides the mixed values), routed experts, a latent layer, a second mixing layer
    "a": config([layer("attention", attention(), moe()),
                 layer("latent_attention", latent(), dense()),
                 layer("attention", attention(heads=6, kv_heads=2, dim=8, vdim=8, size=9, keep_first=0, bias_max=17, rows=8), None),
                 layer("attention", attention(heads=2, kv_heads=2, dim=24, vdim=8, size=70, keep_first=66, bias_max=100, rows=20), dense(ff=20, limit=0.7))]),
    # latent first; sizes the tensor-core kernel for runs takes (32 / 64), windows wider than a page, one kv head,
    # a layer that does not mix between two that do, groups of one expert, no shared expert
    "b": config([layer("latent_attention", latent(heads=2, dim=8, vdim=20, kv_rank=32, q_rank=16, scale=0.5), moe(experts=6, top=3, groups=(6, 4), ff=24, limit=2.0, shared=None)),
                 layer("attention", attention(heads=4, kv_heads=1, dim=32, vdim=64, scale=0.2, size=130, keep_first=65, bias_max=300, rows=32), dense()),
                 layer("attention", attention(heads=2, kv_heads=1, dim=64, vdim=32, scale=0.15, size=64, keep_first=1, bias_max=64, rows=16, v_mix=False), None),
                 layer("attention", attention(heads=2, kv_heads=1, dim=32, vdim=64, scale=0.2, size=33, keep_first=64, bias_max=90, rows=10), moe(experts=4, top=1, groups=None, ff=8, limit=0.5, shared=(8, 3.0)))],
                vocab=61, width=40, eps=1e-6),
    # no window at all (size 0), every query head its own kv head, one group, as many experts chosen as there are
    "c": config([layer("attention", attention(heads=3, kv_heads=3, dim=16, vdim=16, size=0, keep_first=0, bias_max=500, rows=64, v_mix=False), moe(experts=3, top=3, groups=(1, 1), ff=12, limit=1.0, shared=(16, 1.0))),
                 layer("latent_attention", latent(heads=1, dim=32, vdim=32, kv_rank=288, q_rank=96, scale=0.2), None)],
                vocab=128, width=64),
}


def tensor_shapes(cfg):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        out[p + "norm1"] = (W,)
        if l["type"] == "attention":
            H, G = m["heads"], m["kv_heads"]
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = (H * m["dim"], W), (G * m["dim"], W), (G * m["vdim"], W)
            out[p + "mix.rel"] = (m["_rows"], H)
            if m["v_mix"]:
                out[p + "mix.vmix"] = ()
            out[p + "mix.o"] = (W, H * m["vdim"])
        else:
            H = m["heads"]
            out[p + "mix.dq"], out[p + "mix.dq.norm"] = (m["q_rank"], W), (m["q_rank"],)
            out[p + "mix.uq"] = (H * m["dim"], m["q_rank"])
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = (m["kv_rank"], W), (m["kv_rank"],)
            out[p + "mix.uk"], out[p + "mix.uv"] = (H * m["dim"], m["kv_rank"]), (H * m["vdim"], m["kv_rank"])
            out[p + "mix.o"] = (W, H * m["vdim"])
        mlp = l["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        q = p + "mlp."
        if mlp["kind"] == "dense":
            out[q + "gate"], out[q + "up"], out[q + "down"] = (mlp["ff"], W), (mlp["ff"], W), (W, mlp["ff"])
            continue
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        for e in range(E):
            out[f"{q}e{e}.gate"], out[f"{q}e{e}.up"], out[f"{q}e{e}.down"] = (ff, W), (ff, W), (W, ff)
        out[q + "router"], out[q + "correction"] = (E, W), (E,)
        if mlp.get("shared"):
            s = mlp["shared"]["ff"]
            out[q + "shared.gate"], out[q + "shared.up"], out[q + "shared.down"] = (s, W), (s, W), (W, s)
            out[q + "shared.sg"] = (1, W)
    return out


def make_weights(cfg, seed, sharp=3.0):
    """Random weights with magnitudes that keep every mechanism visible: projections of unit gain, norm weights
    around zero, biases of order one, gates and ups that reach their caps.  `sharp` scales the query projections, so
    that the softmax is peaked and a single key that is wrongly seen or missed moves the output."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            w = 0.3 * rng.standard_normal(shape)                  # stored around zero
        elif leaf == "norm":
            w = 1.0 + 0.2 * rng.standard_normal(shape)            # the latents' norms: plain weights
        elif leaf == "rel":
            w = 1.5 * rng.standard_normal(shape)
        elif leaf == "vmix":
            w = np.asarray(rng.uniform(0.3, 0.7))
        elif leaf == "correction":
            w = 0.2 * rng.standard_normal(shape)
        elif name == "embed":
            w = rng.standard_normal(shape)
        else:
            w = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf in ("q", "uq"):
                w = w * sharp
            if leaf in ("gate", "up", "router"):
                w = w * 2.0
        out[name] = np.asarray(w, dtype=np.float32)
    return out


def write_model(folder, cfg, weights):
    """The folder as the design stores it: the helper's private keys are not part of config.json."""
    clean = copy.deepcopy(cfg)
    for l in clean["layers"]:
        l["mixer"].pop("_rows", None)
    return write_folder(folder, clean, weights)


def run_steps_with_routing(engine, steps, ends, leave_open=False):
    """Like run_steps, and per request the experts the engine chose: {request: [per routed layer {position: ids}]}.
    leave_open: requests that no step ends stay live (the caller closes them)."""
    import turboquant_cpp_b200 as tq
    live, pos, logits, routing = {}, {}, {}, {}
    for si, step in enumerate(steps):
        entries = []
        for rid, toks, want in step:
            if rid not in live:
                live[rid] = engine.open()
                pos[rid] = 0
            entries.append(tq.StepEntry(live[rid], list(toks), list(want)))
        engine.debug = {}
        out = engine.step(entries)
        ids = [a.cpu().numpy() for a in engine.debug.get("router_ids", [])]
        engine.debug = None
        out = None if out is None else out.float().cpu().numpy()
        row = t0 = 0
        for rid, toks, want in step:
            for w in want:
                logits.setdefault(rid, {})[pos[rid] + w] = out[row]
                row += 1
            per_layer = routing.setdefault(rid, [dict() for _ in ids])
            for li, a in enumerate(ids):
                for j in range(len(toks)):
                    per_layer[li][pos[rid] + j] = a[t0 + j]
            pos[rid] += len(toks)
            t0 += len(toks)
        for rid in ends.get(si, []):
            engine.close(live.pop(rid))
    engine.check_kernels()
    assert leave_open or not live
    return logits, routing


# below this gap between the last chosen and the first dropped score another choice is as right (the scores are
# probabilities: of order 1 / experts)
FLIP_MARGIN = {"float32": 1e-5, "bfloat16": 4e-2}


def check_against_plain(plain, tokens, logits, routing, dtype, what):
    """The engine's logits {position: row} against the plain model.  Routed layer by routed layer: where the engine
    chose other experts than the plain model (run with the engine's choices in the layers before), the plain
    model's own margin there must be tiny and such places rare; the logits are then held against the plain model
    run with the engine's choices."""
    n = len(tokens)
    rec = []
    ref = plain.forward(list(tokens), routing=rec)
    flips, forced, li = 0, [], 0
    while li < len(rec):
        ids, _, margins = rec[li]
        got = routing[li]
        assert sorted(got) == list(range(n)), f"{what}: routed layer {li} did not see every position exactly once"
        eng = np.stack([got[p] for p in range(n)])
        differ = np.nonzero(np.any(np.sort(ids, axis=1) != np.sort(eng, axis=1), axis=1))[0]
        for p in differ:
            assert margins[p] < FLIP_MARGIN[dtype], (f"{what}: routed layer {li} position {p}: engine chose {eng[p].tolist()}, "
                                                     f"plain {ids[p].tolist()} with margin {margins[p]:.3e}")
        flips += len(differ)
        forced.append(eng)
        li += 1
        if len(differ) and li < len(rec):         # the later layers see what the engine's choice made of this one
            rec = []
            ref = plain.forward(list(tokens), routing=rec, forced=forced)
    assert flips <= max(2, n * max(1, len(rec)) // 20), f"{what}: {flips} expert choices differ"
    if flips:
        ref = plain.forward(list(tokens), forced=forced)
    return assert_close(logits, ref, dtype, what)

"""The Lumevik decoder in the engine against the plain implementation (tests/plain/lumevik_plain.py): whole prompts,
decoding token by token, prompts in portions, batches of unequal requests, pages and slots used again, the edges of
windows and of the kept first positions, far keys, other sizes, generation through the entry point, and trace
replay as a user runs it."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT
from lumevik_util import (CONFIGS, assert_close, attention, check_against_plain, config, dense, latent, layer,
                          make_weights, moe, run_steps, run_steps_with_routing, write_model)
from plain.lumevik_plain import PlainLumevik
from replay_util import batched, whole, with_tail

pytestmark = pytest.mark.gpu

_plain = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        out[name] = write_model(str(tmp_path_factory.mktemp(f"lumevik_{name}")), cfg, make_weights(cfg, 200 + i))
    return out


def plain_model(folder):
    if folder not in _plain:
        _plain[folder] = PlainLumevik(folder)
    return _plain[folder]


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def engine_for(folder, dtype, max_tokens=1024, **kw):
    import turboquant_cpp_b200 as tq
    return tq.Engine(tq.load_model(folder, dtype), max_tokens=max_tokens, record_routing=True, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_whole_prompts_decoding_and_batches_agree_with_plain(folders, name, dtype):
    cfg, folder = CONFIGS[name], folders[name]
    reqs = {"r0": tokens_for(cfg, 150, 1), "r1": tokens_for(cfg, 1, 2), "r2": tokens_for(cfg, 77, 3), "r3": tokens_for(cfg, 200, 4)}
    eng = engine_for(folder, dtype, max_tokens=64 * 12)
    try:
        modes = {}
        steps, ends = [], {}
        for rid, toks in reqs.items():                        # each alone and whole, one after another
            s, e = whole(rid, toks)
            ends.update({k + len(steps): v for k, v in e.items()})
            steps += s
        modes["whole"] = run_steps_with_routing(eng, steps, ends)
        steps, ends = [], {}
        for rid, toks in reqs.items():                        # the last 80 tokens one by one (windows pass over decoded tokens)
            s, e = with_tail(rid, toks, 80)
            ends.update({k + len(steps): v for k, v in e.items()})
            steps += s
        modes["tail"] = run_steps_with_routing(eng, steps, ends)
        s, e = batched(reqs, {"r0": 100, "r1": 1, "r2": 64, "r3": 129})     # unequal prompts, then decoded together
        modes["batched"] = run_steps_with_routing(eng, s, e)
        eng.cache.book.check_invariants()
        assert eng.cache.book.slots.n_held == 0 and all(p.n_held == 0 for p in eng.cache.book.pools)
        for rid, toks in reqs.items():
            for mode, (got, routing) in modes.items():
                assert sorted(got[rid]) == list(range(len(toks))), f"{mode} {rid}"
                check_against_plain(plain_model(folder), toks, got[rid], routing[rid], dtype, f"{name} {mode} {rid}")
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,sizes", [("a", [2, 3, 64, 1, 2, 7, 50, 17]), ("b", [63, 2, 2, 65, 5, 40, 16]), ("c", [5, 128, 2, 30])])
def test_prompts_in_portions(folders, name, sizes, dtype):
    """A prompt cut into portions, down to two tokens, beside a request that goes on token by token."""
    cfg, folder = CONFIGS[name], folders[name]
    toks, other = tokens_for(cfg, sum(sizes), 7), tokens_for(cfg, len(sizes) + 20, 8)
    eng = engine_for(folder, dtype)
    try:
        steps, at = [], 0
        for i, n in enumerate(sizes):
            step = [("p", toks[at:at + n], list(range(n)))]
            if i == 0:
                step.append(("o", other[:21], list(range(21))))
            else:
                step.append(("o", [other[20 + i]], [0]))
            steps.append(step)
            at += n
        got, routing = run_steps_with_routing(eng, steps, {len(steps) - 1: ["p", "o"]})
        check_against_plain(plain_model(folder), toks, got["p"], routing["p"], dtype, f"{name} portions")
        check_against_plain(plain_model(folder), other, got["o"], routing["o"], dtype, f"{name} beside portions")
    finally:
        eng.release()


def test_slots_and_pages_used_again_carry_nothing_over(folders):
    """A request run after others have ended gets their slot and pages; its logits are those of a fresh engine."""
    cfg, folder = CONFIGS["a"], folders["a"]
    eng = engine_for(folder, "float32", max_tokens=64 * 4, max_slots=2)
    try:
        a, b, c = tokens_for(cfg, 130, 11), tokens_for(cfg, 90, 12), tokens_for(cfg, 140, 13)
        s1, e1 = batched({"a": a, "b": b}, {"a": 100, "b": 80})
        run_steps(eng, s1, e1)
        s2, e2 = with_tail("c", c, 30)
        got, routing = run_steps_with_routing(eng, s2, e2)
        check_against_plain(plain_model(folder), c, got["c"], routing["c"], "float32", "after reuse")
        eng.cache.book.check_invariants()
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_gives_pages_back_and_keeps_the_first(folders, dtype):
    """300 tokens decoded one by one from a 3-token prompt: windows pass over decoded tokens, pages that fell out of
    every window are given back, the pages of the kept first positions stay; graphs are replayed."""
    cfg, folder = CONFIGS["b"], folders["b"]
    toks = tokens_for(cfg, 303, 21)
    eng = engine_for(folder, dtype)
    try:
        s, e = with_tail("x", toks, 300)
        got, routing = run_steps_with_routing(eng, s[:-1], {}, leave_open=True)
        live = list(eng.cache.book.live.values())
        assert len(live) == 1 and live[0].length == 302
        gaps = 0
        for g, need in enumerate(eng.cache.groups):
            held = [p is not None for p in live[0].pages[g]]
            kept = -(-need.keep_first // 64) if need.window else len(held)
            gone = max(kept, (302 + 1 - need.window) // 64) if need.window else kept
            assert held == [i < kept or i >= gone for i in range(len(held))], (need, held)
            gaps += gone > kept
        assert gaps >= 2                                      # the test's model has windows that did move on
        eng.close(live[0])
        assert eng.graphs is not None and eng.graphs.replays >= 280
        check_against_plain(plain_model(folder), toks[:-1], got["x"], routing["x"], dtype, "long decoding")
    finally:
        eng.release()


VARIANTS = {
    # one mechanism a model
    "attention_alone": [layer("attention", attention(v_mix=False))],
    "latent_alone": [layer("latent_attention", latent())],
    "dense_alone": [layer("latent_attention", latent(heads=1, dim=8, vdim=8, kv_rank=8, q_rank=8), dense(ff=40, limit=0.4))],
    "experts_alone": [layer("latent_attention", latent(heads=1, dim=8, vdim=8, kv_rank=8, q_rank=8), moe(experts=12, top=4, groups=(3, 2), ff=8, limit=0.9, shared=(12, 0.3)))],
    # sizes and options
    "window_of_one": [layer("attention", attention(size=1, keep_first=0, rows=4, bias_max=3))],
    "only_first_kept": [layer("attention", attention(size=1, keep_first=40, rows=6, bias_max=50))],
    "keep_more_than_seen": [layer("attention", attention(size=5, keep_first=500, rows=30, bias_max=16))],
    "wide_value": [layer("attention", attention(heads=2, kv_heads=1, dim=8, vdim=136, size=20, keep_first=2)),
                   layer("attention", attention(heads=4, kv_heads=1, dim=200, vdim=136, size=7, keep_first=9))],
    "odd_sizes": [layer("attention", attention(heads=5, kv_heads=5, dim=7, vdim=3, size=13, keep_first=1, rows=6, bias_max=9), dense(ff=5)),
                  layer("latent_attention", latent(heads=5, dim=6, vdim=9, kv_rank=10, q_rank=3), moe(experts=5, top=2, groups=(5, 3), ff=3, shared=(7, 1.0)))],
    "many_experts": [layer("latent_attention", latent(), moe(experts=72, top=6, groups=(8, 3), ff=8, shared=None))],
    "mixing_far_apart": [layer("attention", attention(size=30)), layer("latent_attention", latent(), dense()),
                         layer("latent_attention", latent()), layer("attention", attention(heads=2, kv_heads=2, size=11, keep_first=0))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_other_sizes_and_options(tmp_path, variant, dtype):
    cfg = config(copy.deepcopy(VARIANTS[variant]), vocab=50, width=36)
    folder = write_model(str(tmp_path / variant), cfg, make_weights(cfg, 5))
    toks = tokens_for(cfg, 110, 31)
    eng = engine_for(folder, dtype)
    try:
        s, e = with_tail("x", toks, 25)
        got, routing = run_steps_with_routing(eng, s, e)
        check_against_plain(plain_model(folder), toks, got["x"], routing["x"], dtype, variant)
    finally:
        eng.release()


def test_a_wrong_edge_a_missing_sink_or_unmixed_values_would_show(folders, tmp_path):
    """The tests above mean something only if the plain model itself reacts to these faults: with the weights used
    here, moving a window's edge or the kept positions by one token, another far distance of the bias, a
    correction left out, or values left unmixed moves the logits by far more than the tolerance."""
    cfg, folder = CONFIGS["a"], folders["a"]
    toks = tokens_for(cfg, 160, 1)
    ref = plain_model(folder).forward(toks)
    weights = make_weights(cfg, 200)
    spread = ref.std()

    def changed(change, new_weights=None):
        wrong = copy.deepcopy(cfg)
        change(wrong)
        f = write_model(str(tmp_path / f"v{len(os.listdir(tmp_path))}"), wrong, new_weights or weights)
        return np.abs(PlainLumevik(f).forward(toks) - ref).max()

    assert changed(lambda c: c["layers"][0]["mixer"]["mask"].update(size=25)) > 1e-2 * spread
    assert changed(lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=4)) > 1e-2 * spread
    assert changed(lambda c: c["layers"][3]["mixer"]["mask"].update(keep_first=65)) > 1e-3 * spread
    assert changed(lambda c: c["layers"][0]["mixer"].update(bias_max=60)) > 1e-3 * spread
    assert changed(lambda c: c["layers"][2]["mixer"].update(v_mix=False),
                   {k: v for k, v in weights.items() if k != "l2.mix.vmix"}) > 1e-2 * spread
    assert changed(lambda c: None, dict(weights, **{"l0.mlp.correction": np.zeros_like(weights["l0.mlp.correction"])})) > 1e-2 * spread
    assert changed(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4)) > 1e-2 * spread
    assert changed(lambda c: c["layers"][1]["mlp"].update(limit=1.4)) > 1e-3 * spread


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_that_stands_out_is_found(tmp_path, dtype):
    """One key hundreds of positions back (in the first page, kept beyond the window; and once deep inside a full
    causal layer) carries almost all the weight of the last queries: its token's key and the queries' token are
    scaled so that their score stands out."""
    cfg = config([layer("attention", attention(heads=2, kv_heads=1, dim=32, vdim=32, size=40, keep_first=10, bias_max=600, rows=16, v_mix=False)),
                  layer("latent_attention", latent(heads=2, dim=16, vdim=16, kv_rank=24, q_rank=24))], vocab=40, width=32)
    w = make_weights(cfg, 9, sharp=1.0)
    # token 1 is the far key's token, token 2 the asking token: their rows of the embedding are made parallel, and the
    # first layer's query and key projections share rows, so that q(2) . k(1) is large whenever 2 looks at 1
    w["embed"][1] = 1.5 * np.sign(w["embed"][1])
    w["embed"][2] = w["embed"][1]
    w["l0.mix.k"][:] = w["l0.mix.q"][:32] * 1.0
    w["l0.mix.v"] *= 3.0              # what the far key brings weighs in the stream
    w["l0.mix.o"] *= 2.0
    toks = np.random.default_rng(3).integers(3, 40, size=400).tolist()
    toks[7] = 1                       # inside the kept first positions
    toks[12] = 1                      # just outside them: must not be seen from afar
    for p in (300, 395, 399):
        toks[p] = 2
    folder = write_model(str(tmp_path / "far"), cfg, w)
    plain = PlainLumevik(folder)
    ref = plain.forward(toks)
    moved = copy.deepcopy(toks)
    moved[7] = 5                      # without the far key the asking positions' logits are others
    assert np.abs(plain.forward(moved)[399] - ref[399]).max() > 0.03 * ref.std()
    eng = engine_for(folder, dtype)
    try:
        s, e = with_tail("x", toks, 10)
        got = run_steps(eng, s, e)
        assert_close(got["x"], ref, dtype, "far key")
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    import turboquant_cpp_b200 as tq
    cfg, folder = CONFIGS["a"], folders["a"]
    prompts = [tokens_for(cfg, n, 40 + n) for n in (1, 9, 40, 70)]
    n_new = 12
    with tq.Model(folder, temperature=0.0, max_tokens=n_new, dtype=dtype, max_batch=4, context_length=128) as m:
        outs = m.generate_batch(prompts)
        assert m.generate_batch(prompts[::-1])[::-1] == outs          # another order in the batch, slots used again
        assert [m.ask(p) for p in prompts] == outs                    # each alone
        m.engine.cache.book.check_invariants()
        assert m.engine.cache.book.slots.n_held == 0
    plain = plain_model(folder)
    floor = 1e-4 if dtype == "float32" else 0.15
    for p, o in zip(prompts, outs):
        toks = list(p)
        for i, t in enumerate(o):
            l = plain.forward(toks)[-1]
            top = np.sort(l)[-2:]
            if int(np.argmax(l)) != t:
                assert top[1] - top[0] < floor * l.std(), f"token {i}: engine {t}, plain {int(np.argmax(l))}"
                break                                                   # after a near-tie the texts part ways
            toks.append(t)


def test_trace_replay_as_a_user_runs_it(folders, tmp_path):
    cfg, folder = CONFIGS["b"], folders["b"]
    reqs = {"a": tokens_for(cfg, 45, 50), "b": tokens_for(cfg, 140, 51), "c": tokens_for(cfg, 1, 52)}
    s, e = batched(reqs, {"a": 13, "b": 100, "c": 1})
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in step], "end": e.get(i, [])})
             for i, step in enumerate(s)]
    out_dir = str(tmp_path / "out")
    need = sum(len(t) for t in reqs.values())                 # padding not counted
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", str(need)], input="\n".join(lines) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(s))]
    got, pos = {}, {}
    for i, step in enumerate(s):
        a = np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        row = 0
        for rid, toks, want in step:
            for w in want:
                got.setdefault(rid, {})[pos.get(rid, 0) + w] = a[row]
                row += 1
            pos[rid] = pos.get(rid, 0) + len(toks)
    for rid, toks in reqs.items():
        assert_close(got[rid], plain_model(folder).forward(toks), "float32", f"replay {rid}")

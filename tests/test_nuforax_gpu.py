"""The Nuforax decoder in the engine against the plain implementation (tests/plain/nuforax_plain.py): whole
prompts, decoding token by token, prompts in portions, batches of unequal requests, pages and slots used again,
windows' edges, other sizes, generation through the entry point, and trace replay as a user runs it."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT
from nuforax_util import CONFIGS, assert_close, config, latent, layer, make_weights, mamba, run_steps, write_folder
from plain.nuforax_plain import PlainNuforax
from replay_util import batched, whole, with_tail

pytestmark = pytest.mark.gpu

_plain_logits = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        out[name] = write_folder(str(tmp_path_factory.mktemp(f"nuforax_{name}")), cfg, make_weights(cfg, 100 + i, sharp=3.0))
    return out


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain_logits:
        _plain_logits[key] = PlainNuforax(folder).forward(list(tokens))
    return _plain_logits[key]


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def engine_for(folder, dtype, max_tokens=1024, **kw):
    import turboquant_cpp_b200 as tq
    return tq.Engine(tq.load_model(folder, dtype), max_tokens=max_tokens, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
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
        modes["whole"] = run_steps(eng, steps, ends)
        steps, ends = [], {}
        for rid, toks in reqs.items():                        # the last 70 tokens one by one (windows pass over decoded tokens)
            s, e = with_tail(rid, toks, 70)
            ends.update({k + len(steps): v for k, v in e.items()})
            steps += s
        modes["tail"] = run_steps(eng, steps, ends)
        s, e = batched(reqs, {"r0": 100, "r1": 1, "r2": 64, "r3": 129})     # unequal prompts, then decoded together
        modes["batched"] = run_steps(eng, s, e)
        eng.cache.book.check_invariants()
        assert eng.cache.book.slots.n_held == 0 and all(p.n_held == 0 for p in eng.cache.book.pools)
        for rid, toks in reqs.items():
            ref = plain_logits(folder, toks)
            for mode, got in modes.items():
                assert sorted(got[rid]) == list(range(len(toks))), f"{mode} {rid}"
                assert_close(got[rid], ref, dtype, f"{name} {mode} {rid}")
    finally:
        eng.release()


@pytest.mark.parametrize("name,sizes", [("a", [2, 3, 64, 1, 2, 7, 50]), ("b", [63, 2, 2, 65, 5]), ("c", [5, 128, 2, 30])])
def test_prompts_in_portions(folders, name, sizes):
    """A prompt cut into portions, down to two tokens, beside a request that goes on token by token."""
    cfg, folder = CONFIGS[name], folders[name]
    toks, other = tokens_for(cfg, sum(sizes), 7), tokens_for(cfg, len(sizes) + 20, 8)
    eng = engine_for(folder, "float32")
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
        got = run_steps(eng, steps, {len(steps) - 1: ["p", "o"]})
        assert_close(got["p"], plain_logits(folder, toks), "float32", f"{name} portions")
        assert_close(got["o"], plain_logits(folder, other), "float32", f"{name} beside portions")
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
        got = run_steps(eng, s2, e2)
        assert_close(got["c"], plain_logits(folder, c), "float32", "after reuse")
        eng.cache.book.check_invariants()
    finally:
        eng.release()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """300 tokens decoded one by one from a 3-token prompt: states and windows over many steps, graphs replayed."""
    cfg, folder = CONFIGS["b"], folders["b"]
    toks = tokens_for(cfg, 303, 21)
    eng = engine_for(folder, dtype)
    try:
        s, e = with_tail("x", toks, 300)
        got = run_steps(eng, s, e)
        assert eng.graphs is not None and eng.graphs.replays >= 290
        assert_close(got["x"], plain_logits(folder, toks), dtype, "long decoding")
    finally:
        eng.release()


@pytest.mark.parametrize("variant", ["no_rotation", "partial_rotation", "no_plain_dims", "one_tap", "state_200", "many_heads"])
def test_other_sizes_and_options(tmp_path, variant):
    layers = {
        "no_rotation": [layer("latent_attention", latent(rot_dim=0, dims=0, window=0), ff=32)],
        "partial_rotation": [layer("latent_attention", latent(rot_dim=12, dims=4, window=3), ff=None)],
        "no_plain_dims": [layer("latent_attention", latent(dim=0, rot_dim=16, window=17))],
        "one_tap": [layer("mamba2", mamba(conv=1, groups=1, heads=1, vdim=33, state=5, norm_groups=3))],
        "state_200": [layer("mamba2", mamba(heads=2, vdim=36, state=200, groups=2, conv=8, norm_groups=1), ff=16)],
        "many_heads": [layer("latent_attention", latent(heads=9, dim=4, rot_dim=4, vdim=4, kv_rank=8, window=33)),
                       layer("latent_attention", latent(heads=9, dim=4, rot_dim=4, vdim=4, kv_rank=8, window=2, kv_from=0))],
    }[variant]
    cfg = config(layers, vocab=50, width=36, bigram=(7, 2, 9))
    folder = write_folder(str(tmp_path / variant), cfg, make_weights(cfg, 5, sharp=2.0))
    toks = tokens_for(cfg, 90, 31)
    eng = engine_for(folder, "float32")
    try:
        s, e = with_tail("x", toks, 20)
        got = run_steps(eng, s, e)
        assert_close(got["x"], plain_logits(folder, toks), "float32", variant)
    finally:
        eng.release()


def test_a_wrong_window_a_missing_sink_or_a_lost_state_would_show(folders, tmp_path):
    """The tests above mean something only if the plain model itself reacts to these faults: with the weights
    used here, moving a window's edge by one token, dropping the sinks, or forgetting the pair table's state moves
    the logits by far more than the tolerance."""
    import copy
    cfg, folder = CONFIGS["a"], folders["a"]
    toks = tokens_for(cfg, 60, 1)
    ref = plain_logits(folder, toks)
    weights = make_weights(cfg, 100, sharp=3.0)
    spread = ref.std()
    wrong = copy.deepcopy(cfg)
    wrong["layers"][1]["mixer"]["mask"]["size"] += 1
    f2 = write_folder(str(tmp_path / "window"), wrong, weights)
    assert np.abs(PlainNuforax(f2).forward(toks) - ref)[20:].max() > 1e-2 * spread
    w2 = dict(weights)
    for k in w2:
        if k.endswith("sink"):
            w2[k] = np.full_like(w2[k], -30.0)
    f3 = write_folder(str(tmp_path / "sink"), cfg, w2)
    assert np.abs(PlainNuforax(f3).forward(toks) - ref).max() > 1e-2 * spread
    # the token before a portion's first token: without it the portion's first row takes the first-token row
    assert np.abs(PlainNuforax(folder).forward(toks[30:])[0] - ref[30]).max() > 1e-2 * spread


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
    plain = PlainNuforax(folder)
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
    cfg, folder = CONFIGS["c"], folders["c"]
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
        assert_close(got[rid], plain_logits(folder, toks), "float32", f"replay {rid}")

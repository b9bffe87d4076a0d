"""Parts of the Lumevik decoder that need no GPU: the configuration reader, the model's plan of tensors and cache
needs, the cache's bookkeeping of kept first positions, the distance buckets, and the plain implementation's own
consistency."""
import copy

import numpy as np
import pytest

from lumevik_util import CONFIGS, make_weights, tensor_shapes, write_model
from plain import lumevik_plain as P


def clean(cfg):
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        l["mixer"].pop("_rows", None)
    return c


def test_the_models_plan_names_every_tensor_with_its_shape():
    import turboquant_cpp_b200 as tq
    for name, cfg in CONFIGS.items():
        model = tq.build_model(clean(cfg), "bfloat16")
        plan = {s.name: tuple(s.shape) for s in model.weight_specs()}
        want = tensor_shapes(cfg)
        assert set(plan) == set(want), name
        for n, shape in plan.items():        # -1: a size that only the stored tensor gives (the bias table's rows)
            assert len(shape) == len(want[n]) and all(a in (-1, b) for a, b in zip(shape, want[n])), (name, n)
            assert (-1 in shape) == n.endswith("mix.rel")


def test_cache_needs_carry_windows_and_kept_positions():
    import turboquant_cpp_b200 as tq
    needs = tq.build_model(clean(CONFIGS["a"]), "float32").cache_needs()
    # attention: one plane of [key | value] rows per kv head, the window and what is kept of the start
    assert (needs[0].n_kv_heads, needs[0].head_dim, needs[0].window, needs[0].keep_first, needs[0].planes) == (2, 24, 24, 3, 1)
    assert (needs[3].window, needs[3].keep_first) == (70, 66)
    # latent attention: one row of kv_rank elements, everything kept
    assert (needs[1].n_kv_heads, needs[1].head_dim, needs[1].window, needs[1].planes) == (1, 40, 0, 1)
    needs = tq.build_model(clean(CONFIGS["c"]), "float32").cache_needs()
    assert needs[0].window == 0 and needs[0].keep_first == 0          # no mask: nothing is ever given back


def test_a_windowed_group_keeps_the_pages_of_its_first_positions():
    from turboquant_cpp_b200.cache.allocator import CacheBook
    book = CacheBook([16, 16, 16], [100, 100, 0], 64, 4, keep_first=[0, 70, 0])
    s = book.open()
    for n in (300, 1, 1, 200):
        book.reserve(s, n)
        book.commit(s, n)
    held = [[p is not None for p in pages] for pages in s.pages]
    first_visible = (502 + 1 - 100) // 64
    assert held[0] == [i >= first_visible for i in range(8)]
    assert held[1] == [i < 2 or i >= first_visible for i in range(8)]         # 70 positions: two pages stay
    assert all(held[2])
    book.check_invariants()
    book.close(s)
    assert all(p.n_held == 0 for p in book.pools)


def test_distance_buckets_are_the_plain_formula_and_end_in_the_last_row():
    from turboquant_cpp_b200.parts.bias_attention import distance_buckets
    for rows, far in ((32, 120), (8, 17), (16, 128), (6, 9), (64, 500), (4, 3)):
        got = distance_buckets(rows, far)
        assert got == [P.distance_bucket(n, rows, far) for n in range(far + 1)]
        assert got[:rows // 2] == list(range(rows // 2)) and got[-1] == rows - 1
        assert all(b >= a for a, b in zip(got, got[1:]))
        assert P.distance_bucket(far + 1000, rows, far) == rows - 1          # what the kernels clamp to


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("dim", 300), "dim"),
    (lambda c: c["layers"][0].__setitem__("type", "mamba2"), "type"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("keep", 1), "choices"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "conv"), "kind"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 16), "v_mix"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_key(change, word):
    import turboquant_cpp_b200 as tq
    cfg = clean(CONFIGS["a"])
    change(cfg)
    with pytest.raises(tq.ConfigError) as e:
        tq.build_model(cfg, "float32")
    assert word in str(e.value)


def test_random_weights_need_the_bias_tables_rows_in_the_configuration(tmp_path):
    import turboquant_cpp_b200 as tq
    cfg = clean(CONFIGS["a"])
    with pytest.raises(ValueError):
        tq.write_random_folder(str(tmp_path / "no_rows"), cfg, 1)
    for l in cfg["layers"]:
        if l["type"] == "attention":
            l["mixer"]["bias_rows"] = 10
    tq.write_random_folder(str(tmp_path / "rows"), cfg, 1)
    m = P.PlainLumevik(str(tmp_path / "rows"))
    assert m.t["l0.mix.rel"].shape == (10, 4) and m.t["l0.mix.vmix"].shape == ()
    assert np.isfinite(m.forward([1, 2, 3])).all()


def test_plain_decoding_by_recomputation_is_causal(tmp_path):
    """The plain model has no cache: the logits of a prefix are the first rows of the logits of the whole."""
    cfg = CONFIGS["a"]
    folder = write_model(str(tmp_path / "m"), cfg, make_weights(cfg, 1))
    m = P.PlainLumevik(folder)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 60).tolist()
    assert np.abs(m.forward(toks)[:35] - m.forward(toks[:35])).max() < 1e-9


def test_plain_routing_respects_groups_and_weights_sum_to_one():
    rng = np.random.default_rng(5)
    h = rng.standard_normal((50, 16))
    w = {"router": rng.standard_normal((12, 16)), "correction": 0.3 * rng.standard_normal(12)}
    r = {"experts": 12, "top": 4, "groups": {"count": 4, "keep": 2}}
    ids, wts = P.route(h, w, r)
    assert np.allclose(wts.sum(axis=1), 1.0)
    for row in ids:
        assert len(set(row.tolist())) == 4 and len({e // 3 for e in row}) <= 2
    loose, _ = P.route(h, w, dict(r, groups={"count": 4, "keep": 4}))
    assert np.any(np.sort(loose, axis=1) != np.sort(ids, axis=1))       # the groups do bind with these weights

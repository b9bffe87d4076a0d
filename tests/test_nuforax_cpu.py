"""Parts of the Nuforax decoder that need no GPU: the configuration reader, the model's plan of tensors and cache
needs, and the plain implementation's own consistency."""
import copy

import numpy as np
import pytest

from nuforax_util import CONFIGS, make_weights, tensor_shapes, write_folder
from plain import nuforax_plain as P


def test_the_models_plan_names_every_tensor_with_its_shape():
    import turboquant_cpp_b200 as tq
    for name, cfg in CONFIGS.items():
        model = tq.build_model(cfg, "bfloat16")
        assert {s.name: tuple(s.shape) for s in model.weight_specs()} == tensor_shapes(cfg), name


def test_cache_needs_follow_the_readers_windows():
    import turboquant_cpp_b200 as tq
    needs = tq.build_model(CONFIGS["b"], "float32").cache_needs()
    # layer 1 (window 5) is read by layer 2 (window 70): its rows are kept for 70 positions; one row, one plane
    assert needs[0] is None and needs[2] is None and needs[3] is None
    assert (needs[1].window, needs[1].planes, needs[1].n_kv_heads, needs[1].head_dim) == (70, 1, 1, 36)
    needs = tq.build_model(CONFIGS["a"], "float32").cache_needs()
    assert needs[0].window == 24 and needs[3].window == 0 and needs[1] is None
    states = tq.build_model(CONFIGS["a"], "float32").state_needs()
    assert [s is not None for s in states] == [False, False, True, False]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 41), "kv_rank"),
    (lambda c: c["layers"][0].__setitem__("type", "attention"), "type"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 9), "dims"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("state", 1000), "state"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_key(change, word):
    import turboquant_cpp_b200 as tq
    cfg = copy.deepcopy(CONFIGS["a"])
    change(cfg)
    with pytest.raises(tq.ConfigError) as e:
        tq.build_model(cfg, "float32")
    assert word in str(e.value)


def test_plain_decoding_by_recomputation_is_causal(tmp_path):
    """The plain model has no cache: the logits of a prefix are the first rows of the logits of the whole."""
    cfg = CONFIGS["a"]
    folder = write_folder(str(tmp_path / "m"), cfg, make_weights(cfg, 1, sharp=3.0))
    m = P.PlainNuforax(folder)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 40).tolist()
    assert np.abs(m.forward(toks)[:25] - m.forward(toks[:25])).max() < 1e-9


def test_scaled_frequencies_keep_fast_pairs_and_slow_down_the_others():
    f0, m0 = P.rotary_frequencies(32, 10000.0)
    f1, m1 = P.rotary_frequencies(32, 10000.0, {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 1.0})
    assert m0 == 1.0 and abs(m1 - (0.1 * np.log(8.0) + 1.0)) < 1e-12
    assert f1[0] == f0[0] and abs(f1[-1] - f0[-1] / 8.0) < 1e-15 and np.all(f1 <= f0) and np.all(f1 >= f0 / 8.0 - 1e-15)

"""The kernels behind the Lumevik parts, each alone against the plain functions (tests/plain/lumevik_plain.py): the
gated activation with caps in its three homes, the selection with corrected scores and groups, the cache write with
mixed values, and both attention kernels over scattered pages (windows' and kept positions' edges, page borders,
every number of key ranges)."""
import math

import numpy as np
import pytest
import torch

from plain import lumevik_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def bf16(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(torch.bfloat16).float().numpy().astype(np.float64)


def rel(got, want):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    return np.abs(got - want).max() / max(1e-30, np.abs(want).max())


@pytest.mark.parametrize("limit", [0.5, 2.0, 7.0])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activation_with_caps(limit, dtype):
    from turboquant_cpp_b200.kernels import elementwise as KE
    rng = np.random.default_rng(1)
    gu = 3.0 * rng.standard_normal((37, 2 * 50))
    out = torch.empty((37, 50), dtype=dtype, device=DEV)
    KE.glu_mul(dev(gu, torch.float32), out, KE.Glu(limit=limit, slope=P.GLU_SLOPE, offset=1.0))
    want = P.capped_glu(gu[:, :50], gu[:, 50:], limit)
    assert (np.abs(gu) > limit).mean() > 0.02            # the caps do bind
    assert rel(out, want) < (1e-6 if dtype == torch.float32 else 5e-3)
    # the default is silu(gate) * up
    KE.glu_mul(dev(gu, torch.float32), out)
    assert rel(out, gu[:, :50] / (1 + np.exp(-gu[:, :50])) * gu[:, 50:]) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("R,N,K,G", [(3, 24, 40, 4), (70, 64, 48, 5), (300, 136, 192, 8)])
@pytest.mark.parametrize("packed", [False, True])
def test_experts_products_with_the_capped_activation(R, N, K, G, packed):
    """The grouped products with the gate's caps, slope and offset in their epilogues: the exact kernels (both
    forms) and the tensor-core kernel."""
    from turboquant_cpp_b200.kernels import elementwise as KE, gemm_tc as KT, moe as KM
    rng = np.random.default_rng(R + N)
    a = bf16(rng.normal(size=(R, K)))
    w = bf16(2.0 * rng.normal(size=(G, 2 * N, K)) / math.sqrt(K))
    glu = KE.Glu(limit=1.3, slope=P.GLU_SLOPE, offset=1.0)
    ids = rng.integers(0, G, size=(R, 1)).astype(np.int32)
    tile = 64
    lay = KM.ExpertLayout(R, G, tile, DEV)
    KM.moe_align(dev(ids, torch.int32), lay)
    order = lay.sorted_pair.cpu().numpy()[:R]
    x = a[order]
    want = np.zeros((R, N))
    for g in range(G):
        sel = np.nonzero(ids[order, 0] == g)[0]
        if len(sel):
            want[sel] = P.capped_glu(x[sel] @ w[g, :N].T, x[sel] @ w[g, N:].T, 1.3)
    if packed:
        out = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        KT.gemm_tc(dev(x, torch.bfloat16), KT.pack_weights(dev(w, torch.bfloat16), True), out, lay, tile, glu=glu)
        KT.check_status()
        assert rel(out, want) < 6e-3
        return
    for few in (False, True):
        for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 6e-3)):
            out = torch.full((R, N), float("nan"), dtype=dt, device=DEV)
            KM.grouped_gemm(dev(x, dt), dev(w, dt), out, lay, True, few_rows=few, glu=glu)
            assert rel(out, want) < tol, (few, dt)


@pytest.mark.parametrize("E,k,groups,keep", [(12, 3, 3, 2), (8, 2, 1, 1), (6, 6, 6, 6), (64, 8, 8, 3), (300, 5, 10, 4), (40, 1, 40, 1)])
@pytest.mark.parametrize("corrected", [True, False])
def test_selection_with_corrected_scores_and_groups(E, k, groups, keep, corrected):
    from turboquant_cpp_b200.kernels import moe as KM
    rng = np.random.default_rng(E * 31 + k)
    T, H = 97, 24
    h = rng.standard_normal((T, H))
    w = {"router": 0.3 * rng.standard_normal((E, H)), "correction": (0.3 / E * rng.standard_normal(E)) if corrected else np.zeros(E)}
    sg = rng.standard_normal((1, H))
    r = {"experts": E, "top": k, "groups": {"count": groups, "keep": keep}}
    margins = []
    ids, wts = P.route(h, w, r, margins=margins)
    logits = KM.router_logits(dev(h, torch.float32), dev(w["router"], torch.float32), dev(sg, torch.float32),
                              torch.empty((T, E + 1), dtype=torch.float32, device=DEV))
    got_ids = torch.empty((T, k), dtype=torch.int32, device=DEV)
    got_w = torch.empty((T, k), dtype=torch.float32, device=DEV)
    scale = torch.empty((T,), dtype=torch.float32, device=DEV)
    KM.router_select_corrected(logits, dev(w["correction"], torch.float32) if corrected else None, k, True, P.WEIGHT_FLOOR,
                               groups, keep, got_ids, got_w, scale)
    assert rel(scale, P.sigmoid(h @ sg.T)[:, 0]) < 1e-5
    gi, gw = got_ids.cpu().numpy(), got_w.cpu().numpy()
    clear = np.array(margins) > 1e-6
    assert clear.mean() > 0.8
    for t in np.nonzero(clear)[0]:
        assert sorted(gi[t].tolist()) == sorted(ids[t].tolist()), (t, gi[t], ids[t])
        order_g, order_p = np.argsort(gi[t]), np.argsort(ids[t])
        assert np.abs(gw[t][order_g] - wts[t][order_p]).max() < 1e-5
    assert np.abs(gw.sum(axis=1) - 1.0).max() < 1e-5


def scattered_cache(T, G, dr, dtype, rng, extra_pages=3):
    """A cache of more pages than the sequence needs, filled with a large value where nothing is written, and a page
    table that visits the pages in a shuffled order."""
    n = -(-T // 64)
    cache = torch.full((n + extra_pages, 1, G, 64, dr), 1e30, dtype=dtype, device=DEV)
    table = torch.tensor(rng.permutation(n + extra_pages)[:n].reshape(1, n), dtype=torch.int32, device=DEV)
    return cache, table


ATT_CASES = [
    # T, H, G, dk, dv, window, keep_first, rows, far
    (200, 4, 2, 32, 64, 70, 5, 16, 100),          # the tensor-core kernel's sizes; a window wider than a page
    (300, 2, 1, 64, 32, 64, 64, 8, 20),           # window and kept positions of exactly a page
    (150, 3, 3, 128, 128, 0, 0, 32, 120),         # no window
    (131, 6, 2, 24, 40, 33, 66, 10, 50),          # sizes only the token kernel takes; kept positions beyond a page
    (260, 2, 2, 32, 32, 1, 129, 4, 3),            # a window of one: itself and the kept first positions
    (190, 16, 2, 64, 64, 50, 3, 12, 60),          # eight heads a key/value head
    (140, 24, 2, 128, 32, 40, 70, 12, 60),        # twelve: the heads of a key/value head are shared out over blocks
    (100, 8, 4, 32, 128, 30, 2, 6, 40),           # a value four times the key
]


@pytest.mark.parametrize("case", ATT_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_write_and_both_attention_kernels(case, dtype):
    from turboquant_cpp_b200.kernels import bias_attention as KB
    T, H, G, dk, dv, window, keep, rows, far = case
    rng = np.random.default_rng(T + H)
    m = {"scale": 0.9 / math.sqrt(dk), "bias_max": far}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    qkv = rng.standard_normal((T, H * dk + G * (dk + dv))) * 1.5
    v_first = rng.standard_normal((T, G * dv))
    lam = 0.37
    relt = 1.5 * rng.standard_normal((rows, H))
    q = qkv[:, :H * dk].reshape(T, H, dk)
    k = qkv[:, H * dk:H * dk + G * dk].reshape(T, G, dk)
    v = P.mix_values(qkv[:, H * dk + G * dk:], v_first, lam).reshape(T, G, dv)
    if dtype == torch.bfloat16:
        q, k, v = bf16(q), bf16(k), bf16(v)
    want = P.biased_attention_core(q, k, v, relt, m).reshape(T, H * dv)

    cache, table = scattered_cache(T, G, dk + dv, dtype, rng)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    seq_of_token = torch.zeros(T, dtype=torch.int32, device=DEV)
    q_dev = torch.empty((T, H, dk), dtype=dtype, device=DEV)
    kept_values = torch.empty((T, G * dv), dtype=torch.float32, device=DEV)
    KB.kv_write(dev(qkv, torch.float32), q_dev, cache, kept_values, dev(v_first, torch.float32), lam, positions,
                seq_of_token, table, 64, H, G, dk, dv)
    assert rel(kept_values, P.mix_values(qkv[:, H * dk + G * dk:], v_first, lam)) < 1e-6
    from turboquant_cpp_b200.parts.bias_attention import distance_buckets
    bias = dev(relt[distance_buckets(rows, far)], torch.float32)
    sink = torch.zeros(H, dtype=torch.float32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    import os
    for n_splits in (1, 2, 5, 64):
        # a block per head; then, where built, a block per key/value head on CUDA cores and on tensor cores
        for bias_t, form in ((None, ""), (bias.t().contiguous(), "group"), (bias.t().contiguous(), "heads")):
            os.environ["TQ_BIAS_TOKEN_FORM"] = form
            try:
                out = torch.full((T, H * dv), float("nan"), dtype=dtype, device=DEV)
                KB.attention(q_dev, cache, bias, sink, positions, seq_of_token, table, 64, window, keep, m["scale"], out, H, G,
                             dk, dv, n_splits=n_splits, bias_t=bias_t)
            finally:
                os.environ.pop("TQ_BIAS_TOKEN_FORM", None)
            assert rel(out, want) < tol, (n_splits, form)
    if KB.runs_usable(dtype, dk, dv, 64):
        # the same tokens as one run, and as a run that continues a sequence (its first 77 tokens already cached)
        for start in (0, 77):
            out = torch.full((T - start, H * dv), float("nan"), dtype=dtype, device=DEV)
            cu = torch.tensor([0, T - start], dtype=torch.int32, device=DEV)
            st = torch.tensor([start], dtype=torch.int32, device=DEV)
            KB.attention_runs(q_dev[start:].contiguous(), cache, bias.t().contiguous(), sink, cu, st, table, 64, window, keep,
                              m["scale"], out, 1, T - start, H, G, dk, dv)
            assert rel(out, want[start:]) < tol, start
    # without a sink and without a bias the kernels compute an ordinary softmax: against the closed form at one row
    out = torch.empty((T, H * dv), dtype=dtype, device=DEV)
    KB.attention(q_dev, cache, None, None, positions, seq_of_token, table, 64, 0, 0, m["scale"], out, H, G, dk, dv)
    i, a = T - 1, H - 1
    s = k[:, a // (H // G)] @ q[i, a] * m["scale"]
    p = np.exp(s - s.max())
    row = (p / p.sum()) @ v[:, a // (H // G)]
    assert np.abs(out[i].float().cpu().numpy().reshape(H, dv)[a] - row).max() < tol * max(1.0, np.abs(row).max()) * 3


@pytest.mark.parametrize("T,E,k,groups,keep,H", [(1, 12, 3, 3, 2, 64), (8, 60, 4, 4, 2, 128), (5, 8, 8, 1, 1, 40), (24, 16, 2, 8, 3, 72)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_one_launch_router_chooses_like_the_separate_kernels(T, E, k, groups, keep, H, dtype):
    """Decode steps take logits, corrected selection, layout and the rows' copies in one launch: the same choices,
    weights and layout as the separate kernels give."""
    from turboquant_cpp_b200.kernels import elementwise as KE, moe as KM
    rng = np.random.default_rng(T * 100 + E)
    x = dev(rng.standard_normal((T, H)), dtype)
    wr = dev(0.3 * rng.standard_normal((E, H)), dtype)
    sg = dev(rng.standard_normal((1, H)), dtype)
    corr = dev(0.3 / E * rng.standard_normal(E), torch.float32)
    i32 = dict(dtype=torch.int32, device=DEV)
    f32 = dict(dtype=torch.float32, device=DEV)
    ids_a, w_a, s_a = torch.empty((T, k), **i32), torch.empty((T, k), **f32), torch.empty((T,), **f32)
    ids_b, w_b, s_b = torch.empty((T, k), **i32), torch.empty((T, k), **f32), torch.empty((T,), **f32)
    logits = KM.router_logits(x, wr, sg, torch.empty((T, E + 1), **f32))
    KM.router_select_corrected(logits, corr, k, True, P.WEIGHT_FLOOR, groups, keep, ids_a, w_a, s_a)
    lay_a = KM.ExpertLayout(T * k, E, 16, DEV)
    KM.moe_align(ids_a, lay_a)
    rows_a = KE.gather_rows(x, lay_a.sorted_pair, k, torch.empty((T * k, H), dtype=dtype, device=DEV))
    lay_b = KM.ExpertLayout(T * k, E, 16, DEV)
    rows_b = torch.empty((T * k, H), dtype=dtype, device=DEV)
    KM.router_small(x, wr, sg, k, True, ids_b, w_b, s_b, lay_b, rows_b, correction=corr, corrected=True,
                    floor=P.WEIGHT_FLOOR, n_groups=groups, keep_groups=keep)
    assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b) and torch.equal(s_a, s_b)
    assert torch.equal(lay_a.sorted_pair[:T * k], lay_b.sorted_pair[:T * k]) and torch.equal(lay_a.row_of_pair[:T * k], lay_b.row_of_pair[:T * k])
    n = int(lay_a.n_tiles.item())
    assert n == int(lay_b.n_tiles.item()) and torch.equal(lay_a.tile_expert[:n], lay_b.tile_expert[:n])
    assert torch.equal(rows_a, rows_b)
    # and against the plain choice, where its margin is clear
    margins = []
    w = {"router": wr.float().cpu().numpy().astype(np.float64), "correction": corr.cpu().numpy().astype(np.float64)}
    ids, _ = P.route(x.float().cpu().numpy().astype(np.float64), w, {"experts": E, "top": k, "groups": {"count": groups, "keep": keep}}, margins=margins)
    for t in range(T):
        if margins[t] > 1e-5:
            assert sorted(ids_b[t].tolist()) == sorted(ids[t].tolist())

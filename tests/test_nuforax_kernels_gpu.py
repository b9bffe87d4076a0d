"""Each mechanism of the Nuforax decoder alone: a kernel (or a part) against the plain function of the same
name in tests/plain/nuforax_plain.py, with inputs made so that a fault shows: one key whose score stands far out
just inside or just outside a window, at a page's border, or hundreds of tokens away; a sink that takes most of
the weight; states carried over steps."""
import numpy as np
import pytest
import torch

from plain import nuforax_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def plain_rows_attention(q_lat, q_rot, rows, R, sink, window, scale, pos):
    """One token's heads over cached rows [n, R + rot]: softmax with a sink of the scores, weighted sum of the
    rows' first R elements."""
    j0 = 0 if window <= 0 else max(0, pos - window + 1)
    out = np.zeros((q_lat.shape[0], R))
    for a in range(q_lat.shape[0]):
        s = (rows[j0:pos + 1, :R] @ q_lat[a] + rows[j0:pos + 1, R:] @ q_rot[a]) * scale
        m = max(s.max(), sink[a])
        e = np.exp(s - m)
        out[a] = e @ rows[j0:pos + 1, :R] / (e.sum() + np.exp(sink[a] - m))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,rot,window,n_ctx,lead", [
    (3, 40, 8, 37, 300, 5), (5, 288, 32, 0, 700, 8), (1, 30, 6, 64, 130, 5), (6, 160, 32, 65, 200, 8), (6, 160, 32, 65, 200, 5),
    (2, 512, 64, 129, 400, 8), (20, 64, 16, 50, 300, 6), (17, 32, 0, 33, 100, 8)])
def test_latent_attention_with_one_key_that_stands_out(dtype, H, R, rot, window, n_ctx, lead):
    """Queries at several positions; for each, one key is given a score far above the rest: the key just inside
    the window, the key just outside it, a key at a page's first or last place, the first key of the sequence.
    Outside the window (or with a sink above it) the result must not move; inside it must follow the key.
    `lead` plain dimensions stand in front of a head's rotated ones (8: rows the kernels can copy 16 bytes at a
    time; 5: an odd head size, which keeps bfloat16 off the tensor-core form; 6: that form with single copies)."""
    from turboquant_cpp_b200.kernels import latent_attention as KL
    rng = np.random.default_rng(R + window)
    page_size, n_pages = 64, 16
    pages = rng.permutation(n_pages)[:-(-n_ctx // page_size)]
    rows = rng.standard_normal((n_ctx, R + rot)) * 0.3
    sink = rng.standard_normal(H)
    sink[0] = 3.0
    scale = 0.4
    special = {}
    positions = [0, 1, 63, 64, window - 1 if window else 5, window if window else 6, n_ctx - 1, n_ctx - 2, n_ctx - 66]
    positions = sorted({p for p in positions if 0 <= p < n_ctx})
    targets = {}
    for p in positions:
        edge = p - window + 1 if window else 0
        for tag, j in (("in", max(edge, 0)), ("out", edge - 1), ("page", (p // page_size) * page_size), ("first", 0)):
            if 0 <= j <= p:
                targets[(p, tag)] = j
    cache = torch.zeros((n_pages, 1, 1, page_size, R + rot), dtype=dtype, device=DEV)
    if dtype == torch.bfloat16:
        rows = dev(rows, dtype).float().cpu().numpy().astype(np.float64)
    for j in range(n_ctx):
        cache[pages[j // page_size], 0, 0, j % page_size] = dev(rows[j], dtype)
    table = i32([list(pages) + [-1] * (n_pages - len(pages))])
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for (p, tag), j in targets.items():
        # a query aligned with key j in head 1 (head 0 has the heavy sink), ordinary in the others
        q_lat = rng.standard_normal((H, R)) * 0.3
        q_rot = rng.standard_normal((H, rot)) * 0.3
        hh = min(1, H - 1)
        q_lat[hh] = rows[j, :R] * (12.0 / scale / max(1e-9, (rows[j, :R] ** 2).sum()))
        ql = dev(q_lat[None], dtype)
        qfull = torch.zeros((1, H * (lead + rot)), dtype=dtype, device=DEV)          # plain dimensions in front
        qfull.view(1, H, lead + rot)[:, :, lead:] = dev(q_rot[None], dtype)
        ref = plain_rows_attention(ql[0].float().cpu().numpy().astype(np.float64),
                                   qfull.view(H, lead + rot)[:, lead:].float().cpu().numpy().astype(np.float64), rows, R, sink,
                                   window, scale, p)
        for n_splits in (1, 3, 7):
            out = torch.empty((1, H, R), dtype=dtype, device=DEV)
            partial = torch.empty(H * n_splits * (R + 2), dtype=torch.float32, device=DEV)
            KL.latent_attention(ql, qfull, lead, cache, dev(sink), i32([p]), i32([0]), table, page_size, window, scale, out, H,
                                R, rot, n_splits, partial)
            err = np.abs(out[0].float().cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err < tol, f"position {p}, key {j} ({tag}), {n_splits} ranges: {err:.2e}"
        # the test's own meaning: the key that stands out decides the result exactly when it is visible
        w = np.abs(ref[hh] - rows[j, :R]).max()
        visible = window == 0 or p - j < window
        if H > 1:
            assert (w < 0.05) == visible, f"position {p}, key {j} ({tag})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare_norms_rotates_and_writes_the_row(dtype):
    from turboquant_cpp_b200.kernels import latent_attention as KL
    from turboquant_cpp_b200.parts.rotary import ScaledRotaryEncoding
    rng = np.random.default_rng(3)
    T, H, dim, rot, R, dims = 7, 3, 5, 12, 20, 8
    enc = ScaledRotaryEncoding(dims, 5000.0, factor=3.0, original=40.0, fast=6.0, slow=0.5)
    enc.prepare(DEV)
    f, mag = P.rotary_frequencies(dims, 5000.0, {"factor": 3.0, "original": 40.0, "fast": 6.0, "slow": 0.5})
    assert np.allclose(enc.freq.cpu().numpy(), f, rtol=1e-6) and abs(enc.mag - mag) < 1e-12
    pos = [130, 131, 0, 1, 2, 63, 64]                   # two sequences: one continues at 130, one starts
    seq = [0, 0, 1, 1, 1, 0, 0]
    table = i32([[2, 5, 0], [1, -1, -1]])
    q = rng.standard_normal((T, H, dim + rot))
    d = rng.standard_normal((T, R + rot))
    w = 1.0 + 0.1 * rng.standard_normal(R)
    qd = dev(q.reshape(T, -1), dtype)
    q_in = qd.float().cpu().numpy().astype(np.float64).reshape(T, H, dim + rot)
    cache = torch.zeros((6, 1, 1, 64, R + rot), dtype=dtype, device=DEV)
    KL.latent_prepare(qd, dev(d), dev(w, dtype), 1e-5, enc.freq, enc.mag, i32(pos), i32(seq), table, 64, cache, H, dim, rot, R)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    wq = dev(w, dtype).float().cpu().numpy().astype(np.float64)
    d32 = dev(d).cpu().numpy().astype(np.float64)
    for t in range(T):
        want_q = q_in[t].copy()
        want_q[:, dim:] = P.rotate_interleaved(q_in[t:t + 1, :, dim:], [pos[t]], f, mag)[0]
        assert np.abs(qd[t].float().cpu().numpy().reshape(H, -1) - want_q).max() < tol * 4
        page = int(table[seq[t], pos[t] // 64])
        row = cache[page, 0, 0, pos[t] % 64].float().cpu().numpy()
        want = np.concatenate([P.rms(d32[t, :R], 1e-5) * wq, P.rotate_interleaved(d32[t:t + 1, R:], [pos[t]], f, mag)[0]])
        assert np.abs(row - want).max() < tol * 4, f"token {t}"


def test_pair_embedding_remembers_the_token_before_across_steps():
    from turboquant_cpp_b200.kernels import elementwise as K
    rng = np.random.default_rng(4)
    V, W, buckets, mp, mc = 30, 16, 11, 7, 3
    table, pairs = rng.standard_normal((V, W)), rng.standard_normal((buckets + 1, W))
    seqs = {0: rng.integers(0, V, 9).tolist(), 1: rng.integers(0, V, 6).tolist()}
    want = {s: P.embed_tokens(t, dev(table).cpu().numpy().astype(np.float64), 2.5, dev(pairs).cpu().numpy().astype(np.float64),
                              buckets, mp, mc) for s, t in seqs.items()}
    last = torch.full((8,), 12345, dtype=torch.int32, device=DEV)          # stale values of earlier users of the slots
    slots = {0: 5, 1: 2}
    cuts = [(4, 3), (1, 1), (4, 2)]                                          # portions of both sequences per step
    at = {0: 0, 1: 0}
    for n0, n1 in cuts:
        toks = seqs[0][at[0]:at[0] + n0] + seqs[1][at[1]:at[1] + n1]
        out = torch.empty((n0 + n1, W), dtype=torch.float32, device=DEV)
        K.embed_pair_rows(i32(toks), dev(table), dev(pairs), 2.5, buckets, mp, mc, i32([0] * n0 + [1] * n1), i32([0, n0, n0 + n1]),
                          i32([at[0], at[1]]), i32([slots[0], slots[1]]), last, out)
        got = out.cpu().numpy()
        assert np.abs(got[:n0] - want[0][at[0]:at[0] + n0]).max() < 1e-5
        assert np.abs(got[n0:] - want[1][at[1]:at[1] + n1]).max() < 1e-5
        at[0] += n0
        at[1] += n1


@pytest.mark.parametrize("H", [50, 52, 1536, 4096, 4100])
def test_norm_on_the_sublayer_output_is_added_in_float32(H):
    """Rows of 50 and 4,100 elements take the kernel's plain form, the others the one that keeps y in registers (one,
    two and four pieces a thread)."""
    from turboquant_cpp_b200.kernels import elementwise as K
    rng = np.random.default_rng(5)
    x, y, w = rng.standard_normal((6, H)) * 100, rng.standard_normal((6, H)), 1 + 0.1 * rng.standard_normal(H)
    for with_copy in (True, False):
        xd = dev(x)
        copy = torch.empty((6, H), dtype=torch.bfloat16, device=DEV) if with_copy else None
        want = dev(x).cpu().numpy().astype(np.float64) + P.rms(dev(y).cpu().numpy().astype(np.float64), 1e-3) * dev(w).cpu().numpy()
        K.add_rmsnorm(xd, dev(y), dev(w), 1e-3, copy)
        assert np.abs(xd.cpu().numpy() - want).max() < 2e-5
        if with_copy:
            assert torch.equal(copy, xd.to(torch.bfloat16))
    h = torch.empty((6, H), dtype=torch.float32, device=DEV)
    K.map_elements(dev(y), h, K.MAP_RELU_SQUARED)
    assert np.abs(h.cpu().numpy() - P.relu_squared(dev(y).cpu().numpy().astype(np.float64))).max() < 1e-6


@pytest.mark.parametrize("heads,vdim,N,groups,taps", [(4, 12, 16, 2, 3), (2, 40, 64, 1, 4), (3, 33, 130, 3, 2), (1, 8, 256, 1, 1)])
def test_convolution_and_recurrence_carry_their_state_over_steps(heads, vdim, N, groups, taps):
    """Two sequences fed in portions of unequal sizes (one token, two, many) from slots that held other values
    before; the convolution's kept inputs and the state must give what the plain functions give on the whole."""
    from turboquant_cpp_b200.kernels import ssm as KS
    rng = np.random.default_rng(N + taps)
    inner, gn = heads * vdim, groups * N
    C, Pr = inner + 2 * gn, 2 * inner + 2 * gn + heads
    lens = {0: 341, 1: 28}
    proj = {s: dev(rng.standard_normal((n, Pr))).cpu().numpy().astype(np.float64) for s, n in lens.items()}
    w_conv, b_conv = rng.standard_normal((C, taps)) * 0.5, rng.standard_normal(C) * 0.3
    dt_bias, a_log, d_skip = rng.standard_normal(heads), rng.standard_normal(heads) * 0.5, rng.standard_normal(heads)
    f32 = lambda a: dev(a).cpu().numpy().astype(np.float64)
    want_y, want_xbc = {}, {}
    for s in lens:
        xbc = P.silu(P.causal_conv(proj[s][:, inner:inner + C], f32(w_conv), f32(b_conv)))
        dt = P.softplus(proj[s][:, inner + C:] + f32(dt_bias))
        want_xbc[s] = xbc
        want_y[s] = P.state_space_scan(xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:], dt, f32(a_log), f32(d_skip),
                                       heads, vdim, N, groups)
    n_slots, kept_size = 4, (taps - 1) * C
    st = torch.zeros((n_slots, kept_size + heads * N * vdim), dtype=torch.float32, device=DEV)
    kept = st[:, :kept_size].unflatten(1, (taps - 1, C))
    S = st[:, kept_size:].unflatten(1, (heads, vdim, N))
    slots = {0: 3, 1: 1}
    cuts = [(1, 2), (2, 1), (17, 1), (300, 5), (1, 17), (20, 2)]     # the long step takes the form with several tokens a thread
    at = {0: 0, 1: 0}
    for n0, n1 in cuts:
        pr = dev(np.concatenate([proj[0][at[0]:at[0] + n0], proj[1][at[1]:at[1] + n1]]))
        T = n0 + n1
        xbc = torch.empty((T, C), dtype=torch.float32, device=DEV)
        cu, sl, sot = i32([0, n0, T]), i32([slots[0], slots[1]]), i32([0] * n0 + [1] * n1)
        KS.conv_silu(pr, inner, dev(w_conv), dev(b_conv), kept, xbc, sot, cu, sl)
        y = torch.empty((T, inner), dtype=torch.float32, device=DEV)
        KS.ssm_scan(xbc, pr, inner + C, dev(dt_bias), dev(a_log), dev(d_skip), S, y, heads, vdim, N, groups, cu, sl)
        for s, lo, n in ((0, 0, n0), (1, n0, n1)):
            ref_x, ref_y = want_xbc[s][at[s]:at[s] + n], want_y[s][at[s]:at[s] + n]
            assert np.abs(xbc[lo:lo + n].cpu().numpy() - ref_x).max() < 1e-5 * max(1.0, np.abs(ref_x).max())
            assert np.abs(y[lo:lo + n].cpu().numpy() - ref_y).max() < 2e-5 * max(1.0, np.abs(want_y[s]).max()), (s, at[s], n)
        at[0] += n0
        at[1] += n1
    assert at == lens


@pytest.mark.parametrize("T,inner,groups", [(5, 36, 3), (11, 1000, 2), (3, 1200, 1), (2, 9000, 1)])
def test_gate_comes_before_the_group_norm(T, inner, groups):
    """Parts short and long: the last one has more elements than a block's threads keep in registers."""
    from turboquant_cpp_b200.kernels import ssm as KS
    rng = np.random.default_rng(6)
    y, proj, w = rng.standard_normal((T, inner)), rng.standard_normal((T, inner + 9)), 1 + 0.1 * rng.standard_normal(inner)
    out = torch.empty((T, inner), dtype=torch.float32, device=DEV)
    KS.gated_group_norm(dev(y), dev(proj), 0, dev(w), groups, 1e-5, out)
    f32 = lambda a: dev(a).cpu().numpy().astype(np.float64)
    g = f32(y) * P.silu(f32(proj)[:, :inner])
    want = P.rms(g.reshape(T, groups, -1), 1e-5).reshape(T, inner) * f32(w)
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5


@pytest.mark.parametrize("H,R,rot,lead", [(16, 512, 64, 128), (6, 128, 32, 24), (20, 64, 16, 8), (5, 160, 32, 16), (3, 32, 0, 8),
                                           (7, 64, 48, 8), (9, 448, 32, 64)])
def test_tensor_core_form_agrees_with_the_float32_token_form(H, R, rot, lead):
    """The same bfloat16-rounded queries and rows through the bfloat16 kernel (tensor-core form at these sizes: four or
    eight warps, odd and even numbers of 16-element steps, one to eight output tiles a warp) and through the float32
    token form: they may differ by the rounding of the weights and of the output (2^-8 of a row's largest element),
    which a dropped step of a row or a key's wrong place would exceed many times."""
    from turboquant_cpp_b200.kernels import latent_attention as KL
    assert KL.tensor_core_form(torch.bfloat16, R, rot)
    gen = torch.Generator(device="cpu").manual_seed(R + rot)
    T, window, ctx, ps = 6, 700, 1500, 64
    Dk, pages_per = R + rot, 1500 // 64 + 1
    r32 = lambda *shape, s: (torch.randn(shape, generator=gen) * s).to(torch.bfloat16).float().to(DEV)
    cache32 = r32(T * pages_per, 1, 1, ps, Dk, s=0.5)
    table = torch.arange(T * pages_per, dtype=torch.int32, device=DEV).view(T, pages_per)
    q_lat32, q32 = r32(T, H, R, s=0.15), r32(T, H * (lead + rot), s=0.15)
    sink = torch.randn(H, generator=gen).to(DEV)
    pos, seq = i32([ctx - 1, 0, 5, window, window - 1, 1234]), i32(list(range(T)))
    for n_splits in (1, 5):
        outs = {}
        for dt in (torch.float32, torch.bfloat16):
            out = torch.empty((T, H, R), dtype=dt, device=DEV)
            partial = torch.empty(T * H * n_splits * (R + 2), dtype=torch.float32, device=DEV)
            KL.latent_attention(q_lat32.to(dt), q32.to(dt), lead, cache32.to(dt), sink, pos, seq, table, ps, window, 0.11, out,
                                H, R, rot, n_splits, partial)
            outs[dt] = out.float()
        ref, got = outs[torch.float32], outs[torch.bfloat16]
        err = ((got - ref).abs() / ref.abs().amax(dim=-1, keepdim=True)).max().item()
        assert err < 6e-3, f"{n_splits} ranges: {err:.2e}"

// Attention with a learned distance bias, a window that keeps a sequence's first positions, and a sink in the
// softmax's denominator, over a paged cache whose rows hold a key and a value of different sizes.
//
//   score(i, j) = q_i . k_j * scale + bias[min(i - j, far)][head]        (bias: a table per distance, or none)
//   i sees j    iff j <= i and (window == 0 or i - j < window or j < keep_first)
//   p_j         = exp(score_j) / (exp(sink[head]) + sum over the visible j of exp(score_j))   (sink: per head, or none)
//   out_i       = sum_j p_j v_j
//
// Query head h reads key/value head h / (heads / kv heads).  Scores, the softmax and the weighted sums are fp32.
// Cache layout of one layer: [page][kv head][slot in page][dk + dv], a position's key followed by its value; a
// sequence's position p lives in page table[seq][p / page_size] at slot p % page_size.
//
//   tq_bias_kv_write       splits a fused projection [q | k | v] (fp32): queries to a buffer, keys and values into the
//                          cache; values may be mixed with another layer's values of the same token,
//                          v <- (1 - lambda) v + lambda v_other, and may be kept (unmixed or mixed, as cached) for such
//                          a layer to read
//   tq_bias_attention      every (token, head) on its own, its visible keys cut into n_splits ranges (decode steps,
//                          short runs; any sizes, both dtypes) + the merge of the ranges
//   tq_bias_attention_runs runs of new tokens (prompts): a block's queries share tiles of keys and values through
//                          shared memory
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define BA_MAX_DIM 256
#define BA_WARPS 4
#define BA_EPL (BA_MAX_DIM / 32)      // elements of a key or a value per lane

// ---------------------------------------------------------------------------------------
// One block per token walks the elements of its fused row.
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void bias_kv_write_kernel(const float* __restrict__ qkv, TA* __restrict__ q_out, TA* __restrict__ cache,
                                     float* __restrict__ v_keep, const float* __restrict__ v_other, float lambda,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                     const int* __restrict__ page_table, int table_stride, int page_size,
                                     int nh, int nkv, int dk, int dv, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const int nq = nh * dk, nk = nkv * dk, nv = nkv * dv;
    const float* row = qkv + (size_t)t * (nq + nk + nv);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q_out[(size_t)t * nq + i] = tq_from_float<TA>(row[i]);
    if (cache == nullptr && v_keep == nullptr) return;
    const int pos = positions[t];
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;
    const int page = TQ_CHECKED(table[TQ_CHECKED(pos / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
    const int slot = pos % page_size, dr = dk + dv;
    for (int i = threadIdx.x; i < nk + nv; i += blockDim.x) {
        float v = row[nq + i];
        int g, e;
        if (i < nk) { g = i / dk; e = i % dk; }
        else {
            const int j = i - nk;
            g = j / dv; e = dk + j % dv;
            if (v_other) v = (1.0f - lambda) * v + lambda * v_other[(size_t)t * nv + j];
            if (v_keep) v_keep[(size_t)t * nv + j] = v;
        }
        if (cache) cache[(((size_t)page * nkv + g) * page_size + slot) * dr + e] = tq_from_float<TA>(v);
    }
}

TQ_EXPORT int tq_bias_kv_write(const float* qkv, void* q_out, void* cache, int act_dtype, float* v_keep,
                               const float* v_other, float lambda, const int* positions, const int* seq_of_token,
                               const int* page_table, int table_stride, int page_size, int T_, int nh, int nkv, int dk,
                               int dv, int n_seqs, int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(nh >= 1 && nkv >= 1 && dk >= 1 && dv >= 1, "bias_kv_write: bad sizes %d %d %d %d", nh, nkv, dk, dv);
    const int n = nh * dk + nkv * (dk + dv);
    const int threads = n >= 1024 ? 512 : (n >= 256 ? 256 : 128);
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch(T_, threads, 0, stream)(bias_kv_write_kernel<TA>, qkv, (TA*)q_out, (TA*)cache, v_keep, v_other, lambda,
            positions, seq_of_token, page_table, table_stride, page_size, nh, nkv, dk, dv, n_seqs, n_pages)));
    TQ_CHECK_LAUNCH("bias_kv_write");
    return 0;
}

// The visible positions of a query at `pos`, in order: [0, n_first) and [start, pos].
struct BaSpan {
    int n_first, start, count;
    __device__ __forceinline__ int at(int n) const { return n < n_first ? n : start + (n - n_first); }
};
__device__ __forceinline__ BaSpan ba_span(int pos, int window, int keep_first) {
    BaSpan s;
    s.start = window > 0 ? max(0, pos + 1 - window) : 0;
    s.n_first = min(keep_first, s.start);
    s.count = s.n_first + (pos + 1 - s.start);
    return s;
}

// ---------------------------------------------------------------------------------------
// Token form: grid (T, heads, n_splits), 4 warps.  The block's range of the visible positions is walked key by key,
// warp w taking every fourth; a lane holds elements lane, lane + 32, ... of the key and of the value; online softmax
// per warp, merged through shared memory in warp order.  The sink enters as the first warp's starting state in the
// first range.  With n_splits > 1 the block's state (max, sum, weighted values) goes to `partial`.
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(BA_WARPS * 32)
bias_attention_kernel(const TA* __restrict__ q, const TA* __restrict__ cache, const float* __restrict__ bias, int far,
                      const float* __restrict__ sink, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int table_stride,
                      int page_size, int window, int keep_first, float scale, TA* __restrict__ out,
                      float* __restrict__ partial, int n_splits, int nh, int nkv, int dk, int dv, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_m[BA_WARPS], s_l[BA_WARPS];
    __shared__ float s_acc[BA_WARPS][BA_MAX_DIM];
    const int t = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = h / (nh / nkv), dr = dk + dv;
    const int pos = positions[t];
    const BaSpan span = ba_span(pos, window, keep_first);
    const int per = (span.count + n_splits - 1) / n_splits;
    const int n0 = split * per, n1 = min(span.count, n0 + per);
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;

    float qv[BA_EPL], acc[BA_EPL];
    const TA* qp = q + ((size_t)t * nh + h) * dk;
#pragma unroll
    for (int j = 0; j < BA_EPL; ++j) {
        const int e = lane + 32 * j;
        qv[j] = e < dk ? tq_to_float(qp[e]) * scale : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    if (sink != nullptr && split == 0 && warp == 0) { m = sink[h]; l = 1.f; }
    for (int n = n0 + warp; n < n1; n += BA_WARPS) {
        const int p = span.at(n);
        const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const TA* kp = cache + (((size_t)page * nkv + g) * page_size + p % page_size) * dr;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < BA_EPL; ++j) {
            const int e = lane + 32 * j;
            if (e < dk) s += qv[j] * tq_to_float(kp[e]);
        }
        s = tq_warp_sum(s);
        if (bias) s += bias[(size_t)min(pos - p, far) * nh + h];
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);          // exp(-inf) = 0 on the first key
        const float pexp = expf(s - m_new);
        l = l * corr + pexp;
#pragma unroll
        for (int j = 0; j < BA_EPL; ++j) {
            const int e = lane + 32 * j;
            if (e < dv) acc[j] = acc[j] * corr + pexp * tq_to_float(kp[dk + e]);
        }
        m = m_new;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < BA_EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < dv) s_acc[warp][e] = acc[j];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < BA_WARPS; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f;
    float f[BA_WARPS];
#pragma unroll
    for (int w = 0; w < BA_WARPS; ++w) {
        f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);
        L += s_l[w] * f[w];
    }
    if (n_splits > 1) {
        float* pr = partial + (((size_t)t * nh + h) * n_splits + split) * (dv + 2);
        if (threadIdx.x == 0) { pr[0] = M; pr[1] = L; }
        for (int e = threadIdx.x; e < dv; e += blockDim.x) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < BA_WARPS; ++w) v += s_acc[w][e] * f[w];
            pr[2 + e] = v;
        }
        return;
    }
    TA* op = out + ((size_t)t * nh + h) * dv;
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < BA_WARPS; ++w) v += s_acc[w][e] * f[w];
        op[e] = tq_from_float<TA>(v / L);
    }
}

// The ranges of one (token, head), added up in range order: grid (T * heads).
template <typename TA>
__global__ void bias_attention_merge_kernel(const float* __restrict__ partial, int n_splits, int dv, TA* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const float* p = partial + (size_t)blockIdx.x * n_splits * (dv + 2);
    float M = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) M = fmaxf(M, p[(size_t)sp * (dv + 2)]);
    float L = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
        const float ms = p[(size_t)sp * (dv + 2)];
        if (ms != -INFINITY) L += p[(size_t)sp * (dv + 2) + 1] * expf(ms - M);
    }
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float a = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float ms = p[(size_t)sp * (dv + 2)];
            if (ms != -INFINITY) a += p[(size_t)sp * (dv + 2) + 2 + e] * expf(ms - M);
        }
        out[(size_t)blockIdx.x * dv + e] = tq_from_float<TA>(a / L);
    }
}

TQ_EXPORT int tq_bias_attention(const void* q, const void* cache, int act_dtype, const float* bias, int far,
                                const float* sink, const int* positions, const int* seq_of_token,
                                const int* page_table, int table_stride, int page_size, int window, int keep_first,
                                float scale, void* out, float* partial, int n_splits, int T_, int nh, int nkv, int dk,
                                int dv, int n_seqs, int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(dk >= 1 && dk <= BA_MAX_DIM && dv >= 1 && dv <= BA_MAX_DIM, "bias_attention: key size %d or value size %d exceeds %d", dk, dv, BA_MAX_DIM);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "bias_attention: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE(nh <= 65535 && n_splits >= 1 && n_splits <= 65535, "bias_attention: %d heads or %d ranges exceed the grid limit", nh, n_splits);
    TQ_REQUIRE(window >= 0 && keep_first >= 0 && far >= 0, "bias_attention: negative window, kept positions or distance");
    TQ_REQUIRE(n_splits == 1 || partial != nullptr, "bias_attention: %d ranges need scratch for their states", n_splits);
    dim3 grid(T_, nh, n_splits);
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch(grid, BA_WARPS * 32, 0, stream)(bias_attention_kernel<TA>, (const TA*)q, (const TA*)cache, bias, far, sink,
            positions, seq_of_token, page_table, table_stride, page_size, window, keep_first, scale, (TA*)out, partial,
            n_splits, nh, nkv, dk, dv, n_seqs, n_pages)));
    TQ_CHECK_LAUNCH("bias_attention");
    if (n_splits > 1) {
        TQ_DISPATCH(act_dtype, TA,
            (tq_launch(T_ * nh, dv >= 128 ? 128 : 64, 0, stream)(bias_attention_merge_kernel<TA>, partial, n_splits, dv, (TA*)out)));
        TQ_CHECK_LAUNCH("bias_attention_merge");
    }
    return 0;
}

// Attention over a cache of latent rows.
//
// A layer of this kind caches ONE row per position, shared by all heads: [c | kr], the latent c (R elements, already
// normed) and a rotated key part kr (rot elements).  Head a's key is W_uk,a c and its value W_uv,a c, so with
//   q~_a = W_uk,a^T q_a            (the query carried into the latent space, R elements)
// the score is (q~_a . c + q_a,rot . kr) * scale and the head's output is W_uv,a applied to sum_j p_j c_j: attention
// with one key/value head whose value is the first R elements of its key row.  The two products with W_uk and W_uv
// are batched matrix products outside; the kernels here are
//   latent_prepare    norm of the latent, rotation of kr and of the queries' rotated part, cache write
//   latent_attention  scores, softmax with an optional sink per head, weighted sum of latents
//   latent_merge      joins the key ranges of a split launch
// and, for long runs of new tokens (prompts), where scores and sums are matrix products of the library,
//   latent_gather     a range of one sequence's rows from the pages into a dense matrix
//   latent_softmax    rows of scores -> weights: mask (causal, window), scale, softmax with the sink
// Scores, softmax and sums are fp32.  A sink is a learned logit per head that takes part in the softmax's
// denominator and has no value: out = sum_j e^{s_j - M} c_j / (sum_j e^{s_j - M} + e^{sink - M}).
// Window w > 0: position i sees j with 0 <= i - j < w.
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define LAT_MAX_ROW 1024      // R + rot at most
#define LAT_WARPS 4
#define LAT_HG 4              // heads per block: they share every key row the block loads

// ---------------------------------------------------------------------------------------
// latent_prepare: one block per token.
//   dkv given: row = [ d[0:R] / sqrt(mean(d[0:R]^2) + eps) * wnorm | rotate(d[R:R+rot]) ] -> cache at the token's place
//   q: the rotated part of every head (elements q_off .. q_off+rot of a head of q_dim elements) turns in place
// Rotation: pairs (2i, 2i+1), i < n_pairs, angle = position * freq[i] in fp32, cos and sin times mag; elements
// beyond 2 n_pairs pass unchanged.
// ---------------------------------------------------------------------------------------
template <typename TA, typename TW>
__global__ void latent_prepare_kernel(TA* __restrict__ q, const float* __restrict__ dkv, const TW* __restrict__ wnorm,
                                      float eps, const float* __restrict__ freq, float mag,
                                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                      const int* __restrict__ page_table, int table_stride, int page_size,
                                      TA* __restrict__ cache, int heads, int q_dim, int q_off, int rot, int n_pairs,
                                      int R, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    __shared__ float s_cos[LAT_MAX_ROW / 2], s_sin[LAT_MAX_ROW / 2];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const float fpos = (float)pos;
    // the token's cos and sin once (times mag), for the key part and for every head
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        float s, c;
        sincosf(fpos * freq[i], &s, &c);
        s_cos[i] = c * mag;
        s_sin[i] = s * mag;
    }
    __syncthreads();
    if (dkv) {
        const float* d = dkv + (size_t)t * (R + rot);
        float ss = 0.f;
        for (int i = threadIdx.x; i < R; i += blockDim.x) ss += d[i] * d[i];
        ss = tq_block_sum(ss, scratch);
        const float rs = 1.0f / sqrtf(ss / (float)R + eps);
        const int seq = TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE);
        const int page = TQ_CHECKED(page_table[(size_t)seq * table_stride + TQ_CHECKED(pos / page_size, table_stride, TQ_IDX_TABLE_COLUMN)],
                                    n_pages, TQ_IDX_PAGE);
        TA* row = cache + ((size_t)page * page_size + pos % page_size) * (R + rot);
        for (int i = threadIdx.x; i < R; i += blockDim.x) row[i] = tq_from_float<TA>(d[i] * rs * tq_to_float(wnorm[i]));
        for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
            const float s = s_sin[i], c = s_cos[i];
            const float u = d[R + 2 * i], v = d[R + 2 * i + 1];
            row[R + 2 * i] = tq_from_float<TA>(u * c - v * s);
            row[R + 2 * i + 1] = tq_from_float<TA>(v * c + u * s);
        }
        for (int e = 2 * n_pairs + threadIdx.x; e < rot; e += blockDim.x) row[R + e] = tq_from_float<TA>(d[R + e]);
    }
    for (int k = threadIdx.x; k < heads * n_pairs; k += blockDim.x) {
        const int h = k / n_pairs, i = k % n_pairs;
        const float s = s_sin[i], c = s_cos[i];
        TA* p = q + ((size_t)t * heads + h) * q_dim + q_off + 2 * i;
        const float u = tq_to_float(p[0]), v = tq_to_float(p[1]);
        p[0] = tq_from_float<TA>(u * c - v * s);
        p[1] = tq_from_float<TA>(v * c + u * s);
    }
}

TQ_EXPORT int tq_latent_prepare(void* q, int act_dtype, const float* dkv, const void* wnorm, int w_dtype, float eps,
                                const float* freq, float mag, const int* positions, const int* seq_of_token,
                                const int* page_table, int table_stride, int page_size, void* cache, int T_, int heads,
                                int q_dim, int q_off, int rot, int n_pairs, int R, int n_seqs, int n_pages,
                                cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(heads >= 1 && R >= 1 && rot >= 0 && R + rot <= LAT_MAX_ROW, "latent_prepare: bad sizes R=%d rot=%d", R, rot);
    TQ_REQUIRE(2 * n_pairs <= rot && q_off >= 0 && q_off + rot <= q_dim, "latent_prepare: the rotated part does not fit "
               "(pairs %d, rot %d, offset %d, head %d)", n_pairs, rot, q_off, q_dim);
    TQ_REQUIRE(!dkv || (cache && page_table && wnorm), "latent_prepare: a projection to cache needs a cache and a norm");
    TQ_REQUIRE(n_pairs == 0 || freq, "latent_prepare: a rotation needs frequencies");
    TQ_DISPATCH(act_dtype, TA, TQ_DISPATCH(w_dtype, TW,
        (tq_launch(T_, 128, 0, stream)(latent_prepare_kernel<TA, TW>, (TA*)q, dkv, (const TW*)wnorm, eps, freq, mag,
                                       positions, seq_of_token, page_table, table_stride, page_size, (TA*)cache, heads,
                                       q_dim, q_off, rot, n_pairs, R, n_seqs, n_pages))));
    TQ_CHECK_LAUNCH("latent_prepare");
    return 0;
}

// ---------------------------------------------------------------------------------------
// latent_attention: grid (tokens, ceil(heads / LAT_HG), n_splits), LAT_WARPS warps.  The block's keys (its share of
// the token's range) go round the warps in groups of neighbours; a lane holds EPL elements of the row in groups of VEC neighbours
// (element VEC*lane + 32*VEC*j + c), so a warp reads a row with 8- or 16-byte loads; the LAT_HG heads' queries
// lie in shared memory.  Each warp keeps an online softmax per head; the warps' states are joined through shared
// memory in warp order.  n_splits == 1: the sink joins and the result is written; otherwise the block's state
// (max, sum, R weighted elements) goes to `partial` and latent_merge finishes.
// ---------------------------------------------------------------------------------------
template <typename TA, int VEC> struct LatRow;
template <> struct LatRow<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float* o) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
};
template <> struct LatRow<__nv_bfloat16, 4> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    }
};
template <typename TA> struct LatRow<TA, 1> {
    static __device__ __forceinline__ void load(const TA* p, float* o) { o[0] = tq_to_float(*p); }
};

template <typename TA, int EPL, int VEC>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_attention_kernel(const TA* __restrict__ q_lat, const TA* __restrict__ q, int q_dim, int q_off,
                        const TA* __restrict__ cache, const float* __restrict__ sink,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        const int* __restrict__ page_table, int table_stride, int page_size, int window, float scale,
                        TA* __restrict__ out, float* __restrict__ partial, int H, int R, int rot, int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ float lat_smem[];
    __shared__ float s_m[LAT_WARPS][LAT_HG], s_l[LAT_WARPS][LAT_HG];
    constexpr int NG = EPL / VEC;
    const int Dk = R + rot;
    float* qs = lat_smem;                       // [LAT_HG][Dk]
    float* s_acc = lat_smem + LAT_HG * Dk;      // [LAT_WARPS][R]
    const int t = blockIdx.x, h0 = blockIdx.y * LAT_HG;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {   // the heads' queries: every thread's loads are issued together (at most EPL of them), then stored
        float tmp[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int k = threadIdx.x + i * LAT_WARPS * 32;
            const int g = k / Dk, e = k - g * Dk, h = h0 + g;
            tmp[i] = 0.f;
            if (k < LAT_HG * Dk && h < H)
                tmp[i] = e < R ? tq_to_float(q_lat[((size_t)t * H + h) * R + e])
                               : tq_to_float(q[((size_t)t * H + h) * q_dim + q_off + (e - R)]);
        }
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int k = threadIdx.x + i * LAT_WARPS * 32;
            if (k < LAT_HG * Dk) qs[k] = tmp[i];
        }
    }
    __syncthreads();
    const int pos = positions[t];
    const int first = window > 0 ? max(0, pos + 1 - window) : 0;
    const int n_keys = pos + 1 - first;
    const int per = (n_keys + (int)gridDim.z - 1) / (int)gridDim.z;
    const int lo = first + (int)blockIdx.z * per, hi = min(pos + 1, lo + per);
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;

    float m[LAT_HG], l[LAT_HG], acc[LAT_HG][EPL];
#pragma unroll
    for (int g = 0; g < LAT_HG; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc[g][j] = 0.f;
    }
    // A warp takes KB neighbouring keys at a time: their rows are asked for together, the KB x LAT_HG scores are
    // summed over the lanes side by side (independent chains of shuffles), and the online softmax moves once per
    // group of keys.
    constexpr int KB = EPL <= 20 ? 4 : 2;
    for (int p0 = lo + warp * KB; p0 < hi; p0 += LAT_WARPS * KB) {
        float kr[KB][EPL];
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const int p = min(p0 + b, hi - 1);           // a group's missing keys repeat its last one and get no weight
            const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
            const TA* kp = cache + ((size_t)page * page_size + p % page_size) * Dk;
#pragma unroll
            for (int j = 0; j < NG; ++j) {
                const int e = VEC * lane + 32 * VEC * j;
                if (e < Dk) LatRow<TA, VEC>::load(kp + e, &kr[b][VEC * j]);
                else {
#pragma unroll
                    for (int c = 0; c < VEC; ++c) kr[b][VEC * j + c] = 0.f;
                }
            }
        }
        float sc[LAT_HG][KB];
#pragma unroll
        for (int g = 0; g < LAT_HG; ++g) {
#pragma unroll
            for (int b = 0; b < KB; ++b) sc[g][b] = 0.f;
#pragma unroll
            for (int j = 0; j < NG; ++j) {
                const int e = VEC * lane + 32 * VEC * j;
                if (e < Dk) {
#pragma unroll
                    for (int c = 0; c < VEC; ++c) {
                        const float qv = qs[g * Dk + e + c];
#pragma unroll
                        for (int b = 0; b < KB; ++b) sc[g][b] += qv * kr[b][VEC * j + c];
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int g = 0; g < LAT_HG; ++g) {
#pragma unroll
                for (int b = 0; b < KB; ++b) sc[g][b] += __shfl_xor_sync(0xffffffffu, sc[g][b], o);
            }
        }
#pragma unroll
        for (int g = 0; g < LAT_HG; ++g) {
            float m_new = m[g];
#pragma unroll
            for (int b = 0; b < KB; ++b) {
                sc[g][b] *= scale;
                if (p0 + b < hi) m_new = fmaxf(m_new, sc[g][b]);
            }
            const float corr = expf(m[g] - m_new);          // exp(-inf) = 0 on the first keys
            l[g] *= corr;
#pragma unroll
            for (int j = 0; j < EPL; ++j) acc[g][j] *= corr;
#pragma unroll
            for (int b = 0; b < KB; ++b) {
                const float pe = p0 + b < hi ? expf(sc[g][b] - m_new) : 0.f;
                l[g] += pe;
#pragma unroll
                for (int j = 0; j < EPL; ++j) acc[g][j] += pe * kr[b][j];
            }
            m[g] = m_new;
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < LAT_HG; ++g) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
    }
#pragma unroll
    for (int g = 0; g < LAT_HG; ++g) {
        __syncthreads();                 // the round before has been read
#pragma unroll
        for (int j = 0; j < NG; ++j) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                const int e = VEC * lane + 32 * VEC * j + c;
                if (e < R) s_acc[warp * R + e] = acc[g][VEC * j + c];
            }
        }
        __syncthreads();
        const int h = h0 + g;
        if (h >= H) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < LAT_WARPS; ++w) M = fmaxf(M, s_m[w][g]);
        const bool whole = gridDim.z == 1;
        const float sk = (whole && sink) ? sink[h] : -INFINITY;
        M = fmaxf(M, sk);
        float f[LAT_WARPS], L = 0.f;
#pragma unroll
        for (int w = 0; w < LAT_WARPS; ++w) {
            f[w] = s_m[w][g] == -INFINITY ? 0.f : expf(s_m[w][g] - M);
            L += s_l[w][g] * f[w];
        }
        if (whole) {
            if (sink) L += expf(sk - M);
            TA* op = out + ((size_t)t * H + h) * R;
            for (int e = threadIdx.x; e < R; e += blockDim.x) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < LAT_WARPS; ++w) v += s_acc[w * R + e] * f[w];
                op[e] = tq_from_float<TA>(v / L);
            }
        } else {
            float* pp = partial + (((size_t)t * H + h) * gridDim.z + blockIdx.z) * (R + 2);
            if (threadIdx.x == 0) { pp[0] = M; pp[1] = L; }      // an empty range leaves M = -inf, L = 0
            for (int e = threadIdx.x; e < R; e += blockDim.x) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < LAT_WARPS; ++w) v += s_acc[w * R + e] * f[w];
                pp[2 + e] = v;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// The same on tensor cores (bfloat16, R a multiple of 32 up to 512, R + rot a multiple of 16): the block's sixteen
// heads are the sixteen rows of mma.sync m16n8k16, so one cached row serves sixteen dot products per
// instruction.  Keys come in tiles of 32 through a two-stage ring in shared memory, filled by 16-byte cp.async
// copies a tile ahead.  Of a tile's scores (16 heads x 32 keys) every warp computes a group of eight keys (with
// eight warps, where R is a multiple of 64, half of the row's elements for it; fp32 accumulators; scale and mask
// on the fragments) and leaves them in shared memory; after a barrier
// every warp reads all of them, keeps the online softmax of its two rows (all warps the same numbers) and
// multiplies the weights, rounded to bfloat16 as the second operand's type demands, with the tile's rows for the
// share of the R output columns that it owns.  Fragments come from shared memory by ldmatrix (transposed for
// the rows as values).
// ---------------------------------------------------------------------------------------
#define LATM_HEADS 16
#define LATM_KEYS 32
#define LATM_PAD 8            // bfloat16 elements between rows in shared memory: eight rows' 16-byte pieces hit all banks
#define LATM_PS 40            // floats per row of the scores' exchange area

__device__ __forceinline__ void lat_mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lat_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// ldmatrix from a shared-memory address (32 bits, bytes)
__device__ __forceinline__ void lat_ldsm4(uint32_t* r, unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a) : "memory");
}
__device__ __forceinline__ void lat_ldsm2(uint32_t* r, unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(a) : "memory");
}
__device__ __forceinline__ void lat_ldsm4_t(uint32_t* r, unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a) : "memory");
}
// NW warps (4 or 8); OT output n-tiles (of 8 columns) per warp: R = 8 * NW * OT.  With eight warps two warps share a
// group of eight keys, each taking half of the row's elements, and their partial scores meet in shared memory.
template <int OT, int NW>
__global__ void __launch_bounds__(NW * 32, 2)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q_lat, const __nv_bfloat16* __restrict__ q, int q_dim,
                            int q_off, const __nv_bfloat16* __restrict__ cache, const float* __restrict__ sink,
                            const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ page_table, int table_stride, int page_size, int window, float scale,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int H, int R, int rot,
                            int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ uint4 latm_smem[];
    const int Dk = R + rot, ld = Dk + LATM_PAD;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(latm_smem);       // [16 heads][ld]
    __nv_bfloat16* Ks = Qs + LATM_HEADS * ld;                               // [2][32 keys][ld]
    float* Ps = reinterpret_cast<float*>(Ks + 2 * LATM_KEYS * ld);          // [NW / 4][16 heads][LATM_PS]
    const int t = blockIdx.x, h0 = blockIdx.y * LATM_HEADS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tq = lane & 3;
    const int chunks = Dk / 8;                                              // 16-byte pieces of a row
    const int pos = positions[t];
    const int first = window > 0 ? max(0, pos + 1 - window) : 0;
    const int n_keys = pos + 1 - first;
    const int per = (n_keys + (int)gridDim.z - 1) / (int)gridDim.z;
    const int lo = first + (int)blockIdx.z * per, hi = min(pos + 1, lo + per);
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;

    // a tile's rows go round the warps; a lane copies every 32nd piece of a row (rows beyond the range as zeros)
    // a tile's rows go round the warps (row r to warp r % NW); the first lanes each find one of the warp's rows in
    // the pages, the others get the place by shuffle; a lane copies every 32nd piece of a row (rows beyond the
    // range as zeros)
    const unsigned ks_s = (unsigned)__cvta_generic_to_shared(Ks);
    auto fetch = [&](int p0, int stage) {
        long long mine = -1;
        {
            const int p = p0 + warp + NW * (lane % (LATM_KEYS / NW));
            if (p < hi) {
                const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
                mine = ((long long)page * page_size + p % page_size) * Dk;
            }
        }
        const unsigned dst = ks_s + (unsigned)(stage * LATM_KEYS * ld) * 2u;
#pragma unroll
        for (int i = 0; i < LATM_KEYS / NW; ++i) {
            const long long off = __shfl_sync(0xffffffffu, mine, i);
            const int r = warp + NW * i;
            const __nv_bfloat16* src = cache + (off < 0 ? 0 : off);
            const int bytes = off < 0 ? 0 : 16;
            for (int c = lane; c < chunks; c += 32)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                             ::"r"(dst + (unsigned)(r * ld + 8 * c) * 2u), "l"(src + (bytes ? 8 * c : 0)), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (lo < hi) fetch(lo, 0);
    {   // the heads' queries, 16 bytes at a time (heads beyond H as zeros)
        const int rc = rot / 8, lc = R / 8;
        const bool rot_vec = (q_dim % 8 == 0) && (q_off % 8 == 0);
        for (int k = threadIdx.x; k < LATM_HEADS * lc; k += blockDim.x) {
            const int r = k / lc, c = k - r * lc, h = h0 + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (h < H) v = reinterpret_cast<const uint4*>(q_lat + ((size_t)t * H + h) * R)[c];
            *reinterpret_cast<uint4*>(Qs + r * ld + 8 * c) = v;
        }
        if (rot_vec) {
            for (int k = threadIdx.x; k < LATM_HEADS * rc; k += blockDim.x) {
                const int r = k / rc, c = k - r * rc, h = h0 + r;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (h < H) v = reinterpret_cast<const uint4*>(q + ((size_t)t * H + h) * q_dim + q_off)[c];
                *reinterpret_cast<uint4*>(Qs + r * ld + R + 8 * c) = v;
            }
        } else {
            for (int k = threadIdx.x; k < LATM_HEADS * rot; k += blockDim.x) {
                const int r = k / rot, e = k - r * rot, h = h0 + r;
                Qs[r * ld + R + e] = h < H ? q[((size_t)t * H + h) * q_dim + q_off + e] : __float2bfloat16_rn(0.f);
            }
        }
    }

    float o[OT][4];
#pragma unroll
    for (int j = 0; j < OT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};                 // rows g and g + 8
    const int col_base = warp * OT * 8;
    // ldmatrix addresses: the queries' 16 x 16 piece (lane i: row i % 16, second eight columns for i >= 16), this
    // warp's eight keys (lane i: key i % 8, columns 8 * (i / 8) on), a tile's 32 rows as values (lane i: row i)
    const unsigned qa = (unsigned)__cvta_generic_to_shared(Qs + (lane & 15) * ld + 8 * (lane >> 4));
    const int nt = warp & 3, kp = warp >> 2;                   // the warp's group of eight keys; its part of the row (NW == 8)
    const unsigned kb_off = (unsigned)((8 * nt + (lane & 7)) * ld + 8 * (lane >> 3)) * 2u;
    const unsigned va_off = (unsigned)(lane * ld + warp * OT * 8) * 2u;
    const int ksteps = Dk / 16;
    const int ks_mid = NW == 8 ? ((ksteps / 2 + 1) & ~1) : ksteps;           // an even number of steps to the first part
    const int ks_lo = kp ? ks_mid : 0, ks_hi = kp ? ksteps : ks_mid;
    const float scale2 = scale * 1.4426950408889634f;           // scores in units of ln 2: the exponentials are exp2

    int stage = 0;
    for (int p0 = lo; p0 < hi; p0 += LATM_KEYS, stage ^= 1) {
        const unsigned kt = ks_s + (unsigned)(stage * LATM_KEYS * ld) * 2u;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                          // the tile has landed for all; the other stage and Ps are free
        if (p0 + LATM_KEYS < hi) fetch(p0 + LATM_KEYS, stage ^ 1);
        // scores of this warp's eight keys: four chains of accumulators, joined at the end
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
        float sc4[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
        int ks = ks_lo;
        for (; ks + 4 <= ks_hi; ks += 4) {
            uint32_t a0[4], a1[4], a2[4], a3[4], b0[4], b1[4];
            lat_ldsm4(a0, qa + 32 * ks);
            lat_ldsm4(a1, qa + 32 * ks + 32);
            lat_ldsm4(a2, qa + 32 * ks + 64);
            lat_ldsm4(a3, qa + 32 * ks + 96);
            lat_ldsm4(b0, kt + kb_off + 32 * ks);
            lat_ldsm4(b1, kt + kb_off + 32 * ks + 64);
            lat_mma16816(sa, a0, b0[0], b0[1]);
            lat_mma16816(sb, a1, b0[2], b0[3]);
            lat_mma16816(sc4, a2, b1[0], b1[1]);
            lat_mma16816(sd, a3, b1[2], b1[3]);
        }
        for (; ks + 2 <= ks_hi; ks += 2) {
            uint32_t a0[4], a1[4], b[4];
            lat_ldsm4(a0, qa + 32 * ks);
            lat_ldsm4(a1, qa + 32 * ks + 32);
            lat_ldsm4(b, kt + kb_off + 32 * ks);
            lat_mma16816(sa, a0, b[0], b[1]);
            lat_mma16816(sb, a1, b[2], b[3]);
        }
        if (ks < ks_hi) {
            uint32_t a0[4], b[2];
            lat_ldsm4(a0, qa + 32 * ks);
            lat_ldsm2(b, kt + kb_off + 32 * ks);      // lanes 0..15 give the addresses: columns 16 ks and 16 ks + 8
            lat_mma16816(sa, a0, b[0], b[1]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) sa[i] = (sa[i] + sb[i]) + (sc4[i] + sd[i]);
        {   // this lane holds keys 8 nt + 2 tq + {0, 1} of rows g (values 0, 1) and g + 8 (values 2, 3)
            const int kc = 8 * nt + 2 * tq;
            const bool s0 = p0 + kc < hi, s1 = p0 + kc + 1 < hi;
            float2 top, bot;
            top.x = s0 ? sa[0] * scale2 : -INFINITY;
            top.y = s1 ? sa[1] * scale2 : -INFINITY;
            bot.x = s0 ? sa[2] * scale2 : -INFINITY;
            bot.y = s1 ? sa[3] * scale2 : -INFINITY;
            float* pw = Ps + kp * LATM_HEADS * LATM_PS;
            *reinterpret_cast<float2*>(pw + g * LATM_PS + kc) = top;
            *reinterpret_cast<float2*>(pw + (g + 8) * LATM_PS + kc) = bot;
        }
        __syncthreads();
        // all 32 scores of rows g and g + 8, in the first operand's layout: sc[r][2 i + {0, 1}] = keys 8 i + 2 tq + {0, 1}
        float sc[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 v = *reinterpret_cast<const float2*>(Ps + (g + 8 * r) * LATM_PS + 8 * i + 2 * tq);
                if (NW == 8) {                      // the other part of the row (masked keys are -inf in both)
                    const float2 u = *reinterpret_cast<const float2*>(Ps + (LATM_HEADS + g + 8 * r) * LATM_PS + 8 * i + 2 * tq);
                    v.x += u.x;
                    v.y += u.y;
                }
                sc[r][2 * i] = v.x;
                sc[r][2 * i + 1] = v.y;
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float tmax = sc[r][0];
#pragma unroll
            for (int i = 1; i < 8; ++i) tmax = fmaxf(tmax, sc[r][i]);
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float m_new = fmaxf(m[r], tmax);             // finite: a tile has at least one key
            corr[r] = exp2f(m[r] - m_new);                      // 2^(-inf) = 0 on the first tile
            m[r] = m_new;
            l[r] *= corr[r];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sc[r][i] = exp2f(sc[r][i] - m_new);
                l[r] += sc[r][i];                               // this lane's share; the quad's shares are added at the end
            }
        }
        uint32_t pa[2][4];                                      // keys 0..15 and 16..31
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
            pa[k2][0] = lat_pack(sc[0][4 * k2], sc[0][4 * k2 + 1]);
            pa[k2][1] = lat_pack(sc[1][4 * k2], sc[1][4 * k2 + 1]);
            pa[k2][2] = lat_pack(sc[0][4 * k2 + 2], sc[0][4 * k2 + 3]);
            pa[k2][3] = lat_pack(sc[1][4 * k2 + 2], sc[1][4 * k2 + 3]);
        }
#pragma unroll
        for (int j = 0; j < OT; ++j) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
            uint32_t b[4];
            lat_ldsm4_t(b, kt + va_off + 16 * j);
            lat_mma16816(o[j], pa[0], b[0], b[1]);
            lat_mma16816(o[j], pa[1], b[2], b[3]);
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        m[r] *= 0.6931471805599453f;                            // back to natural units for the sink and the merge
    }
    const bool whole = gridDim.z == 1;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int h = h0 + g + 8 * r;
        if (h >= H) continue;
        if (whole) {
            const float sk = sink ? sink[h] : -INFINITY;
            const float M = fmaxf(m[r], sk);
            const float f = m[r] == -INFINITY ? 0.f : expf(m[r] - M);
            const float inv = 1.0f / (l[r] * f + (sink ? expf(sk - M) : 0.f));
            __nv_bfloat16* op = out + ((size_t)t * H + h) * R + col_base + 2 * tq;
#pragma unroll
            for (int j = 0; j < OT; ++j)
                *reinterpret_cast<__nv_bfloat162*>(op + j * 8) = __floats2bfloat162_rn(o[j][2 * r] * f * inv, o[j][2 * r + 1] * f * inv);
        } else {
            float* pp = partial + (((size_t)t * H + h) * gridDim.z + blockIdx.z) * (R + 2);
            if (warp == 0 && tq == 0) { pp[0] = m[r]; pp[1] = l[r]; }       // an empty range leaves -inf and 0
#pragma unroll
            for (int j = 0; j < OT; ++j)
                *reinterpret_cast<float2*>(pp + 2 + col_base + j * 8 + 2 * tq) = make_float2(o[j][2 * r], o[j][2 * r + 1]);
        }
    }
}

// joins the ranges of one (token, head) in range order and lets the sink take part: the first warp turns the
// ranges' maxima and sums into one weight per range (the sink only adds to the denominator), then every thread
// adds up one element over the ranges; grid (tokens, heads, ceil(R / LAT_MERGE_THREADS))
#define LAT_MAX_SPLITS 64
#define LAT_MERGE_THREADS 128
template <typename TA>
__global__ void latent_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sink, int n_splits,
                                    int H, int R, TA* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float wgt[LAT_MAX_SPLITS];
    const int t = blockIdx.x, h = blockIdx.y;
    const float* pp = partial + ((size_t)t * H + h) * n_splits * (R + 2);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float sk = sink ? sink[h] : -INFINITY;
        float ms[LAT_MAX_SPLITS / 32], ls[LAT_MAX_SPLITS / 32], M = sk;
#pragma unroll
        for (int i = 0; i < LAT_MAX_SPLITS / 32; ++i) {
            const int s = lane + 32 * i;
            ms[i] = s < n_splits ? pp[(size_t)s * (R + 2)] : -INFINITY;
            ls[i] = s < n_splits ? pp[(size_t)s * (R + 2) + 1] : 0.f;
            M = fmaxf(M, ms[i]);
        }
        M = tq_warp_max(M);                              // finite: some range holds a key
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < LAT_MAX_SPLITS / 32; ++i) {
            ms[i] = ms[i] == -INFINITY ? 0.f : expf(ms[i] - M);
            L += ls[i] * ms[i];
        }
        L = tq_warp_sum(L) + (sink ? expf(sk - M) : 0.f);
#pragma unroll
        for (int i = 0; i < LAT_MAX_SPLITS / 32; ++i) wgt[lane + 32 * i] = ms[i] / L;
    }
    __syncthreads();
    const int e = blockIdx.z * LAT_MERGE_THREADS + threadIdx.x;
    if (e >= R) return;
    float v = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) v += pp[(size_t)s * (R + 2) + 2 + e] * wgt[s];
    out[((size_t)t * H + h) * R + e] = tq_from_float<TA>(v);
}

// TQ_LATENT_NO_MMA=1: the CUDA-core form for bfloat16 too
static bool lat_use_mma() {
    static const bool on = [] { const char* e = getenv("TQ_LATENT_NO_MMA"); return !(e && e[0] && e[0] != '0'); }();
    return on;
}

#define LAT_LAUNCH(TA, EPL, VEC)                                                                                  \
    tq_launch(grid, LAT_WARPS * 32, smem, stream)(latent_attention_kernel<TA, EPL, VEC>, (const TA*)q_lat,        \
        (const TA*)q, q_dim, q_off, (const TA*)cache, sink, positions, seq_of_token, page_table, table_stride,    \
        page_size, window, scale, (TA*)out, partial, H, R, rot, n_seqs, n_pages)

TQ_EXPORT int tq_latent_attention(const void* q_lat, const void* q, int q_dim, int q_off, const void* cache,
                                  int act_dtype, const float* sink, const int* positions, const int* seq_of_token,
                                  const int* page_table, int table_stride, int page_size, int window, float scale,
                                  void* out, float* partial, int n_splits, int T_, int H, int R, int rot, int n_seqs,
                                  int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    const int Dk = R + rot;
    TQ_REQUIRE(H >= 1 && R >= 1 && rot >= 0 && Dk <= LAT_MAX_ROW, "latent_attention: a row of %d + %d elements exceeds %d",
               R, rot, LAT_MAX_ROW);
    TQ_REQUIRE(window >= 0, "latent_attention: negative window %d", window);
    TQ_REQUIRE(n_splits >= 1 && n_splits <= LAT_MAX_SPLITS && (n_splits == 1 || partial), "latent_attention: %d key ranges "
               "(at most %d, and more than one need a scratch buffer)", n_splits, LAT_MAX_SPLITS);
    TQ_REQUIRE((H + LAT_HG - 1) / LAT_HG <= 65535, "latent_attention: %d heads exceed the grid limit", H);
    TQ_REQUIRE(rot == 0 || (q && q_off >= 0 && q_off + rot <= q_dim), "latent_attention: the queries' rotated part does not fit");
    const bool mma = act_dtype == TQ_BF16 && Dk % 16 == 0 && R % 32 == 0 && R <= 512 && (q_dim % 2 == 0) &&
                     ((uintptr_t)cache % 16) == 0 && ((uintptr_t)out % 4) == 0 && ((uintptr_t)q_lat % 16) == 0 &&
                     ((uintptr_t)q % 16) == 0 && (!partial || ((uintptr_t)partial % 8) == 0) && lat_use_mma();
    if (mma) {
        dim3 grid(T_, (H + LATM_HEADS - 1) / LATM_HEADS, n_splits);
        TQ_REQUIRE(grid.y <= 65535, "latent_attention: %d heads exceed the grid limit", H);
        const size_t smem = (size_t)(LATM_HEADS + 2 * LATM_KEYS) * (Dk + LATM_PAD) * sizeof(__nv_bfloat16) +
                            (size_t)2 * LATM_HEADS * LATM_PS * sizeof(float);
#define LATM_LAUNCH(OT_, NW_)                                                                                         \
        do {                                                                                                       \
            auto kern = latent_attention_mma_kernel<OT_, NW_>;                                                         \
            static size_t allowed = 48 * 1024;                                                                     \
            if (smem > allowed) {                                                                                  \
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                if (e != cudaSuccess) TQ_FAIL(-1, "latent_attention: %d bytes of shared memory refused: %s", (int)smem, cudaGetErrorString(e)); \
                allowed = smem;                                                                                    \
            }                                                                                                      \
            tq_launch(grid, NW_ * 32, smem, stream)(kern, (const __nv_bfloat16*)q_lat,                             \
                (const __nv_bfloat16*)q, q_dim, q_off, (const __nv_bfloat16*)cache, sink, positions, seq_of_token, page_table, \
                table_stride, page_size, window, scale, (__nv_bfloat16*)out, partial, H, R, rot, n_seqs, n_pages); \
        } while (0)
        if (R % 64 == 0) {                 // eight warps, R / 64 n-tiles each
            switch (R / 64) {
                case 1: LATM_LAUNCH(1, 8); break;
                case 2: LATM_LAUNCH(2, 8); break;
                case 3: LATM_LAUNCH(3, 8); break;
                case 4: LATM_LAUNCH(4, 8); break;
                case 5: LATM_LAUNCH(5, 8); break;
                case 6: LATM_LAUNCH(6, 8); break;
                case 7: LATM_LAUNCH(7, 8); break;
                default: LATM_LAUNCH(8, 8); break;
            }
        } else {                           // four warps, an odd number of n-tiles each
            switch (R / 32) {
                case 1: LATM_LAUNCH(1, 4); break;
                case 3: LATM_LAUNCH(3, 4); break;
                case 5: LATM_LAUNCH(5, 4); break;
                case 7: LATM_LAUNCH(7, 4); break;
                case 9: LATM_LAUNCH(9, 4); break;
                case 11: LATM_LAUNCH(11, 4); break;
                case 13: LATM_LAUNCH(13, 4); break;
                default: LATM_LAUNCH(15, 4); break;
            }
        }
    } else {
    dim3 grid(T_, (H + LAT_HG - 1) / LAT_HG, n_splits);
    const size_t smem = (size_t)(LAT_HG * Dk + LAT_WARPS * R) * sizeof(float);
    const bool vec = Dk % 4 == 0 && R % 4 == 0 && ((uintptr_t)cache % 16) == 0;
    TQ_DISPATCH(act_dtype, TA, {
        if (!vec) LAT_LAUNCH(TA, 32, 1);
        else if (Dk <= 128) LAT_LAUNCH(TA, 4, 4);
        else if (Dk <= 256) LAT_LAUNCH(TA, 8, 4);
        else if (Dk <= 640) LAT_LAUNCH(TA, 20, 4);
        else LAT_LAUNCH(TA, 32, 4);
    });
    }
    TQ_CHECK_LAUNCH("latent_attention");
    if (n_splits > 1) {
        dim3 mgrid(T_, H, (R + LAT_MERGE_THREADS - 1) / LAT_MERGE_THREADS);
        TQ_REQUIRE(H <= 65535, "latent_attention: %d heads exceed the grid limit", H);
        TQ_DISPATCH(act_dtype, TA,
            (tq_launch(mgrid, LAT_MERGE_THREADS, 0, stream)(latent_merge_kernel<TA>, (const float*)partial, sink, n_splits, H, R, (TA*)out)));
        TQ_CHECK_LAUNCH("latent_merge");
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// Prompt path.  out[j] = the row of position k0 + j of one sequence, j < n (16-byte copies when rows allow it).
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void latent_gather_kernel(const TA* __restrict__ cache, const int* __restrict__ table, int table_stride,
                                     int page_size, int k0, int n, int Dk, TA* __restrict__ out, int vec, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int j = blockIdx.x * warps + (threadIdx.x >> 5); j < n; j += gridDim.x * warps) {
        const int p = k0 + j;
        const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const TA* src = cache + ((size_t)page * page_size + p % page_size) * Dk;
        TA* dst = out + (size_t)j * Dk;
        if (vec) {
            const int n16 = (int)((size_t)Dk * sizeof(TA) / 16);
            for (int i = lane; i < n16; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        } else {
            for (int i = lane; i < Dk; i += 32) dst[i] = src[i];
        }
    }
}

TQ_EXPORT int tq_latent_gather(const void* cache, int act_dtype, const int* table, int table_stride, int page_size, int k0,
                               int n, int Dk, void* out, int n_pages, cudaStream_t stream) {
    if (n == 0) return 0;
    TQ_REQUIRE(n > 0 && k0 >= 0 && Dk >= 1, "latent_gather: bad range %d + %d", k0, n);
    const int esize = act_dtype == TQ_F32 ? 4 : 2;
    const int vec = ((size_t)Dk * esize) % 16 == 0 && ((uintptr_t)cache % 16) == 0 && ((uintptr_t)out % 16) == 0;
    int blocks = (n + 7) / 8;
    if (blocks > 148 * 8) blocks = 148 * 8;
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch(blocks, 256, 0, stream)(latent_gather_kernel<TA>, (const TA*)cache, table, table_stride, page_size, k0, n,
                                           Dk, (TA*)out, vec, n_pages)));
    TQ_CHECK_LAUNCH("latent_gather");
    return 0;
}

// ---------------------------------------------------------------------------------------
// scores [rows, n_keys] fp32 (row r: token r / H of the run, head r % H; column j: position k0 + j) -> weights in
// the activation dtype: w_j = exp(s_j * scale - M) / (sum_visible exp(s * scale - M) + exp(sink_h - M)), 0 where
// the token at position pos0 + r / H does not see position k0 + j (later, or window positions or more back).
// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void latent_softmax_kernel(const float* __restrict__ scores, const float* __restrict__ sink, float scale,
                                      int window, int pos0, int k0, int n_keys, int H, TO* __restrict__ weights) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const size_t r = blockIdx.x;
    const int h = (int)(r % H), pos = pos0 + (int)(r / H);
    const int lo = max(window > 0 ? pos + 1 - window : 0, k0) - k0, hi = min(pos + 1 - k0, n_keys);     // visible columns
    const float* s = scores + r * n_keys;
    TO* w = weights + r * n_keys;
    const float sk = sink ? sink[h] : -INFINITY;
    float m = sk;
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) m = fmaxf(m, s[j] * scale);
    m = tq_block_max(m, scratch);
    float l = 0.f;
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) l += expf(s[j] * scale - m);
    l = tq_block_sum(l, scratch);
    if (sink) l += expf(sk - m);
    const float inv = 1.0f / l;
    for (int j = threadIdx.x; j < n_keys; j += blockDim.x)
        w[j] = tq_from_float<TO>(j >= lo && j < hi ? expf(s[j] * scale - m) * inv : 0.f);
}

TQ_EXPORT int tq_latent_softmax(const float* scores, const float* sink, float scale, int window, int pos0, int k0,
                                int n_keys, int H, void* weights, int out_dtype, long long rows, cudaStream_t stream) {
    if (rows == 0) return 0;
    TQ_REQUIRE(rows > 0 && rows <= 0x7fffffffLL && n_keys >= 1 && H >= 1 && window >= 0 && k0 >= 0 && pos0 >= k0,
               "latent_softmax: bad sizes");
    const int threads = n_keys >= 1024 ? 256 : 128;
    TQ_DISPATCH(out_dtype, TO,
        (tq_launch((int)rows, threads, 0, stream)(latent_softmax_kernel<TO>, scores, sink, scale, window, pos0, k0, n_keys, H,
                                                  (TO*)weights)));
    TQ_CHECK_LAUNCH("latent_softmax");
    return 0;
}

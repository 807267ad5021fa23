// Page scorer: score[s, hq, l] = sum_d max(q*min, q*max) over per-page key
// min/max summaries.  HBM-bound streaming kernel: the summaries of a KV head are
// read once with 128-bit loads and reused for all `rep` query heads of the group.
//
// Mapping (fast path): a page's summary is two rows of D elements.  Sixteen lanes
// cover one page (each lane owns VEC = D/16 consecutive channels of the min row
// and the same channels of the max row), so a warp streams two pages per step
// and a 16-lane shuffle tree finishes the channel sum.
//
// max(q*a, q*b) equals max(q,0)*max(a,b) + min(q,0)*min(a,b): one of the two
// terms is an exact zero, so after ordering the pair once per channel, two FMAs
// per (channel, query head) reproduce the formula for all `rep` heads.  (Real
// summaries already have a <= b; the reference's own tests feed unordered rows.)

#include "da_common.cuh"

namespace da {

constexpr int kScoreThreads = 256;
constexpr int kScoreWarps = kScoreThreads / 32;
constexpr int kScoreUnroll = 4;

template <typename T, int VEC, int REP>
__global__ void __launch_bounds__(kScoreThreads, 2)
score_pages_kernel(const T *__restrict__ q, const T *__restrict__ summaries, float *__restrict__ scores,
                   int n_kv_heads, int n_pages) {
    if (threadIdx.x == 0) trace_stamp(0, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, 0);
    griddep_launch_dependents();   // the selection kernel may move onto free SMs and wait there
    constexpr int D = 16 * VEC;
    constexpr int kWords = VEC * (int)sizeof(T) / 4;
    const int hk = blockIdx.y;
    const int tok = blockIdx.z;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int sub = lane & 15;   // channel block inside the page
    const int half = lane >> 4;  // which page of the pair

    float qpos[REP][VEC], qneg[REP][VEC];
    {
        const T *qrow = q + ((size_t)(tok * n_kv_heads + hk) * REP) * D + sub * VEC;
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            uint32_t w[kWords];
            float f[VEC];
            load_words<kWords>(qrow + (size_t)r * D, w);
            Unpack<T, VEC>::run(w, f);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                qpos[r][i] = fmaxf(f[i], 0.f);
                qneg[r][i] = fminf(f[i], 0.f);
            }
        }
    }

    const T *base = summaries + (size_t)hk * n_pages * 2 * D + sub * VEC;
    float *out = scores + ((size_t)(tok * n_kv_heads + hk) * REP) * n_pages;
    const int n_pairs = (n_pages + 1) >> 1;
    const int stride = gridDim.x * kScoreWarps;

    for (int pair0 = blockIdx.x * kScoreWarps + warp; pair0 < n_pairs; pair0 += stride * kScoreUnroll) {
        uint32_t wmn[kScoreUnroll][kWords], wmx[kScoreUnroll][kWords];
        int page[kScoreUnroll];
#pragma unroll
        for (int u = 0; u < kScoreUnroll; ++u) {
            const int pr = pair0 + u * stride;
            page[u] = (pr < n_pairs) ? pr * 2 + half : n_pages;  // n_pages = nothing to do
            const int pg = page[u] < n_pages ? page[u] : n_pages - 1;
            const T *row = base + (size_t)pg * 2 * D;
            load_words<kWords>(row, wmn[u]);
            load_words<kWords>(row + D, wmx[u]);
        }
#pragma unroll
        for (int u = 0; u < kScoreUnroll; ++u) {
            float mn[VEC], mx[VEC], acc[REP];
            Unpack<T, VEC>::run(wmn[u], mn);
            Unpack<T, VEC>::run(wmx[u], mx);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                const float lo = fminf(mn[i], mx[i]);
                mx[i] = fmaxf(mn[i], mx[i]);
                mn[i] = lo;
            }
#pragma unroll
            for (int r = 0; r < REP; ++r) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < VEC; ++i) a = fmaf(qpos[r][i], mx[i], fmaf(qneg[r][i], mn[i], a));
                acc[r] = a;
            }
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1)
#pragma unroll
                for (int r = 0; r < REP; ++r) acc[r] += __shfl_xor_sync(DA_FULL_MASK, acc[r], off);
            if (sub == 0 && page[u] < n_pages) {
#pragma unroll
                for (int r = 0; r < REP; ++r) out[(size_t)r * n_pages + page[u]] = acc[r];
            }
        }
    }
}

// Any head_dim, any rep: one warp per page, lanes stride over channels.
template <typename T>
__global__ void __launch_bounds__(kScoreThreads)
score_pages_generic_kernel(const T *__restrict__ q, const T *__restrict__ summaries,
                           float *__restrict__ scores, int n_kv_heads, int rep, int n_pages, int head_dim) {
    if (threadIdx.x == 0) trace_stamp(0, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, 0);
    griddep_launch_dependents();   // the selection kernel may move onto free SMs and wait there
    const int hk = blockIdx.y;
    const int tok = blockIdx.z;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const T *base = summaries + (size_t)hk * n_pages * 2 * head_dim;
    for (int page = blockIdx.x * kScoreWarps + warp; page < n_pages; page += gridDim.x * kScoreWarps) {
        const T *mn = base + (size_t)page * 2 * head_dim;
        const T *mx = mn + head_dim;
        for (int r = 0; r < rep; ++r) {
            const size_t row = (size_t)(tok * n_kv_heads + hk) * rep + r;
            const T *qrow = q + row * head_dim;
            float a = 0.f;
            for (int d = lane; d < head_dim; d += 32) {
                const float qv = to_float(qrow[d]);
                const float lo = to_float(mn[d]), hi = to_float(mx[d]);
                a += fmaxf(qv * lo, qv * hi);
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) a += __shfl_xor_sync(DA_FULL_MASK, a, off);
            if (lane == 0) scores[row * n_pages + page] = a;
        }
    }
}

// ---- 16-bit summaries known to be ordered (min <= max): tensor-core path ---------------
//
// With min <= max the score is one dot product of length 2D per (query head, page):
//   score = [min(q,0) | max(q,0)] . [min row | max row]
// and the right-hand vector is exactly the page's summary as it lies in memory.  So
// the scores of a KV head are a (rep x 2D) by (2D x pages) product with the pages as
// the N dimension: mma.sync m16n8k16 with the query rows in the first `rep` rows of A
// and 8 pages per n-tile.  B fragments come straight from global memory with 128-bit
// loads: lane (page n, quad position c) reads the 16-byte chunks c, c+4, c+8, ... of
// its page; the A operand is loaded with the same chunk permutation, so the k order
// inside a step never has to match memory order.  About 20 instructions per 8 pages
// instead of ~500 on CUDA cores, which leaves the kernel bound by HBM.
template <typename T> struct ScoreMma;
template <> struct ScoreMma<__nv_bfloat16> {
    __device__ __forceinline__ static void mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};
template <> struct ScoreMma<__half> {
    __device__ __forceinline__ static void mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};

constexpr int kScoreMmaCtasPerHeadTarget = 296;  // two CTAs per SM in total

template <typename T, int D, int REP>
__global__ void __launch_bounds__(kScoreThreads, 2)
score_pages_mma_kernel(const T *__restrict__ q, const T *__restrict__ summaries, float *__restrict__ scores,
                       int n_kv_heads, int n_pages) {
    if (threadIdx.x == 0) trace_stamp(0, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, 0);
    griddep_launch_dependents();   // the selection kernel may move onto free SMs and wait there
    static_assert(sizeof(T) == 2 && REP <= 8 && (2 * D) % 32 == 0, "16-bit types, at most 8 query rows");
    constexpr int CHUNKS = 2 * D / 8;   // 16-byte chunks per page summary
    constexpr int NI = CHUNKS / 4;      // chunks per lane = pairs of k-steps
    const int hk = blockIdx.y;
    const int tok = blockIdx.z;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int row = lane >> 2;   // query row (A, C) and page inside the n-tile (B)
    const int qd = lane & 3;

    const uint4 *base = reinterpret_cast<const uint4 *>(summaries + (size_t)hk * n_pages * 2 * D);
    float *out = scores + ((size_t)(tok * n_kv_heads + hk) * REP) * n_pages;
    const int n_tiles = (n_pages + 7) >> 3;
    const int workers = gridDim.x * kScoreWarps;
    // warp-major worker ids: the warps that get one tile more are spread over all CTAs
    const int worker = warp * gridDim.x + blockIdx.x;

    // two page tiles in flight per warp; the first two set out before anything waits for the query
    uint4 b[2][NI];
    int page0[2];
    auto load_tiles = [&](int t0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int tile = t0 + u * workers;
            page0[u] = tile < n_tiles ? tile * 8 : -1;
            int pg = (page0[u] < 0 ? 0 : page0[u]) + row;
            if (pg >= n_pages) pg = n_pages - 1;
            const uint4 *src = base + (size_t)pg * CHUNKS + qd;
#pragma unroll
            for (int i = 0; i < NI; ++i) b[u][i] = __ldcs(src + 4 * i);
        }
    };
    if (worker < n_tiles) load_tiles(worker);

    // A fragments: [min(q,0) | max(q,0)] of query row `row`, chunk permutation as for B
    uint32_t a0[2 * NI], a2[2 * NI];
    {
        const T *qrow = q + ((size_t)(tok * n_kv_heads + hk) * REP + (row < REP ? row : 0)) * D;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int c = qd + 4 * i;            // chunk of the concatenated vector
            const bool pos_half = 8 * c >= D;    // second half: max(q, 0)
            const int e0 = 8 * c - (pos_half ? D : 0);
            uint32_t w[4];
            float f[8];
            load_words<4>(qrow + e0, w);
            Unpack<T, 8>::run(w, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = (row < REP) ? (pos_half ? fmaxf(f[j], 0.f) : fminf(f[j], 0.f)) : 0.f;
            a0[2 * i] = ScoreMma<T>::pack(f[0], f[1]);
            a2[2 * i] = ScoreMma<T>::pack(f[2], f[3]);
            a0[2 * i + 1] = ScoreMma<T>::pack(f[4], f[5]);
            a2[2 * i + 1] = ScoreMma<T>::pack(f[6], f[7]);
        }
    }

    for (int t0 = worker; t0 < n_tiles;) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (page0[u] < 0) continue;  // warp-uniform
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                ScoreMma<T>::mma(c, a0[2 * i], a2[2 * i], b[u][i].x, b[u][i].y);
                ScoreMma<T>::mma(c, a0[2 * i + 1], a2[2 * i + 1], b[u][i].z, b[u][i].w);
            }
            if (row < REP) {
                const int pg = page0[u] + 2 * qd;
                if (pg < n_pages) out[(size_t)row * n_pages + pg] = c[0];
                if (pg + 1 < n_pages) out[(size_t)row * n_pages + pg + 1] = c[1];
            }
        }
        t0 += 2 * workers;
        if (t0 < n_tiles) load_tiles(t0);
    }
    if (g_trace_buf != nullptr) {
        __syncthreads();
        if (threadIdx.x == 0) trace_stamp(0, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, 1);
    }
}

template <typename T, int D>
static cudaError_t launch_mma(const void *q, const void *summaries, float *scores, int n_tokens, int n_kv_heads,
                              int rep, int n_pages, cudaStream_t stream) {
    int per_row = kScoreMmaCtasPerHeadTarget / (n_kv_heads * n_tokens);
    if (per_row < 1) per_row = 1;
    const int n_tiles = (n_pages + 7) / 8;
    int gx = (n_tiles + kScoreWarps - 1) / kScoreWarps;
    if (gx > per_row) gx = per_row;
    dim3 grid(gx, n_kv_heads, n_tokens);
    const T *qq = static_cast<const T *>(q);
    const T *ss = static_cast<const T *>(summaries);
    switch (rep) {
    case 1: score_pages_mma_kernel<T, D, 1><<<grid, kScoreThreads, 0, stream>>>(qq, ss, scores, n_kv_heads, n_pages); break;
    case 2: score_pages_mma_kernel<T, D, 2><<<grid, kScoreThreads, 0, stream>>>(qq, ss, scores, n_kv_heads, n_pages); break;
    case 4: score_pages_mma_kernel<T, D, 4><<<grid, kScoreThreads, 0, stream>>>(qq, ss, scores, n_kv_heads, n_pages); break;
    case 8: score_pages_mma_kernel<T, D, 8><<<grid, kScoreThreads, 0, stream>>>(qq, ss, scores, n_kv_heads, n_pages); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

template <typename T, int VEC>
static cudaError_t launch_fast(const void *q, const void *summaries, float *scores, int n_tokens,
                               int n_kv_heads, int rep, int n_pages, cudaStream_t stream) {
    const int n_pairs = (n_pages + 1) / 2;
    // two resident CTAs per SM; spread them over the heads and tokens of the launch
    int per_row = (148 * 2) / (n_kv_heads * n_tokens);
    if (per_row < 1) per_row = 1;
    int gx = (n_pairs + kScoreWarps * kScoreUnroll - 1) / (kScoreWarps * kScoreUnroll);
    if (gx > per_row) gx = per_row;
    if (gx < 1) gx = 1;
    dim3 grid(gx, n_kv_heads, n_tokens);
    const T *qq = static_cast<const T *>(q);
    const T *ss = static_cast<const T *>(summaries);
    switch (rep) {
    case 1: score_pages_kernel<T, VEC, 1><<<grid, kScoreThreads, 0, stream>>>(qq, ss, scores, n_kv_heads, n_pages); break;
    case 2: score_pages_kernel<T, VEC, 2><<<grid, kScoreThreads, 0, stream>>>(qq, ss, scores, n_kv_heads, n_pages); break;
    case 4: score_pages_kernel<T, VEC, 4><<<grid, kScoreThreads, 0, stream>>>(qq, ss, scores, n_kv_heads, n_pages); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_generic(const void *q, const void *summaries, float *scores, int n_tokens,
                                  int n_kv_heads, int rep, int n_pages, int head_dim, cudaStream_t stream) {
    int gx = (n_pages + kScoreWarps - 1) / kScoreWarps;
    if (gx > 592) gx = 592;
    dim3 grid(gx, n_kv_heads, n_tokens);
    score_pages_generic_kernel<T><<<grid, kScoreThreads, 0, stream>>>(
        static_cast<const T *>(q), static_cast<const T *>(summaries), scores, n_kv_heads, rep, n_pages, head_dim);
    return cudaGetLastError();
}

template <typename T>
static cudaError_t dispatch(const void *q, const void *summaries, float *scores, int n_tokens, int n_kv_heads,
                            int rep, int n_pages, int head_dim, bool ordered, cudaStream_t stream) {
    const bool aligned = (((uintptr_t)q | (uintptr_t)summaries) & 15) == 0;
    if constexpr (sizeof(T) == 2) {
        if (ordered && aligned && (rep == 1 || rep == 2 || rep == 4 || rep == 8)) {
            if (head_dim == 128) return launch_mma<T, 128>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, stream);
            if (head_dim == 64) return launch_mma<T, 64>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, stream);
        }
    }
    const bool rep_ok = rep == 1 || rep == 2 || rep == 4;
    if (aligned && rep_ok) {
        if (head_dim == 128) return launch_fast<T, 8>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, stream);
        if (head_dim == 64) return launch_fast<T, 4>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, stream);
    }
    return launch_generic<T>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, head_dim, stream);
}

}  // namespace da

extern "C" int da_score_pages(const void *q, const void *summaries, float *scores, int n_tokens,
                              int n_kv_heads, int rep, int n_pages, int head_dim, int dtype,
                              int summaries_ordered, da_stream_t stream) {
    if (!q || !summaries || !scores) return DA_ERR_NULL;
    if (n_tokens < 1 || n_kv_heads < 1 || rep < 1 || n_pages < 1 || head_dim < 1) return DA_ERR_SHAPE;
    if (n_kv_heads > 65535 || n_tokens > 65535) return DA_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    switch (dtype) {
    case DA_F32: e = da::dispatch<float>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, head_dim, summaries_ordered != 0, s); break;
    case DA_F16: e = da::dispatch<__half>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, head_dim, summaries_ordered != 0, s); break;
    case DA_BF16: e = da::dispatch<__nv_bfloat16>(q, summaries, scores, n_tokens, n_kv_heads, rep, n_pages, head_dim, summaries_ordered != 0, s); break;
    default: return DA_ERR_DTYPE;
    }
    return (int)e;
}

DA_DEFINE_TRACE_SETTER(trace_set_score)

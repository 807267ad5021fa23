// Pieces shared by the two decode-attention kernels (float32 on CUDA cores,
// 16-bit types on tensor cores): launch geometry, the parameter block, and the
// final merge of the per-CTA partials.
#pragma once

#include "da_common.cuh"

namespace da {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kUnitTokens = 16;
constexpr int kCounterBytes = 1024;
constexpr int kAttnTargetCtas = 296;  // 2 per SM on 148 SMs
constexpr int kAttnMaxSplits = 148;

__host__ __device__ inline int attn_splits(int n_kv_heads) {
    int s = kAttnTargetCtas / n_kv_heads;
    if (s > kAttnMaxSplits) s = kAttnMaxSplits;
    if (s < 1) s = 1;
    return s;
}

struct AttnParams {
    const unsigned char *q;
    const unsigned char *prefix;
    long long prefix_head_stride;  // elements
    int n_prefix_tokens;
    unsigned char *local_k, *local_v;
    long long local_tok_stride, local_head_stride;  // elements
    int local_capacity;
    const unsigned char *new_k, *new_v;
    const int32_t *start_pos_dev;
    int start_pos_host;
    int dram_tokens;
    unsigned char *out;
    float *lse_out;
    float *partials;
    unsigned int *counters;
    int32_t *status;
    float scale_log2;
};

// Final merge of the per-CTA partials of one head by one CTA of kAttnThreads threads.
// partial row = acc[D] (already weighted to the row's max), max, l.  `scratch` holds
// at least splits * REP floats of shared memory.  Loads bypass L1 (the rows were
// written by other SMs) and are issued in batches so that only a few L2 round trips
// are exposed.
template <typename T, int D, int REP>
__device__ __forceinline__ void merge_splits(const AttnParams &p, int h, int splits, float *scratch) {
    constexpr int PW = D + 2;
    constexpr float NEG_INF = -INFINITY;
    __shared__ float sh_m[REP], sh_l[REP];
    const int tid = threadIdx.x;
    const float *hp = p.partials + ((size_t)h * splits * REP) * PW;
    const int n = splits * REP;
    for (int e = tid; e < n; e += kAttnThreads) scratch[e] = __ldcg(hp + (size_t)e * PW + D);
    if (tid < REP) sh_l[tid] = 0.f;
    __syncthreads();
    if (tid < REP) {
        float mn = NEG_INF;
        for (int s = 0; s < splits; ++s) mn = fmaxf(mn, scratch[s * REP + tid]);
        sh_m[tid] = (mn == NEG_INF) ? 0.f : mn;
    }
    __syncthreads();
    for (int e = tid; e < n; e += kAttnThreads) {
        const float w = fast_exp2(scratch[e] - sh_m[e % REP]);
        scratch[e] = w;
        atomicAdd(&sh_l[e % REP], w * __ldcg(hp + (size_t)e * PW + D + 1));
    }
    __syncthreads();
    for (int e = tid; e < REP * D; e += kAttnThreads) {
        const int r = e / D;
        const int c = e % D;
        const float *col = hp + (size_t)r * PW + c;
        float a = 0.f;
        int s = 0;
        for (; s + 8 <= splits; s += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(col + (size_t)(s + u) * REP * PW);
#pragma unroll
            for (int u = 0; u < 8; ++u) a = fmaf(v[u], scratch[(s + u) * REP + r], a);
        }
        for (; s < splits; ++s) a = fmaf(__ldcg(col + (size_t)s * REP * PW), scratch[s * REP + r], a);
        const float ll = sh_l[r];
        reinterpret_cast<T *>(p.out)[(size_t)(h * REP + r) * D + c] = from_float<T>(ll > 0.f ? a / ll : 0.f);
        if (c == 0 && p.lse_out) p.lse_out[h * REP + r] = (sh_m[r] + log2f(ll)) * 0.6931471805599453f;
    }
}

// 16-bit element types: tensor-core kernel (attn_mma.cu).
cudaError_t launch_attention_mma(const AttnParams &p, int n_kv_heads, int rep, int head_dim, int dtype,
                                 cudaStream_t stream);

}  // namespace da

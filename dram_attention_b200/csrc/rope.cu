// Rotary position embedding of the new queries and keys, the step of the caller that
// feeds the page scorer (evaluation/dram-attention/model.py:125-135 and :201 of the reference:
// apply_rotary_emb on xq, xk right before the operator call).  Channels are taken in
// adjacent pairs (x[2i], x[2i+1]) as one complex number and multiplied by
// freqs_cis[token][i] = cos + i sin; the arithmetic is fp32, the result is rounded to the
// input type.  One launch covers q and k of all tokens of the call and is chained to the
// scorer by a programmatic dependent launch, so the caller's half-dozen elementwise
// launches become one short kernel in front of the step.

#include "da_common.cuh"

namespace da {

constexpr int kRopeThreads = 256;

template <typename T> struct Pair;
template <> struct Pair<float> {
    using type = float2;
    static __device__ __forceinline__ float2 load(const float *p) { return *reinterpret_cast<const float2 *>(p); }
    static __device__ __forceinline__ void store(float *p, float a, float b) { *reinterpret_cast<float2 *>(p) = make_float2(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16 *p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, float a, float b) {
        __nv_bfloat162 v;
        v.x = __float2bfloat16_rn(a);
        v.y = __float2bfloat16_rn(b);
        *reinterpret_cast<__nv_bfloat162 *>(p) = v;
    }
};
template <> struct Pair<__half> {
    static __device__ __forceinline__ float2 load(const __half *p) {
        return __half22float2(*reinterpret_cast<const __half2 *>(p));
    }
    static __device__ __forceinline__ void store(__half *p, float a, float b) {
        __half2 v;
        v.x = __float2half_rn(a);
        v.y = __float2half_rn(b);
        *reinterpret_cast<__half2 *>(p) = v;
    }
};

// q (n_tokens, n_q_heads, D), k (n_tokens, n_kv_heads, D), contiguous; freqs (n_tokens, D / 2) of
// (cos, sin).  Pair index space: token-major, then the q heads, then the k heads.
template <typename T>
__global__ void __launch_bounds__(kRopeThreads)
rope_qk_kernel(const T *__restrict__ q, const T *__restrict__ k, const float2 *__restrict__ freqs,
               T *__restrict__ q_out, T *__restrict__ k_out, int n_tokens, int n_q_heads, int n_kv_heads,
               int half_dim) {
    griddep_wait();                // the projections that made q and k come from the kernel before this one
    griddep_launch_dependents();   // the scorer may move onto the SMs and wait there
    const int heads = n_q_heads + n_kv_heads;
    const long long total = (long long)n_tokens * heads * half_dim;
    for (long long i = (long long)blockIdx.x * kRopeThreads + threadIdx.x; i < total;
         i += (long long)gridDim.x * kRopeThreads) {
        const int c = (int)(i % half_dim);
        const int h = (int)((i / half_dim) % heads);
        const int t = (int)(i / ((long long)half_dim * heads));
        const float2 f = freqs[(size_t)t * half_dim + c];
        const bool is_q = h < n_q_heads;
        const size_t at = is_q ? ((size_t)t * n_q_heads + h) * half_dim * 2 + 2 * c
                               : ((size_t)t * n_kv_heads + (h - n_q_heads)) * half_dim * 2 + 2 * c;
        const float2 x = Pair<T>::load((is_q ? q : k) + at);
        // (x.x + i x.y) * (f.x + i f.y), each product rounded, then the sum: as a complex64 multiply does it
        const float re = __fsub_rn(__fmul_rn(x.x, f.x), __fmul_rn(x.y, f.y));
        const float im = __fadd_rn(__fmul_rn(x.x, f.y), __fmul_rn(x.y, f.x));
        Pair<T>::store((is_q ? q_out : k_out) + at, re, im);
    }
}

template <typename T>
static cudaError_t launch_rope(const void *q, const void *k, const void *freqs, void *q_out, void *k_out,
                               int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, cudaStream_t stream) {
    const long long total = (long long)n_tokens * (n_q_heads + n_kv_heads) * (head_dim / 2);
    long long blocks = (total + kRopeThreads - 1) / kRopeThreads;
    if (blocks > 148 * 4) blocks = 148 * 4;
    const cudaError_t e = launch_dependent(rope_qk_kernel<T>, dim3((unsigned)blocks), dim3(kRopeThreads), (size_t)0,
                                           stream, static_cast<const T *>(q), static_cast<const T *>(k),
                                           static_cast<const float2 *>(freqs), static_cast<T *>(q_out),
                                           static_cast<T *>(k_out), n_tokens, n_q_heads, n_kv_heads, head_dim / 2);
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

}  // namespace da

extern "C" int da_rope_qk(const void *q, const void *k, const void *freqs_cis, void *q_out, void *k_out,
                          int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int dtype,
                          da_stream_t stream) {
    if (!q || !k || !freqs_cis || !q_out || !k_out) return DA_ERR_NULL;
    if (n_tokens < 1 || n_q_heads < 1 || n_kv_heads < 1 || head_dim < 2 || (head_dim & 1)) return DA_ERR_SHAPE;
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(freqs_cis) | reinterpret_cast<uintptr_t>(q_out) |
                          reinterpret_cast<uintptr_t>(k_out);
    if (all & 7) return DA_ERR_ALIGN;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    switch (dtype) {
    case DA_F32: e = da::launch_rope<float>(q, k, freqs_cis, q_out, k_out, n_tokens, n_q_heads, n_kv_heads, head_dim, s); break;
    case DA_BF16: e = da::launch_rope<__nv_bfloat16>(q, k, freqs_cis, q_out, k_out, n_tokens, n_q_heads, n_kv_heads, head_dim, s); break;
    case DA_F16: e = da::launch_rope<__half>(q, k, freqs_cis, q_out, k_out, n_tokens, n_q_heads, n_kv_heads, head_dim, s); break;
    default: return DA_ERR_UNSUPPORTED;
    }
    return (int)e;
}

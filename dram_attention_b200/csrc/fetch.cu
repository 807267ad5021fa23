// Miss-page fetch (gather-copy DRAM -> HBM slots, driven by the device-side miss
// list) and the cache construction pass (pagination, page summaries, warm start).

#include "da_common.cuh"

namespace da {

constexpr int kFetchThreads = 256;
constexpr int kFetchCtasPerHead = 64;

// One CTA per page in flight; each thread moves 16 bytes per load.  The source
// may be pinned host memory mapped into the device address space: many CTAs with
// several independent 128-bit loads each keep the host link busy.
__global__ void __launch_bounds__(kFetchThreads)
fetch_pages_kernel(const uint4 *__restrict__ dram, uint4 *__restrict__ slots,
                   const int32_t *__restrict__ miss_pages, const int32_t *__restrict__ miss_slots,
                   const int32_t *__restrict__ n_miss, int list_len, int n_dram_pages, int n_slots,
                   int page_vecs) {
    const int h = blockIdx.y;
    const int n = min(n_miss[h], list_len);
    for (int j = blockIdx.x; j < n; j += gridDim.x) {
        const int p = miss_pages[(size_t)h * list_len + j];
        const int v = miss_slots[(size_t)h * list_len + j];
        if (p < 0 || p >= n_dram_pages || v < 0 || v >= n_slots) continue;
        const uint4 *src = dram + ((size_t)h * n_dram_pages + p) * page_vecs;
        uint4 *dst = slots + ((size_t)h * n_slots + v) * page_vecs;
        for (int i0 = threadIdx.x; i0 < page_vecs; i0 += kFetchThreads * 4) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * kFetchThreads;
                if (i < page_vecs) r[u] = __ldcs(src + i);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * kFetchThreads;
                if (i < page_vecs) dst[i] = r[u];
            }
        }
    }
}

__global__ void __launch_bounds__(kFetchThreads)
fetch_pages_bytes_kernel(const unsigned char *__restrict__ dram, unsigned char *__restrict__ slots,
                         const int32_t *__restrict__ miss_pages, const int32_t *__restrict__ miss_slots,
                         const int32_t *__restrict__ n_miss, int list_len, int n_dram_pages, int n_slots,
                         size_t page_bytes) {
    const int h = blockIdx.y;
    const int n = min(n_miss[h], list_len);
    for (int j = blockIdx.x; j < n; j += gridDim.x) {
        const int p = miss_pages[(size_t)h * list_len + j];
        const int v = miss_slots[(size_t)h * list_len + j];
        if (p < 0 || p >= n_dram_pages || v < 0 || v >= n_slots) continue;
        const unsigned char *src = dram + ((size_t)h * n_dram_pages + p) * page_bytes;
        unsigned char *dst = slots + ((size_t)h * n_slots + v) * page_bytes;
        for (size_t i = threadIdx.x; i < page_bytes; i += kFetchThreads) dst[i] = src[i];
    }
}

// Cache construction: CTA (page, head), thread = channel.  Reads K and V rows of
// the page's tokens, writes the page payload (token-major, key then value), the
// per-channel min/max summary, and the slot copy for the pages that start out
// resident.
template <typename T>
__global__ void build_pages_kernel(const T *__restrict__ k, const T *__restrict__ v, long long tok_stride,
                                   long long head_stride, T *__restrict__ dram, T *__restrict__ summaries,
                                   T *__restrict__ slots, int n_pages, int n_slots, int page_size,
                                   int head_dim) {
    const int page = blockIdx.x;
    const int h = blockIdx.y;
    const int first_resident = n_pages - n_slots;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float mn = 0.f, mx = 0.f;
        T tmn = T(), tmx = T();
        for (int t = 0; t < page_size; ++t) {
            const size_t src = (size_t)(page * (long long)page_size + t) * tok_stride + (size_t)h * head_stride + d;
            const T kv = k[src];
            const T vv = v[src];
            const float kf = to_float(kv);
            if (t == 0 || kf < mn) { mn = kf; tmn = kv; }
            if (t == 0 || kf > mx) { mx = kf; tmx = kv; }
            const size_t off = ((size_t)t * 2) * head_dim + d;
            if (dram) {
                T *pg = dram + ((size_t)h * n_pages + page) * page_size * 2 * head_dim;
                pg[off] = kv;
                pg[off + head_dim] = vv;
            }
            if (slots && page >= first_resident) {
                T *sl = slots + ((size_t)h * n_slots + (page - first_resident)) * page_size * 2 * head_dim;
                sl[off] = kv;
                sl[off + head_dim] = vv;
            }
        }
        if (summaries) {
            T *sm = summaries + ((size_t)h * n_pages + page) * 2 * head_dim;
            sm[d] = tmn;
            sm[head_dim + d] = tmx;
        }
    }
}

template <typename T>
static cudaError_t launch_build(const void *k, const void *v, long long tok_stride, long long head_stride,
                                void *dram, void *summaries, void *slots, int n_kv_heads, int n_pages,
                                int n_slots, int page_size, int head_dim, cudaStream_t stream) {
    int threads = head_dim < 32 ? 32 : (head_dim > 256 ? 256 : (head_dim + 31) / 32 * 32);
    dim3 grid(n_pages, n_kv_heads);
    build_pages_kernel<T><<<grid, threads, 0, stream>>>(
        static_cast<const T *>(k), static_cast<const T *>(v), tok_stride, head_stride, static_cast<T *>(dram),
        static_cast<T *>(summaries), static_cast<T *>(slots), n_pages, n_slots, page_size, head_dim);
    return cudaGetLastError();
}

}  // namespace da

extern "C" int da_fetch_pages(const void *dram_pages, void *slots, const int32_t *miss_pages,
                              const int32_t *miss_slots, const int32_t *n_miss, int list_len, int n_kv_heads,
                              int n_dram_pages, int n_slots, size_t page_bytes, da_stream_t stream) {
    if (!dram_pages || !slots || !miss_pages || !miss_slots || !n_miss) return DA_ERR_NULL;
    if (list_len < 1 || n_kv_heads < 1 || n_dram_pages < 1 || n_slots < 1 || page_bytes < 1) return DA_ERR_SHAPE;
    if (n_kv_heads > 65535) return DA_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int gx = list_len < da::kFetchCtasPerHead ? list_len : da::kFetchCtasPerHead;
    dim3 grid(gx, n_kv_heads);
    const bool vec = (page_bytes % 16 == 0) && ((((uintptr_t)dram_pages | (uintptr_t)slots) & 15) == 0) &&
                     (page_bytes / 16 < (size_t)1 << 30);
    if (vec) {
        da::fetch_pages_kernel<<<grid, da::kFetchThreads, 0, s>>>(
            static_cast<const uint4 *>(dram_pages), static_cast<uint4 *>(slots), miss_pages, miss_slots, n_miss,
            list_len, n_dram_pages, n_slots, (int)(page_bytes / 16));
    } else {
        da::fetch_pages_bytes_kernel<<<grid, da::kFetchThreads, 0, s>>>(
            static_cast<const unsigned char *>(dram_pages), static_cast<unsigned char *>(slots), miss_pages,
            miss_slots, n_miss, list_len, n_dram_pages, n_slots, page_bytes);
    }
    return (int)cudaGetLastError();
}

extern "C" int da_build_pages(const void *k, const void *v, long long kv_token_stride, long long kv_head_stride,
                              void *dram_pages, void *summaries, void *slots, int n_kv_heads, int n_pages,
                              int n_slots, int page_size, int head_dim, int dtype, da_stream_t stream) {
    if (!k || !v) return DA_ERR_NULL;
    if (n_kv_heads < 1 || n_pages < 1 || page_size < 1 || head_dim < 1 || n_slots < 0 || n_slots > n_pages)
        return DA_ERR_SHAPE;
    if (n_kv_heads > 65535) return DA_ERR_UNSUPPORTED;
    if (slots && n_slots < 1) return DA_ERR_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    switch (dtype) {
    case DA_F32: e = da::launch_build<float>(k, v, kv_token_stride, kv_head_stride, dram_pages, summaries, slots, n_kv_heads, n_pages, n_slots, page_size, head_dim, s); break;
    case DA_F16: e = da::launch_build<__half>(k, v, kv_token_stride, kv_head_stride, dram_pages, summaries, slots, n_kv_heads, n_pages, n_slots, page_size, head_dim, s); break;
    case DA_BF16: e = da::launch_build<__nv_bfloat16>(k, v, kv_token_stride, kv_head_stride, dram_pages, summaries, slots, n_kv_heads, n_pages, n_slots, page_size, head_dim, s); break;
    default: return DA_ERR_DTYPE;
    }
    return (int)e;
}

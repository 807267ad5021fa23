// Shared device helpers: element-type conversion, vector loads, warp reductions,
// mbarrier / bulk-copy wrappers (sm_90+ PTX, built here for sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dram_attention_b200.h"

#define DA_FULL_MASK 0xffffffffu

namespace da {

// ---- element types ---------------------------------------------------------

template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> { static constexpr int kCode = DA_F32; };
template <> struct ElemTraits<__half> { static constexpr int kCode = DA_F16; };
template <> struct ElemTraits<__nv_bfloat16> { static constexpr int kCode = DA_BF16; };

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// Unpack one 32-bit word holding two 16-bit elements (low half first).
template <typename T> __device__ __forceinline__ void unpack2(uint32_t w, float &lo, float &hi);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float &lo, float &hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t w, float &lo, float &hi) {
    __half2 h = *reinterpret_cast<__half2 *>(&w);
    float2 f = __half22float2(h);
    lo = f.x;
    hi = f.y;
}

// Convert N consecutive elements, given as raw 32-bit words, to float.
template <typename T, int N> struct Unpack {
    static constexpr int kWords = N * (int)sizeof(T) / 4;
    __device__ __forceinline__ static void run(const uint32_t (&w)[kWords], float (&out)[N]) {
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int i = 0; i < N; ++i) out[i] = __uint_as_float(w[i]);
        } else {
#pragma unroll
            for (int i = 0; i < N / 2; ++i) unpack2<T>(w[i], out[2 * i], out[2 * i + 1]);
        }
    }
};

// Raw load of kWords 32-bit words from a suitably aligned address, widest form.
template <int kWords> __device__ __forceinline__ void load_words(const void *p, uint32_t (&w)[kWords]) {
    if constexpr (kWords % 4 == 0) {
#pragma unroll
        for (int i = 0; i < kWords / 4; ++i) {
            uint4 v = reinterpret_cast<const uint4 *>(p)[i];
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    } else if constexpr (kWords % 2 == 0) {
#pragma unroll
        for (int i = 0; i < kWords / 2; ++i) {
            uint2 v = reinterpret_cast<const uint2 *>(p)[i];
            w[2 * i] = v.x; w[2 * i + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = reinterpret_cast<const uint32_t *>(p)[i];
    }
}

// Pointer forms of the two helpers above, for slices of register arrays.
template <typename T, int N> __device__ __forceinline__ void load_elems(const void *p, float *out) {
    constexpr int kWords = N * (int)sizeof(T) / 4;
    uint32_t w[kWords];
    load_words<kWords>(p, w);
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = __uint_as_float(w[i]);
    } else {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) unpack2<T>(w[i], out[2 * i], out[2 * i + 1]);
    }
}

// ---- optional device-side time stamps (profiling) ----------------------------------
// da_trace_set() hands every kernel file a buffer of kTraceKernels x kTraceCtas x kTraceEvents
// 64-bit words.  While it is set, thread 0 of every CTA writes the global nanosecond timer at a
// few points of the kernel (event 0 = the CTA runs, event 1 = it is done; the attention kernel
// also 2 = its warps are through their units, 3 = its ticket is taken), so that the host can
// read where a step's time goes while the kernels overlap on several streams, which events on a
// stream cannot show.  A launch overwrites the stamps of the launch before it.  Unset (the
// default) a stamp site costs one load of the pointer.
constexpr int kTraceKernels = 6;   // 0 scorer, 1 selection, 2 LRU update, 3 attention (single launch or phase 1), 4 phase 2,
                                   // 5 gather of the head shards (events: 0 on the SM, 2 rows ready, 3 sent, 1 all there and copied)
constexpr int kTraceGather = 5;
constexpr int kTraceCtas = 1024;   // CTA index modulo this
constexpr int kTraceEvents = 4;
static __device__ unsigned long long *g_trace_buf;   // one copy per kernel file, all set together

__device__ __forceinline__ void trace_stamp(int kernel, int cta, int event) {
    unsigned long long *buf = g_trace_buf;
    if (buf != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        buf[((size_t)kernel * kTraceCtas + (cta % kTraceCtas)) * kTraceEvents + event] = t;
    }
}

// Each kernel file defines its setter with this; api.cu calls them all.
#define DA_DEFINE_TRACE_SETTER(name)                                                      \
    namespace da {                                                                        \
    cudaError_t name(void *buffer) {                                                      \
        unsigned long long *b = static_cast<unsigned long long *>(buffer);                \
        return cudaMemcpyToSymbol(g_trace_buf, &b, sizeof(b));                            \
    }                                                                                     \
    }
cudaError_t trace_set_score(void *buffer);
cudaError_t trace_set_topk(void *buffer);
cudaError_t trace_set_lru(void *buffer);
cudaError_t trace_set_attn(void *buffer);
cudaError_t trace_set_attn_mma(void *buffer);
cudaError_t trace_set_gather(void *buffer);

// ---- programmatic dependent launch ---------------------------------------------
// The kernels of a generate step form a chain (scores -> page list -> tables -> attention).  A
// kernel launched with launch_dependent() may be placed on the SMs while its predecessor in the
// stream is still running; it must call griddep_wait() before it touches anything an earlier
// kernel of the stream wrote (the call returns once those kernels have completed and their
// writes are visible).  A predecessor lets its successor in early with
// griddep_launch_dependents().  Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- peer gather words ---------------------------------------------------------------
// The all-gather of the head shards moves 8-byte words {4 bytes of payload, the step's tag}: one naturally
// aligned 8-byte store per word arrives whole, so a word that carries the tag carries its payload.
__device__ __forceinline__ void st_word_sys(uint2 *p, uint32_t payload, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(payload), "r"(tag) : "memory");
}

// ---- small math ------------------------------------------------------------

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- shared-memory barriers and bulk copies ----------------------------------

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after `limit` polls and reports false.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int limit = (1 << 20)) {
    for (int i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Untiled bulk copy global -> shared of this CTA, completion counted in bytes on
// `bar`.  Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                              uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}


// Same, with an L2 eviction-priority hint for the lines it brings in.  Streaming reads that
// nobody will touch again soon should be marked evict-first so that they do not push small,
// latency-critical data (scores, tables) of concurrently running kernels out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void bulk_copy_g2s_hint(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                                   uint64_t *bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_addr(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
        : "memory");
}

}  // namespace da

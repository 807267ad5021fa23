// Version, error text and the profiling switch of the C ABI.

#include "da_common.cuh"

extern "C" int da_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char *da_error_string(int code) {
    switch (code) {
    case DA_OK: return "ok";
    case DA_ERR_NULL: return "a required pointer is null";
    case DA_ERR_SHAPE: return "a size is zero, negative or inconsistent";
    case DA_ERR_DTYPE: return "unknown dtype code";
    case DA_ERR_ALIGN: return "a pointer or stride breaks the required alignment";
    case DA_ERR_UNSUPPORTED: return "shape outside what the kernels are built for";
    case DA_ERR_WORKSPACE: return "workspace too small";
    case DA_ERR_STATIC_SCRATCH: return "shape needs more scratch than the library's built-in buffer holds; use da_decode_attention with a workspace";
    default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error code";
}

extern "C" size_t da_trace_bytes(void) {
    return (size_t)da::kTraceKernels * da::kTraceCtas * da::kTraceEvents * sizeof(unsigned long long);
}

extern "C" int da_trace_set(void *buffer) {
    cudaError_t e;
    if ((e = da::trace_set_score(buffer)) != cudaSuccess) return (int)e;
    if ((e = da::trace_set_topk(buffer)) != cudaSuccess) return (int)e;
    if ((e = da::trace_set_lru(buffer)) != cudaSuccess) return (int)e;
    if ((e = da::trace_set_attn(buffer)) != cudaSuccess) return (int)e;
    if ((e = da::trace_set_attn_mma(buffer)) != cudaSuccess) return (int)e;
    if ((e = da::trace_set_gather(buffer)) != cudaSuccess) return (int)e;
    return 0;
}

// All-gather of the per-KV-head-shard attention outputs over NVLink peer memory, for
// KV-head sharding on the GPUs of one node.  One launch of one CTA per rank per step:
//
//   push   the rank's own rows go into slot (seq & 1) of EVERY rank's gather buffer
//          (plain 128-bit stores to peer pointers), a system-scope fence, then one flag
//          per peer is set to seq + 1;
//   wait   the CTA polls its OWN flags (one per source rank) until all carry seq + 1 -
//          bounded by the GPU's nanosecond timer: after `timeout_us` it sets
//          DA_STATUS_WAIT_TIMEOUT and goes on;
//   copy   the assembled (world, rows) block is copied to the caller's output tensor (the rows
//          of a rank whose flag never came are filled with 0xFF bytes, a NaN in every
//          floating-point format, so that a timed-out gather cannot pass for a result) and the
//          step counter is advanced.
//
// Two slots suffice: a rank can start step s + 2 (which reuses slot s & 1) only after its
// wait of step s + 1 saw every peer's flag of step s + 1, and a peer sets that flag after
// (in stream order) its own copy of step s.  No multimem, no multicast loads: ordinary
// peer stores and local loads.  The payload is a few KiB, so the step is latency-bound:
// one NVLink store round instead of the several a library ring/tree takes.

#include "da_common.cuh"

namespace da {

constexpr int kGatherThreads = 512;
constexpr int kGatherMaxWorld = 16;
constexpr unsigned int kGatherDefaultTimeoutUs = 200000;   // 0.2 s: far beyond any skew between ranks in step

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void st_release_sys(int32_t *p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t *p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Layout of every rank's symmetric buffer: [2 slots][world][bytes_per_rank] payload, then at
// flag_offset [2 slots][world] int32 flags.
__global__ void __launch_bounds__(kGatherThreads)
gather_heads_kernel(const unsigned char *__restrict__ local, int bytes_per_rank, unsigned char *const *peer_bufs,
                    long long flag_offset, int32_t *seq, int rank, int world, unsigned char *out,
                    unsigned int timeout_us, int32_t *status) {
    __shared__ int sh_timeout;
    __shared__ int sh_missing[kGatherMaxWorld];
    const int tid = threadIdx.x;
    const int s = *reinterpret_cast<volatile int32_t *>(seq);
    const int slot = s & 1;
    const int tag = s + 1;
    const size_t slot_bytes = (size_t)world * bytes_per_rank;
    if (tid == 0) sh_timeout = 0;
    if (tid < kGatherMaxWorld) sh_missing[tid] = 0;

    // ---- push ---------------------------------------------------------------------------
    const int vecs = bytes_per_rank / 16;
    for (int i = tid; i < vecs * world; i += kGatherThreads) {
        const int g = i / vecs, v = i % vecs;
        const uint4 val = reinterpret_cast<const uint4 *>(local)[v];
        uint4 *dst = reinterpret_cast<uint4 *>(peer_bufs[g] + slot * slot_bytes + (size_t)rank * bytes_per_rank);
        dst[v] = val;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < world) {
        int32_t *flags = reinterpret_cast<int32_t *>(peer_bufs[tid] + flag_offset);
        st_release_sys(flags + slot * world + rank, tag);
    }

    // ---- wait (bounded) -----------------------------------------------------------------
    if (tid < world) {
        const int32_t *mine = reinterpret_cast<const int32_t *>(peer_bufs[rank] + flag_offset) + slot * world + tid;
        const unsigned long long deadline = global_timer_ns() + (unsigned long long)timeout_us * 1000ull;
        while (ld_acquire_sys(mine) < tag) {
            if (global_timer_ns() > deadline) {
                sh_timeout = 1;
                sh_missing[tid] = 1;
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();
    if (sh_timeout && tid == 0) atomicOr(status, DA_STATUS_WAIT_TIMEOUT);

    // ---- copy out (L2 loads: the rows were written by other GPUs) ----------------------------
    const uint4 *src = reinterpret_cast<const uint4 *>(peer_bufs[rank] + slot * slot_bytes);
    for (int i = tid; i < vecs * world; i += kGatherThreads) {
        const uint4 v = sh_missing[i / vecs] ? make_uint4(~0u, ~0u, ~0u, ~0u) : __ldcg(src + i);
        reinterpret_cast<uint4 *>(out)[i] = v;
    }
    if (tid == 0) *seq = tag;
}

}  // namespace da

extern "C" size_t da_gather_heads_buffer_bytes(int bytes_per_rank, int world) {
    if (bytes_per_rank < 16 || world < 1 || world > da::kGatherMaxWorld) return 0;
    return (size_t)2 * world * bytes_per_rank + (size_t)2 * world * sizeof(int32_t);
}

extern "C" int da_gather_heads(const void *local, int bytes_per_rank, void *const *peer_buffers, int32_t *seq,
                               int rank, int world, void *out, int timeout_us, int32_t *status,
                               da_stream_t stream) {
    if (!local || !peer_buffers || !seq || !out || !status) return DA_ERR_NULL;
    if (world < 1 || world > da::kGatherMaxWorld || rank < 0 || rank >= world) return DA_ERR_SHAPE;
    if (bytes_per_rank < 16 || bytes_per_rank % 16 != 0 || timeout_us < 0) return DA_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(local) | reinterpret_cast<uintptr_t>(out)) & 15) return DA_ERR_ALIGN;
    const long long flag_offset = (long long)2 * world * bytes_per_rank;
    da::gather_heads_kernel<<<1, da::kGatherThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const unsigned char *>(local), bytes_per_rank,
        reinterpret_cast<unsigned char *const *>(peer_buffers), flag_offset, seq, rank, world,
        static_cast<unsigned char *>(out),
        timeout_us > 0 ? (unsigned int)timeout_us : da::kGatherDefaultTimeoutUs, status);
    return (int)cudaGetLastError();
}

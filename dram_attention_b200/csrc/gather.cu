// All-gather of the per-KV-head-shard attention outputs over NVLink peer memory, for
// KV-head sharding on the GPUs of one node.  One launch of one CTA per rank per step:
//
//   push   the rank's own rows go into slot (seq & 1) of EVERY rank's gather buffer as 8-byte
//          words {4 bytes of payload, the step's tag seq + 1}: one naturally aligned 8-byte store
//          per word, which arrives whole, so the tag travels with the data it vouches for and
//          no fence, flag or second round over the link is needed;
//   wait   every thread polls the words of its OWN buffer that it will copy until they carry
//          the step's tag - bounded by the GPU's nanosecond timer: after `timeout_us` the block
//          sets DA_STATUS_WAIT_TIMEOUT and goes on;
//   copy   the payload halves go to the caller's output tensor (words whose tag never came are
//          written as 0xFFFFFFFF, a NaN in every floating-point format, so that a timed-out
//          gather cannot pass for a result) and the step counter is advanced.
//
// Two slots suffice: a rank can start step s + 2 (which reuses slot s & 1) only after its
// wait of step s + 1 saw every peer's words of step s + 1, and a peer sends those after
// (in stream order) its own copy of step s.  A tag is used once per slot (it grows by one per
// step), and the buffers start out zero.  No multimem, no multicast loads: ordinary peer stores
// and local loads.  The payload is a few KiB, so the step is latency-bound: one NVLink store
// round instead of the several a library ring/tree takes.
//
// The kernel is launched as a programmatic dependent of the kernel before it in the stream
// (the attention kernel, which releases its dependents early): its block is on an SM, with
// its arguments and the step counter read, when the rows it sends are ready.

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

__device__ __forceinline__ uint2 ld_word_sys(const uint2 *p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// Layout of every rank's symmetric buffer: [2 slots][world][bytes_per_rank / 4] words of 8 bytes.
__global__ void __launch_bounds__(kGatherThreads)
gather_heads_kernel(const uint32_t *__restrict__ local, int words_per_rank, uint2 *const *peer_bufs,
                    int32_t *seq, int rank, int world, uint32_t *out, unsigned int timeout_us, int32_t *status) {
    __shared__ int sh_timeout;
    const int tid = threadIdx.x;
    if (tid == 0) trace_stamp(kTraceGather, 0, 0);
    // the step counter was last written by this stream's previous gather, which is long complete
    const int s = *reinterpret_cast<volatile int32_t *>(seq);
    const int slot = s & 1;
    const uint32_t tag = (uint32_t)(s + 1);
    const int total = words_per_rank * world;
    const size_t slot_words = (size_t)total;
    if (tid == 0) sh_timeout = 0;
    uint2 *dst0 = nullptr;
    if (tid < total) dst0 = peer_bufs[tid / words_per_rank];   // first target of this thread, read early
    __syncthreads();
    // With rows of its own to send, the kernel needs the launch before it complete first.  Without (the
    // attention launch has sent them, every word vouched for by its tag), that wait moves to the end, behind
    // the wait for the other ranks.
    if (local != nullptr) griddep_wait();
    if (tid == 0) trace_stamp(kTraceGather, 0, 2);

    // ---- push (not when the attention kernel has sent the rows itself: local == nullptr) ------------
    for (int i = tid; local != nullptr && i < total; i += kGatherThreads) {
        const int g = i / words_per_rank, w = i % words_per_rank;
        uint2 *dst = (i == tid ? dst0 : peer_bufs[g]) + slot * slot_words + (size_t)rank * words_per_rank + w;
        st_word_sys(dst, local[w], tag);
    }
    if (tid == 0) trace_stamp(kTraceGather, 0, 3);

    // ---- wait (bounded) and copy out ------------------------------------------------------
    const uint2 *mine = peer_bufs[rank] + slot * slot_words;
    const unsigned long long deadline = global_timer_ns() + (unsigned long long)timeout_us * 1000ull;
    bool late = false;
    for (int i = tid; i < total; i += kGatherThreads) {
        uint2 v = ld_word_sys(mine + i);
        while (v.y != tag) {
            if (late || global_timer_ns() > deadline) {   // once late, the thread's other words get one look each
                late = true;
                v.x = ~0u;
                break;
            }
            __nanosleep(20);
            v = ld_word_sys(mine + i);
        }
        out[i] = v.x;
    }
    if (late) sh_timeout = 1;
    if (local == nullptr) griddep_wait();   // nothing after this kernel starts before the launch before it is complete
    __syncthreads();
    if (tid == 0) {
        if (sh_timeout) atomicOr(status, DA_STATUS_WAIT_TIMEOUT);
        *seq = (int32_t)tag;
        trace_stamp(kTraceGather, 0, 1);
    }
}

}  // namespace da

DA_DEFINE_TRACE_SETTER(trace_set_gather)

extern "C" size_t da_gather_heads_buffer_bytes(int bytes_per_rank, int world) {
    if (bytes_per_rank < 16 || world < 1 || world > da::kGatherMaxWorld) return 0;
    return (size_t)2 * world * 2 * bytes_per_rank;
}

extern "C" int da_gather_heads(const void *local, int bytes_per_rank, void *const *peer_buffers, int32_t *seq,
                               int rank, int world, void *out, int timeout_us, int32_t *status,
                               da_stream_t stream) {
    if (!peer_buffers || !seq || !out || !status) return DA_ERR_NULL;   // local may be NULL: see the header
    if (world < 1 || world > da::kGatherMaxWorld || rank < 0 || rank >= world) return DA_ERR_SHAPE;
    if (bytes_per_rank < 16 || bytes_per_rank % 16 != 0 || timeout_us < 0) return DA_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(local) | reinterpret_cast<uintptr_t>(out)) & 15) return DA_ERR_ALIGN;
    const cudaError_t e = da::launch_dependent(
        da::gather_heads_kernel, dim3(1), dim3(da::kGatherThreads), (size_t)0, static_cast<cudaStream_t>(stream),
        static_cast<const uint32_t *>(local), bytes_per_rank / 4, reinterpret_cast<uint2 *const *>(peer_buffers), seq,
        rank, world, static_cast<uint32_t *>(out),
        timeout_us > 0 ? (unsigned int)timeout_us : da::kGatherDefaultTimeoutUs, status);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

// Dense causal attention of the prompt (the "prefill" stage) for 16-bit element types and
// head_dim 128, on the 5th-generation tensor cores: tcgen05.mma with both operands in shared
// memory (filled by TMA tensor copies, 128-byte swizzle) and the accumulators in tensor memory.
//
// One CTA per (128 query rows, query head), TWO CTAs per SM: four softmax warps and one issuing
// warp each.  Softmax thread t owns query row t, which is lane t of tensor memory, so the
// softmax needs no shuffles: a row's logits come back with tcgen05.ld as plain registers of
// its thread.  One lane of the fifth warp issues every MMA, one lane of the sixth every TMA
// copy; the roles meet only at mbarriers (tile arrived, S ready, P ready, product complete),
// never at a CTA-wide barrier.  The MMA lane's instruction stream sets the pace of the CTA
// (measured with time stamps: 1.4 us per tile when it also issued the copies and rebuilt its
// operand descriptors per MMA), hence a warp of its own and descriptors made before the loop.
// A CTA alone leaves the tensor core idle most of the time: its softmax is a chain of phases
// (read S, maximum, exponentials on the special-function unit, sum, conversion, write P) that
// the same four warps walk tile after tile.  Two CTAs on an SM walk it out of step, so one's
// exponentials overlap the other's loads, conversions and hand-offs, and both feed the tensor
// core.  To fit twice, a CTA takes 64-key tiles (97 KB of shared memory) and 256 columns of
// tensor memory.  Per 64-key tile:
//
//   S = Q K^T      8 MMAs (M128 N64 K16), Q and the key tile K-major          -> TMEM columns 0..63 / 64..127
//   softmax        row max / exp2 / row sum in registers (log2 domain, online rescale);
//                  P goes back into tensor memory as packed 16-bit pairs, over the first 32
//                  columns of the S buffer it was computed from (tcgen05.st: a thread writes
//                  its own lane, no shared-memory traffic)
//   O += P V       4 MMAs (M128 N128 K16) with P as the A operand from tensor memory and the
//                  value tile as an MN-major B operand from shared memory, accumulating over
//                  all tiles                                                   -> TMEM columns 128..255
//
// O never leaves tensor memory until the end: the exponentials of a row are taken against a
// reference that follows the row maximum lazily, and O is rescaled in place (tcgen05.ld / st)
// only when a tile's maximum outgrows the reference by more than 2^8 - after the first tiles,
// hardly ever.  The loop is software-pipelined so that the tensor core is not waited on in
// line: S of tile j+1 is issued (into the second S buffer) before the softmax of tile j starts,
// and the product of tile j runs during the softmax of tile j+1.  The tensor core executes in
// issue order, so S of tile j+2, which overwrites the buffer P of tile j lies in, runs after
// the product that reads it.  Key and value tiles are double-buffered (a key stage is refilled
// as soon as its S is complete, a value stage once its product is).  Every wait on an
// mbarrier is bounded: a wait that runs out sets DA_STATUS_WAIT_TIMEOUT and a flag that makes
// both roles leave their loops; the CTA then frees its tensor memory and returns.
//
// GQA: query head hq reads KV head hq / rep.  Causal: key tiles above the diagonal are
// skipped, the diagonal tile is masked per element.  Rows past the end of the prompt are
// zero-filled by TMA on the way in and not stored on the way out.

#include <cuda.h>

#include "da_common.cuh"

namespace da {

constexpr int kPfRows = 128;    // query rows per CTA (= softmax threads, = TMEM lanes)
constexpr int kPfThreads = kPfRows + 64;   // plus the warp that issues the MMAs and the warp that issues the copies
constexpr int kPfKeys = 64;     // keys per tile
constexpr int kPfDim = 128;     // head_dim
constexpr int kPfQBoxBytes = kPfRows * 128;           // one TMA box of Q: 128 rows x 64 elements
constexpr int kPfQTileBytes = 2 * kPfQBoxBytes;       // 128 x 128 elements
constexpr int kPfBoxBytes = kPfKeys * 128;            // one TMA box of K or V: 64 rows x 64 elements
constexpr int kPfTileBytes = 2 * kPfBoxBytes;         // 64 x 128 elements
constexpr int kPfSmemBytes = kPfQTileBytes + 4 * kPfTileBytes + 1024;   // Q, K x2, V x2, alignment slack
constexpr uint32_t kPfTmemCols = 256;            // two S buffers of 64 columns (P over them), the product

struct PrefillParams {
    void *out;              // (S, Hq, D)
    int seq_len, n_q_heads, rep;
    float scale_log2;
    int32_t *status;
};

// ---- PTX wrappers ---------------------------------------------------------------------------

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int c0, int c1, int c2,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t *holder_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(holder_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], M128 x N128 x K16, 16-bit inputs, float accumulate
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: A is 128 lanes x 8 columns of packed 16-bit pairs (K16)
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// The same two with the accumulate flag known at compile time (no predicate to set up per MMA).
template <bool ACC>
__device__ __forceinline__ void tc_mma_c(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "n"(ACC ? 1 : 0), "r"(0u)
        : "memory");
}
template <bool ACC>
__device__ __forceinline__ void tc_mma_a_tmem_c(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "n"(ACC ? 1 : 0), "r"(0u)
        : "memory");
}

// 32 consecutive columns of this thread's TMEM lane: the load is asynchronous, its registers
// may be read only after tmem_wait32 on the same array (which lists them as operands so that
// the compiler keeps every use behind the wait).
__device__ __forceinline__ void tmem_issue32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_wait32(uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :
        : "memory");
}

__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_wait_store() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// f(chunk, values) for the four 32-column chunks starting at taddr, the load of a chunk in
// flight while the previous one is processed
template <typename F>
__device__ __forceinline__ void tmem_for_chunks(uint32_t taddr, F f) {
    uint32_t ra[32], rb[32];
    tmem_issue32(taddr, ra);
    tmem_wait32(ra);
    tmem_issue32(taddr + 32, rb);
    f(0, ra);
    tmem_wait32(rb);
    tmem_issue32(taddr + 64, ra);
    f(1, rb);
    tmem_wait32(ra);
    tmem_issue32(taddr + 96, rb);
    f(2, ra);
    tmem_wait32(rb);
    f(3, rb);
}

// Shared-memory matrix descriptors, 128-byte swizzle, version 1 (Blackwell).  Addresses and
// offsets in units of 16 bytes.
// K-major operand (rows of 128 bytes, 8-row swizzle atoms 1024 bytes apart).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand: 64 contiguous elements along N per 128-byte row, the next 64 a whole box
// (16 KiB) further; 8-row groups along K 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)(kPfBoxBytes >> 4) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ uint32_t instr_desc(bool bf16, bool b_mn_major, int n) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(kPfRows >> 4) << 24);
}

// Blackwell's two-at-a-time fp32 arithmetic and three-input maximum: the softmax is bound by instruction
// issue, and these halve the count of its multiply-adds, additions and maxima.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ unsigned long long f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f32x2_split(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if constexpr (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

template <bool BF16>
__global__ void __launch_bounds__(kPfThreads, 2)
prefill_attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                            ~(uintptr_t)1023);
    unsigned char *sQ = smem;
    unsigned char *sK = sQ + kPfQTileBytes;           // two stages
    unsigned char *sV = sK + 2 * kPfTileBytes;        // two stages
    __shared__ __align__(8) uint64_t bar_q, bar_k[2], bar_v[2], bar_s[2], bar_p[2], bar_pv;
    __shared__ uint32_t tmem_holder;
    __shared__ int sh_abort;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int n_qtiles = gridDim.x;
    const int qt = n_qtiles - 1 - blockIdx.x;     // the tiles with the most keys start first
    const int hq = blockIdx.y;
    const int hk = hq / p.rep;
    const int q0 = qt * kPfRows;
    constexpr bool bf16 = BF16;

    if (tid == 0) {
        mbar_init(&bar_q, 1);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_k[b], 1);
            mbar_init(&bar_v[b], 1);
            mbar_init(&bar_s[b], 1);
            mbar_init(&bar_p[b], kPfRows);     // every softmax thread arrives
        }
        mbar_init(&bar_pv, 1);
        mbar_fence_init();
        sh_abort = 0;
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&tmem_holder, kPfTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;
    // columns: S of even tiles 0..63, S of odd tiles 64..127 (P over the first 32 of each), O 128..255
    const uint32_t tmem_o = 2 * kPfKeys;

    // keys 0 .. q0 + 127 are visible to this tile's rows
    const int last_key = min(p.seq_len, q0 + kPfRows);
    const int n_tiles = (last_key + kPfKeys - 1) / kPfKeys;
    volatile int *abort_flag = &sh_abort;
    // a wait that ran out: say so, and let every role leave its loop at its next tile
    auto give_up = [&]() {
        atomicOr(p.status, DA_STATUS_WAIT_TIMEOUT);
        *abort_flag = 1;
    };

    if (warp == kPfRows / 32 + 1) {
        // =================== the copy warp: every TMA copy, by one lane ===================================
        // Key tile j+2 goes into the stage of tile j once S(j) is complete, value tile j+2 into the stage
        // of tile j once the product of tile j is.
        if ((tid & 31) == 0) {
            auto load_tile = [&](unsigned char *dst, const CUtensorMap *map, int j, uint64_t *bar) {
                mbar_arrive_expect_tx(bar, kPfTileBytes);
                tma_load_3d(dst, map, 0, hk, j * kPfKeys, bar);
                tma_load_3d(dst + kPfBoxBytes, map, 64, hk, j * kPfKeys, bar);
            };
            mbar_arrive_expect_tx(&bar_q, kPfQTileBytes);
            tma_load_3d(sQ, &map_q, 0, hq, q0, &bar_q);
            tma_load_3d(sQ + kPfQBoxBytes, &map_q, 64, hq, q0, &bar_q);
            load_tile(sK, &map_k, 0, &bar_k[0]);
            load_tile(sV, &map_v, 0, &bar_v[0]);
            if (n_tiles > 1) {
                load_tile(sK + kPfTileBytes, &map_k, 1, &bar_k[1]);
                load_tile(sV + kPfTileBytes, &map_v, 1, &bar_v[1]);
            }
            bool ok = true;
            for (int j = 0; ok && j + 2 < n_tiles; ++j) {
                const int b = j & 1;
                if (*abort_flag) break;
                ok = mbar_wait_bounded(&bar_s[b], (uint32_t)((j >> 1) & 1));
                if (!ok) break;
                load_tile(sK + b * kPfTileBytes, &map_k, j + 2, &bar_k[b]);
                ok = mbar_wait_bounded(&bar_pv, (uint32_t)(j & 1));
                if (!ok) break;
                load_tile(sV + b * kPfTileBytes, &map_v, j + 2, &bar_v[b]);
            }
            if (!ok) give_up();
        }
    } else if (warp == kPfRows / 32) {
        // =================== the issuing warp: every MMA, by one lane =====================================
        // Its instruction stream is the pace of the whole CTA, so everything that can be is computed
        // before the loop: the operand descriptors of both stages (an MMA's own is a 64-bit add away).
        if ((tid & 31) == 0) {
            const uint32_t idesc_s = instr_desc(bf16, false, kPfKeys), idesc_o = instr_desc(bf16, true, kPfDim);
            const uint64_t dq = desc_k_major(smem_addr(sQ));
            const uint64_t dk0 = desc_k_major(smem_addr(sK)), dk1 = desc_k_major(smem_addr(sK + kPfTileBytes));
            const uint64_t dv0 = desc_mn_major(smem_addr(sV)), dv1 = desc_mn_major(smem_addr(sV + kPfTileBytes));
            // S(j) = Q K(j)^T into the S buffer of j's parity; K(j) has arrived when this is called.  That
            // buffer's last readers were the softmax of tile j-2 (done: its P was waited for before the
            // product of tile j-2 was issued) and that product (issued earlier: the tensor core runs in order).
            auto issue_s = [&](int j) {
                tc_fence_after();
                const uint64_t kb = (j & 1) ? dk1 : dk0;
                const uint32_t d = tmem + (j & 1) * kPfKeys;
#pragma unroll
                for (int ks = 0; ks < kPfDim / 16; ++ks) {
                    const uint32_t a_off = ((ks >> 2) * kPfQBoxBytes + (ks & 3) * 32) >> 4;
                    const uint32_t b_off = ((ks >> 2) * kPfBoxBytes + (ks & 3) * 32) >> 4;
                    if (ks == 0) tc_mma_c<false>(d, dq + a_off, kb + b_off, idesc_s);
                    else tc_mma_c<true>(d, dq + a_off, kb + b_off, idesc_s);
                }
                tc_commit(&bar_s[j & 1]);
            };
            bool ok = mbar_wait_bounded(&bar_q, 0) && mbar_wait_bounded(&bar_k[0], 0);
            if (ok) issue_s(0);
            for (int j = 0; ok && j < n_tiles; ++j) {
                const int b = j & 1;
                const uint32_t use = (uint32_t)((j >> 1) & 1);     // parity of this use of a two-deep buffer
                if (*abort_flag) break;
                if (j + 1 < n_tiles) {
                    ok = mbar_wait_bounded(&bar_k[b ^ 1], (uint32_t)(((j + 1) >> 1) & 1));
                    if (!ok) break;
                    issue_s(j + 1);
                }
                // O += P(j) V(j) once every softmax thread has written its row of P (and has
                // rescaled its row of O if it had to)
                ok = mbar_wait_bounded(&bar_p[b], use) && mbar_wait_bounded(&bar_v[b], use);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a0 = tmem + (uint32_t)b * kPfKeys;
                const uint64_t vb = b ? dv1 : dv0;
                if (j == 0) tc_mma_a_tmem_c<false>(tmem + tmem_o, a0, vb, idesc_o);
                else tc_mma_a_tmem_c<true>(tmem + tmem_o, a0, vb, idesc_o);
#pragma unroll
                for (int ks = 1; ks < kPfKeys / 16; ++ks)      // 16 keys further down the tile per step
                    tc_mma_a_tmem_c<true>(tmem + tmem_o, a0 + ks * 8, vb + ((ks * 16 * 128) >> 4), idesc_o);
                tc_commit(&bar_pv);
            }
            if (!ok) give_up();
        }
    } else {
        // =================== the softmax warps: thread t = query row t = TMEM lane t ===================
        const uint32_t tmem_row = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes
        // m_used: the (log2-domain) reference the exponentials of this row are taken against.  It
        // follows the row maximum lazily: O, which accumulates in tensor memory over all tiles, is
        // rescaled only when a tile's maximum exceeds the reference by more than 8 (probabilities
        // stay below 2^8, well inside the 16-bit range; the common factor cancels in the division
        // by l at the end).  After the first few tiles that hardly ever happens, so a tile normally
        // costs one read of S from tensor memory and nothing else.
        float m_used = -INFINITY, l_run = 0.f;
        constexpr float kRescaleSlack = 8.f;
        bool ok = true;

        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            const uint32_t use = (uint32_t)((j >> 1) & 1);
            if (*abort_flag) {
                ok = false;
                break;
            }
            // S(j) was committed after the product of tile j-2 was issued: P's buffer b is free too
            ok = mbar_wait_bounded(&bar_s[b], use);
            if (!__all_sync(DA_FULL_MASK, ok)) {
                ok = false;
                break;
            }
            tc_fence_after();

            // ---- this thread's row of S, read once ------------------------------------------------
            const uint32_t tmem_s = (uint32_t)b * kPfKeys;
            const int qpos = q0 + tid;
            const int key0 = j * kPfKeys;
            const bool diagonal = key0 + kPfKeys - 1 > q0;      // some key of the tile is masked for some row
            const int n_vis = diagonal ? min(max(qpos - key0 + 1, 0), kPfKeys) : kPfKeys;   // keys this row sees
            uint32_t s0[32], s1[32];
            tmem_issue32(tmem_row + tmem_s, s0);
            tmem_issue32(tmem_row + tmem_s + 32, s1);
            tmem_wait32(s0);
            tmem_wait32(s1);
            float mx = -INFINITY;
            auto chunk_max = [&](int c, const uint32_t (&s)[32]) {
                if (!diagonal) {
                    float m1 = -INFINITY;    // two chains of three-input maxima
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        mx = max3(mx, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                        m1 = max3(m1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                    }
                    mx = fmaxf(mx, m1);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < n_vis) mx = fmaxf(mx, __uint_as_float(s[i]));
                }
            };
            chunk_max(0, s0);
            chunk_max(1, s1);
            const float m_tile = mx * p.scale_log2;

            // ---- move the reference if this tile outgrows it (whole warp together: the tensor-memory
            //      accesses are warp-wide) ---------------------------------------------------------------
            const bool grow = m_tile > m_used + kRescaleSlack;     // also true on the first tile (-inf)
            if (__any_sync(DA_FULL_MASK, grow)) {
                const float m_next = grow ? m_tile : m_used;
                const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_next);
                if (j > 0) {
                    // O holds the products up to tile j-1: wait for the last of them, scale the row
                    ok = mbar_wait_bounded(&bar_pv, (uint32_t)((j - 1) & 1));
                    if (!__all_sync(DA_FULL_MASK, ok)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < kPfDim / 32; ++c) {
                        uint32_t t[32];
                        tmem_issue32(tmem_row + tmem_o + c * 32, t);
                        tmem_wait32(t);
#pragma unroll
                        for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
                        tmem_store32(tmem_row + tmem_o + c * 32, t);
                    }
                    tmem_wait_store();
                }
                l_run *= alpha;
                m_used = m_next;
            }
            const float m_ref = (m_used == -INFINITY) ? 0.f : m_used;

            // ---- P = exp2(S * scale - reference) as packed 16-bit pairs into tensor memory, over this
            //      row's own (already read) S --------------------------------------------------------------
            uint32_t packed[32];
            unsigned long long sum2 = f32x2(0.f, 0.f);     // the row sum, even and odd keys apart
            const unsigned long long scale2 = f32x2(p.scale_log2, p.scale_log2), mref2 = f32x2(-m_ref, -m_ref);
            auto chunk_p = [&](int c, const uint32_t (&s)[32]) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float x0, x1;
                    f32x2_split(fma2(f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), scale2, mref2), x0, x1);
                    float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                    if (diagonal) {
                        if (c * 32 + i >= n_vis) p0 = 0.f;
                        if (c * 32 + i + 1 >= n_vis) p1 = 0.f;
                    }
                    sum2 = add2(sum2, f32x2(p0, p1));
                    packed[c * 16 + (i >> 1)] = pack16<BF16>(p0, p1);
                }
            };
            chunk_p(0, s0);
            chunk_p(1, s1);
            tmem_store32(tmem_row + tmem_s, packed);
            tmem_wait_store();
            {
                float s_even, s_odd;
                f32x2_split(sum2, s_even, s_odd);
                l_run += s_even + s_odd;
            }
            tc_fence_before();            // this thread's tensor-memory accesses are ordered before the arrival
            mbar_arrive(&bar_p[b]);
        }

        // ---- this row of O, normalised ---------------------------------------------------------------
        if (ok && n_tiles > 0) {
            ok = mbar_wait_bounded(&bar_pv, (uint32_t)((n_tiles - 1) & 1));
            ok = __all_sync(DA_FULL_MASK, ok);
        }
        if (!ok) {
            if ((tid & 31) == 0) give_up();
        } else {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const bool live = q0 + tid < p.seq_len;
            unsigned char *dst = static_cast<unsigned char *>(p.out) +
                                 ((size_t)(live ? q0 + tid : 0) * p.n_q_heads + hq) * kPfDim * 2;
            tmem_for_chunks(tmem_row + tmem_o, [&](int c, const uint32_t (&t)[32]) {
                if (!live) return;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int i = 8 * q;
                    reinterpret_cast<uint4 *>(dst)[4 * c + q] =
                        make_uint4(pack16<BF16>(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv),
                                   pack16<BF16>(__uint_as_float(t[i + 2]) * inv, __uint_as_float(t[i + 3]) * inv),
                                   pack16<BF16>(__uint_as_float(t[i + 4]) * inv, __uint_as_float(t[i + 5]) * inv),
                                   pack16<BF16>(__uint_as_float(t[i + 6]) * inv, __uint_as_float(t[i + 7]) * inv));
                }
            });
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kPfTmemCols);
}

// ---- host side ------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// (S, H, D) tensor with unit channel stride -> map with boxes of 64 channels x 1 head x box_rows rows
static bool make_map(CUtensorMap *map, const void *base, int seq_len, int heads, long long row_stride_elems,
                     long long head_stride_elems, bool bf16, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)kPfDim, (cuuint64_t)heads, (cuuint64_t)seq_len};
    const cuuint64_t strides[2] = {(cuuint64_t)head_stride_elems * 2, (cuuint64_t)row_stride_elems * 2};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
              const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace da

extern "C" int da_prefill_attention_supported(int head_dim, int dtype) {
    return head_dim == da::kPfDim && (dtype == DA_BF16 || dtype == DA_F16);
}

extern "C" int da_prefill_attention(const void *q, const void *k, const void *v, void *out, int seq_len,
                                    int n_q_heads, int n_kv_heads, int head_dim, long long q_row_stride,
                                    long long kv_row_stride, int dtype, int32_t *status, da_stream_t stream) {
    if (!q || !k || !v || !out || !status) return DA_ERR_NULL;
    if (seq_len < 1 || n_q_heads < 1 || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0) return DA_ERR_SHAPE;
    if (!da_prefill_attention_supported(head_dim, dtype)) return DA_ERR_UNSUPPORTED;
    if (q_row_stride < (long long)n_q_heads * head_dim || kv_row_stride < (long long)n_kv_heads * head_dim)
        return DA_ERR_SHAPE;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) return DA_ERR_ALIGN;
    if ((q_row_stride * 2) % 16 != 0 || (kv_row_stride * 2) % 16 != 0) return DA_ERR_ALIGN;
    const bool bf16 = dtype == DA_BF16;
    CUtensorMap mq, mk, mv;
    if (!da::make_map(&mq, q, seq_len, n_q_heads, q_row_stride, head_dim, bf16, da::kPfRows) ||
        !da::make_map(&mk, k, seq_len, n_kv_heads, kv_row_stride, head_dim, bf16, da::kPfKeys) ||
        !da::make_map(&mv, v, seq_len, n_kv_heads, kv_row_stride, head_dim, bf16, da::kPfKeys))
        return DA_ERR_UNSUPPORTED;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(da::prefill_attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 da::kPfSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(da::prefill_attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     da::kPfSmemBytes);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    da::PrefillParams p;
    p.out = out;
    p.seq_len = seq_len;
    p.n_q_heads = n_q_heads;
    p.rep = n_q_heads / n_kv_heads;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)head_dim);
    p.status = status;
    const dim3 grid((seq_len + da::kPfRows - 1) / da::kPfRows, n_q_heads);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (bf16) da::prefill_attention_kernel<true><<<grid, da::kPfThreads, da::kPfSmemBytes, cs>>>(mq, mk, mv, p);
    else da::prefill_attention_kernel<false><<<grid, da::kPfThreads, da::kPfSmemBytes, cs>>>(mq, mk, mv, p);
    return (int)cudaGetLastError();
}

// Dense causal attention of the prompt (the "prefill" stage) for 16-bit element types and
// head_dim 128, on the 5th-generation tensor cores: tcgen05.mma with both operands in shared
// memory (filled by TMA tensor copies, 128-byte swizzle) and the accumulators in tensor memory.
//
// One CTA of 128 threads per (128 query rows, query head).  Thread t owns query row t, which
// is lane t of tensor memory, so the softmax needs no shuffles: a row's 128 logits come back
// with tcgen05.ld as plain registers of its thread.  Per 128-key tile:
//
//   S = Q K^T      8 MMAs (M128 N128 K16), Q and the key tile K-major      -> TMEM columns 0..127 / 128..255
//   softmax        row max / exp2 / row sum in registers (log2 domain, online rescale);
//                  P is written as 16-bit values into shared memory in the swizzled K-major
//                  layout an A operand has
//   O_tile = P V   8 MMAs, the value tile as an MN-major B operand          -> TMEM columns 256..383
//   O = O * alpha + O_tile in registers (128 floats per thread)
//
// The loop is software-pipelined so that the tensor core is never waited on in line: S of
// tile j+1 is issued (into a second S buffer) before the softmax of tile j starts, and the
// product P V of tile j is added to the registers one iteration later, after the softmax of
// tile j+1.  Key and value tiles are double-buffered (a key stage is refilled as soon as its S
// is complete, a value stage once its product is).  One thread issues all TMA and MMA
// instructions; completion comes back through mbarriers, and every wait on one is bounded (a
// wait that runs out sets DA_STATUS_WAIT_TIMEOUT, and the CTA frees its tensor memory and
// leaves).
//
// GQA: query head hq reads KV head hq / rep.  Causal: key tiles above the diagonal are
// skipped, the diagonal tile is masked per element.  Rows past the end of the prompt are
// zero-filled by TMA on the way in and not stored on the way out.

#include <cuda.h>

#include "da_common.cuh"

namespace da {

constexpr int kPfRows = 128;    // query rows per CTA (= threads, = TMEM lanes)
constexpr int kPfKeys = 128;    // keys per tile
constexpr int kPfDim = 128;     // head_dim
constexpr int kPfBoxBytes = kPfRows * 128;            // one TMA box: 128 rows x 64 elements
constexpr int kPfTileBytes = 2 * kPfBoxBytes;         // 128 x 128 elements
constexpr int kPfSmemBytes = 7 * kPfTileBytes + 1024; // Q, K x2, V x2, P x2, alignment slack
constexpr uint32_t kPfTmemCols = 512;            // 384 used (two S buffers, one product); a power of two

struct PrefillParams {
    void *out;              // (S, Hq, D)
    int seq_len, n_q_heads, rep;
    float scale_log2;
    int32_t *status;
    int is_bf16;
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

__device__ __forceinline__ uint32_t instr_desc(bool bf16, bool b_mn_major) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(kPfKeys >> 3) << 17) |
           ((uint32_t)(kPfRows >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack16(float lo, float hi, bool bf16) {
    if (bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

__global__ void __launch_bounds__(kPfRows, 1)
prefill_attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                            ~(uintptr_t)1023);
    unsigned char *sQ = smem;
    unsigned char *sK = sQ + kPfTileBytes;            // two stages
    unsigned char *sV = sK + 2 * kPfTileBytes;        // two stages
    unsigned char *sP = sV + 2 * kPfTileBytes;        // two buffers
    __shared__ __align__(8) uint64_t bar_q, bar_k[2], bar_v[2], bar_s[2], bar_pv;
    __shared__ uint32_t tmem_holder;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int n_qtiles = gridDim.x;
    const int qt = n_qtiles - 1 - blockIdx.x;     // the tiles with the most keys start first
    const int hq = blockIdx.y;
    const int hk = hq / p.rep;
    const int q0 = qt * kPfRows;
    const bool bf16 = p.is_bf16 != 0;

    if (tid == 0) {
        mbar_init(&bar_q, 1);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_k[b], 1);
            mbar_init(&bar_v[b], 1);
            mbar_init(&bar_s[b], 1);
        }
        mbar_init(&bar_pv, 1);
        mbar_fence_init();
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&tmem_holder, kPfTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;
    const uint32_t tmem_row = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes
    // columns: S of even tiles 0..127, S of odd tiles 128..255, the P V product of one tile 256..383
    const uint32_t tmem_o = 2 * kPfKeys;

    // keys 0 .. q0 + 127 are visible to this tile's rows
    const int last_key = min(p.seq_len, q0 + kPfRows);
    const int n_tiles = (last_key + kPfKeys - 1) / kPfKeys;

    auto load_tile = [&](unsigned char *dst, const CUtensorMap *map, int j, uint64_t *bar) {
        mbar_arrive_expect_tx(bar, kPfTileBytes);
        tma_load_3d(dst, map, 0, hk, j * kPfKeys, bar);
        tma_load_3d(dst + kPfBoxBytes, map, 64, hk, j * kPfKeys, bar);
    };
    const uint32_t idesc_s = instr_desc(bf16, false), idesc_o = instr_desc(bf16, true);
    // S(j) = Q K(j)^T into the S buffer of j's parity; K(j) has arrived when this is called
    auto issue_s = [&](int j) {
        tc_fence_after();
        const uint32_t a0 = smem_addr(sQ), b0 = smem_addr(sK + (j & 1) * kPfTileBytes);
#pragma unroll
        for (int ks = 0; ks < kPfDim / 16; ++ks) {
            const uint32_t off = (ks >> 2) * kPfBoxBytes + (ks & 3) * 32;
            tc_mma(tmem + (j & 1) * kPfKeys, desc_k_major(a0 + off), desc_k_major(b0 + off), idesc_s, ks > 0);
        }
    };

    bool ok = true;
    if (tid == 0) {
        mbar_arrive_expect_tx(&bar_q, kPfTileBytes);
        tma_load_3d(sQ, &map_q, 0, hq, q0, &bar_q);
        tma_load_3d(sQ + kPfBoxBytes, &map_q, 64, hq, q0, &bar_q);
        load_tile(sK, &map_k, 0, &bar_k[0]);
        if (n_tiles > 1) load_tile(sK + kPfTileBytes, &map_k, 1, &bar_k[1]);
        load_tile(sV, &map_v, 0, &bar_v[0]);
        ok = mbar_wait_bounded(&bar_q, 0) && mbar_wait_bounded(&bar_k[0], 0);
        if (ok) issue_s(0);
        tc_commit(&bar_s[0]);   // also on failure: arrives at once, nobody is left waiting
    }
    __syncwarp();

    float o[kPfDim];
#pragma unroll
    for (int i = 0; i < kPfDim; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    // O = O * alpha(j_prev) + the P V product of tile j_prev, once its MMAs are complete (the
    // rescale by a tile's alpha waits for that tile's product, so it is one fused multiply-add)
    float alpha_pending = 1.f;
    auto add_product = [&](int j_prev) {
        ok = mbar_wait_bounded(&bar_pv, (uint32_t)(j_prev & 1)) && ok;
        tc_fence_after();
        tmem_for_chunks(tmem_row + tmem_o, [&](int c, const uint32_t (&t)[32]) {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_pending, __uint_as_float(t[i]));
        });
    };

    for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const uint32_t use = (uint32_t)((j >> 1) & 1);     // parity of this use of a two-deep buffer
        ok = mbar_wait_bounded(&bar_s[b], use) && ok;
        tc_fence_after();
        if (tid == 0) {
            // the tensor core goes on with the next tile's logits while this tile's softmax runs
            if (j + 1 < n_tiles) {
                ok = mbar_wait_bounded(&bar_k[b ^ 1], (uint32_t)(((j + 1) >> 1) & 1)) && ok;
                if (ok) issue_s(j + 1);
                tc_commit(&bar_s[b ^ 1]);
            }
            if (j + 2 < n_tiles) load_tile(sK + b * kPfTileBytes, &map_k, j + 2, &bar_k[b]);   // S(j) is complete
        }
        __syncwarp();

        // ---- softmax of this thread's row -----------------------------------------------------
        const uint32_t tmem_s = (uint32_t)b * kPfKeys;
        const int qpos = q0 + tid;
        const int key0 = j * kPfKeys;
        const bool diagonal = key0 + kPfKeys - 1 > q0;      // some key of the tile is masked for some row
        // keys of this tile visible to this row (all 128 below the diagonal)
        const int n_vis = diagonal ? min(max(qpos - key0 + 1, 0), kPfKeys) : kPfKeys;
        float mx = -INFINITY;
        tmem_for_chunks(tmem_row + tmem_s, [&](int c, const uint32_t (&s)[32]) {
            if (!diagonal) {
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(s[i]));
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (c * 32 + i < n_vis) mx = fmaxf(mx, __uint_as_float(s[i]));
            }
        });
        const float m_new = fmaxf(m_run, mx * p.scale_log2);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = fast_exp2(m_run - m_safe);
        float row_sum = 0.f;
        unsigned char *sPb = sP + b * kPfTileBytes;          // last read by the product of tile j-2: complete
        tmem_for_chunks(tmem_row + tmem_s, [&](int c, const uint32_t (&s)[32]) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), p.scale_log2, -m_safe));
                float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, -m_safe));
                if (diagonal) {
                    if (c * 32 + i >= n_vis) p0 = 0.f;
                    if (c * 32 + i + 1 >= n_vis) p1 = 0.f;
                }
                row_sum += p0 + p1;
                packed[i >> 1] = pack16(p0, p1, bf16);
            }
            // row `tid` of P, keys 32c .. 32c+31 = 64 bytes = four 16-byte chunks of the row's box
            unsigned char *row = sPb + (c >> 1) * kPfBoxBytes + tid * 128;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int chunk = (c & 1) * 4 + q;                     // chunk inside the 128-byte row
                const int phys = chunk ^ (tid & 7);                    // 128-byte swizzle
                *reinterpret_cast<uint4 *>(row + phys * 16) =
                    make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            }
        });
        l_run = l_run * alpha + row_sum;
        m_run = m_new;
        if (j > 0) add_product(j - 1);
        alpha_pending = alpha;
        proxy_fence_async_smem();     // P must be visible to the tensor core's reads of shared memory
        tc_fence_before();
        const bool abort_now = __syncthreads_or(!ok);
        if (abort_now) {
            ok = false;
            break;
        }

        // ---- O_tile = P V (accumulated into registers one iteration later) ------------------------
        if (tid == 0) {
            // the value stage of tile j+1 was last read by the product of tile j-1: complete
            if (j + 1 < n_tiles) load_tile(sV + (b ^ 1) * kPfTileBytes, &map_v, j + 1, &bar_v[b ^ 1]);
            ok = mbar_wait_bounded(&bar_v[b], use) && ok;
            if (ok) {
                tc_fence_after();
                const uint32_t a0 = smem_addr(sPb), b0 = smem_addr(sV + b * kPfTileBytes);
#pragma unroll
                for (int ks = 0; ks < kPfKeys / 16; ++ks) {
                    const uint32_t a_off = (ks >> 2) * kPfBoxBytes + (ks & 3) * 32;
                    const uint32_t b_off = ks * 16 * 128;               // 16 keys further down the tile
                    tc_mma(tmem + tmem_o, desc_k_major(a0 + a_off), desc_mn_major(b0 + b_off), idesc_o, ks > 0);
                }
            }
            tc_commit(&bar_pv);
        }
        __syncwarp();
    }
    if (ok && n_tiles > 0) add_product(n_tiles - 1);

    // ---- write this row -------------------------------------------------------------------------
    const bool failed = __syncthreads_or(!ok);
    if (failed) {
        if (tid == 0) atomicOr(p.status, DA_STATUS_WAIT_TIMEOUT);
    } else if (q0 + tid < p.seq_len) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint4 *dst = reinterpret_cast<uint4 *>(static_cast<unsigned char *>(p.out) +
                                               ((size_t)(q0 + tid) * p.n_q_heads + hq) * kPfDim * 2);
#pragma unroll
        for (int c = 0; c < kPfDim / 8; ++c) {
            dst[c] = make_uint4(pack16(o[8 * c] * inv, o[8 * c + 1] * inv, bf16),
                                pack16(o[8 * c + 2] * inv, o[8 * c + 3] * inv, bf16),
                                pack16(o[8 * c + 4] * inv, o[8 * c + 5] * inv, bf16),
                                pack16(o[8 * c + 6] * inv, o[8 * c + 7] * inv, bf16));
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

// (S, H, D) tensor with unit channel stride -> map with boxes of 64 channels x 1 head x 128 rows
static bool make_map(CUtensorMap *map, const void *base, int seq_len, int heads, long long row_stride_elems,
                     long long head_stride_elems, bool bf16) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)kPfDim, (cuuint64_t)heads, (cuuint64_t)seq_len};
    const cuuint64_t strides[2] = {(cuuint64_t)head_stride_elems * 2, (cuuint64_t)row_stride_elems * 2};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)kPfRows};
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
    if (!da::make_map(&mq, q, seq_len, n_q_heads, q_row_stride, head_dim, bf16) ||
        !da::make_map(&mk, k, seq_len, n_kv_heads, kv_row_stride, head_dim, bf16) ||
        !da::make_map(&mv, v, seq_len, n_kv_heads, kv_row_stride, head_dim, bf16))
        return DA_ERR_UNSUPPORTED;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(da::prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
    p.is_bf16 = bf16 ? 1 : 0;
    const dim3 grid((seq_len + da::kPfRows - 1) / da::kPfRows, n_q_heads);
    da::prefill_attention_kernel<<<grid, da::kPfRows, da::kPfSmemBytes, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv,
                                                                                                           p);
    return (int)cudaGetLastError();
}

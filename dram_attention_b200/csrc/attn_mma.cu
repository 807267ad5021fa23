// Decode attention for 16-bit element types: same split-K structure, unit
// scheduling, append and merge as the float32 kernel (attn.cu), with the two
// contractions of a 16-token unit on tensor cores.
//
// The GQA group has at most 8 query rows, far below the 64-row minimum tile of
// tcgen05.mma, so the contractions use warp-level mma.sync m16n8k16 (rows
// 0..rep-1 of the 16-row A operand are live, the rest are zero).  That cuts the
// instruction count per unit about eightfold against CUDA-core FMAs, which is what
// leaves the kernel waiting on HBM instead of on the issue slots.
//
//   S  = Q K^T   A = Q fragments held in registers for the whole kernel,
//                B = key rows straight from shared memory with ldmatrix;
//   O += P V     A = P re-packed from the S accumulators (FlashAttention-2 register
//                reuse), B = value rows with ldmatrix.trans.
//
// Shared-memory layout of a stage: 16 tokens, each its key row then its value row,
// padded by 16 bytes per token so that the 8 row addresses of an ldmatrix tile fall
// in distinct banks.  A token of the slot table arrives by one bulk copy (TMA) of
// both rows (they are contiguous in the page layout), issued one per lane.

#include "attn_common.cuh"

namespace da {

template <typename T> struct MmaTraits;
template <> struct MmaTraits<__nv_bfloat16> {
    __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __device__ __forceinline__ static void mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
        // rows 8..15 of A are zero: a1 = a3 = 0
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    }
};
template <> struct MmaTraits<__half> {
    __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __device__ __forceinline__ static void mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *row_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(row_addr))
                 : "memory");
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *row_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(row_addr))
                 : "memory");
}

template <typename T, int D, int REP, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 4 ? 2 : 1) decode_attention_mma_kernel(const AttnParams p) {
    static_assert(sizeof(T) == 2 && REP <= 8 && D % 32 == 0, "16-bit types, at most 8 query rows");
    constexpr int E = 2;
    constexpr int ROWB = D * E;                   // one key (or value) row in HBM
    constexpr int PITCH = 2 * ROWB + 16;          // padded token (key row, value row) in shared memory
    constexpr int STAGEB = kUnitTokens * PITCH;
    constexpr int KSTEPS = D / 16;                // k-steps of the QK contraction
    constexpr int NT = D / 8;                     // n-tiles of the PV contraction
    constexpr int PW = PartialRow<D>::kWidth;
    constexpr float NEG_INF = -INFINITY;
    constexpr int THREADS = WARPS * 32;

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t bars[WARPS][STAGES];
    __shared__ float red[WARPS][REP][PW];
    __shared__ int sh_last;
    __shared__ unsigned char perm_s[WARPS][64];

    const int h = blockIdx.y;
    const int x = blockIdx.x;
    const int splits = gridDim.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int row = lane >> 2;  // query row of this lane's accumulators
    const int qd = lane & 3;    // position inside the quad

    // ---- position and unit range ------------------------------------------------
    const int pos = p.start_pos_dev ? *p.start_pos_dev : p.start_pos_host;
    int t_new = pos - p.dram_tokens;
    bool pos_ok = true;
    if (t_new < 0 || t_new >= p.local_capacity) {
        pos_ok = false;
        if (tid == 0 && x == 0) atomicOr(p.status, DA_STATUS_BAD_POSITION);
        t_new = t_new < 0 ? 0 : p.local_capacity - 1;
    }
    const int n_local = t_new + 1;
    const int n_prefix = p.n_prefix_tokens;
    const int n_workers = splits * WARPS;
    const int worker = x * WARPS + warp;
    const UnitPlan plan = plan_units(p, h, n_local, worker, n_workers, lane);
    const int units_prefix = plan.units_slots;   // units of this launch that come from the slot table
    const int n_my = plan.n_my;

    unsigned char *my_stages = smem + (size_t)warp * STAGES * STAGEB;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(&bars[warp][s], 1);
    }
    mbar_fence_init();
    __syncthreads();

    // ---- append the new key/value to the local window -----------------------------
    if (x == 0 && warp == 0 && pos_ok && p.phase != 2) {
        const uint4 *sk = reinterpret_cast<const uint4 *>(p.new_k + (size_t)h * ROWB);
        const uint4 *sv = reinterpret_cast<const uint4 *>(p.new_v + (size_t)h * ROWB);
        const size_t off = ((size_t)t_new * p.local_tok_stride + (size_t)h * p.local_head_stride) * E;
        uint4 *dk = reinterpret_cast<uint4 *>(p.local_k + off);
        uint4 *dv = reinterpret_cast<uint4 *>(p.local_v + off);
        for (int i = lane; i < ROWB / 16; i += 32) {
            dk[i] = sk[i];
            dv[i] = sv[i];
        }
    }

    // ---- Q as A-operand fragments: rows >= REP are zero -------------------------------
    uint32_t qa0[KSTEPS], qa2[KSTEPS];
    {
        const unsigned char *qrow = p.q + ((size_t)(h * REP + (row < REP ? row : 0))) * ROWB;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint32_t w0 = *reinterpret_cast<const uint32_t *>(qrow + (16 * ks + 2 * qd) * E);
            const uint32_t w2 = *reinterpret_cast<const uint32_t *>(qrow + (16 * ks + 8 + 2 * qd) * E);
            qa0[ks] = row < REP ? w0 : 0u;
            qa2[ks] = row < REP ? w2 : 0u;
        }
    }

    float m_run = NEG_INF, l_part = 0.f;  // row max (quad-uniform); this lane's share of the row sum
    float o[NT][4];
#pragma unroll
    for (int d = 0; d < NT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    const uint64_t stream_policy = l2_policy_evict_first();   // the KV stream is read once per step
    // The warp visits its units in the order perm[0], perm[1], ...: DRAM-sourced units first.
    int perm[2] = {0, 0};
    const bool planned = p.slot_source != nullptr;   // then the host guarantees n_my <= 64
    if (planned) plan_order(plan, lane, perm, perm_s[warp]);
    auto unit_index = [&](int it) -> int {
        const int v = plan_lookup(perm, it);
        return planned ? v : it;
    };
    // first slot-table token of the warp's unit with index idx, and the DRAM page to read it from (or -1)
    auto unit_base = [&](int u, int idx) -> int {
        const int b = plan_lookup(plan.base, idx);
        return p.phase == 0 ? u * kUnitTokens : b;
    };
    auto unit_src = [&](int idx) -> int {
        const int v = plan_lookup(plan.src, idx);
        return planned ? v : -1;
    };
    auto unit_tokens = [&](int u, int base) -> int {
        if (u < units_prefix) return min(kUnitTokens, n_prefix - base);
        return min(kUnitTokens, n_local - (u - units_prefix) * kUnitTokens);
    };

    // Slot-table units: one bulk copy per token (its key and value rows are contiguous in
    // HBM), issued by lanes 0..15.  Local-window units: one copy per row, key rows by
    // lanes 0..15 and value rows by lanes 16..31.
    auto issue = [&](int s, int it) {
        const int idx = unit_index(it);
        const int u = worker + idx * n_workers;
        uint64_t *bar = &bars[warp][s];
        unsigned char *dst = my_stages + (size_t)s * STAGEB;
        const int base = unit_base(u, idx);
        const int src_page = unit_src(idx);
        const int ntok = unit_tokens(u, base);
        if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)ntok * 2 * ROWB);
        __syncwarp();
        const int tl = lane & 15;
        const int is_v = lane >> 4;
        if (tl < ntok) {
            if (u < units_prefix) {
                if (!is_v) {
                    const size_t tok = (size_t)base + tl;
                    const unsigned char *src =
                        src_page < 0
                            ? p.prefix + ((size_t)h * p.prefix_head_stride + tok * 2 * D) * E
                            : p.dram + ((size_t)h * p.dram_head_stride +
                                        ((size_t)src_page * p.page_tokens + tok % p.page_tokens) * 2 * D) * E;
                    bulk_copy_g2s_hint(dst + tl * PITCH, src, 2 * ROWB, bar, stream_policy);
                }
            } else {
                const int t = (u - units_prefix) * kUnitTokens + tl;
                const unsigned char *src;
                if (t == t_new) {
                    src = (is_v ? p.new_v : p.new_k) + (size_t)h * ROWB;
                } else {
                    src = (is_v ? p.local_v : p.local_k) +
                          ((size_t)t * p.local_tok_stride + (size_t)h * p.local_head_stride) * E;
                }
                bulk_copy_g2s_hint(dst + tl * PITCH + is_v * ROWB, src, ROWB, bar, stream_policy);
            }
        }
    };

    for (int it = 0; it < STAGES && it < n_my; ++it) issue(it, it);

    // ldmatrix row addresses of this lane inside a stage
    const int lm = lane >> 3;   // which 8x8 tile of the x4 load
    const int lr = lane & 7;    // row inside the tile
    const int k_off = lr * PITCH + lm * 16;                               // key tile: rows lr, 16-byte column block lm
    const int v_off = ROWB + ((lm & 1) * 8 + lr) * PITCH + (lm >> 1) * 16;    // value tile (transposed load)

    for (int it = 0; it < n_my; ++it) {
        const int s = it % STAGES;
        const bool arrived = mbar_wait_bounded(&bars[warp][s], (uint32_t)((it / STAGES) & 1));
        if (!__all_sync(DA_FULL_MASK, arrived)) {
            if (lane == 0) atomicOr(p.status, DA_STATUS_WAIT_TIMEOUT);
            break;
        }
        const int idx = unit_index(it);
        const int u = worker + idx * n_workers;
        const int base = unit_base(u, idx);
        const int ntok = unit_tokens(u, base);
        unsigned char *sb = my_stages + (size_t)s * STAGEB;
        if (unit_src(idx) >= 0 && u < units_prefix) {
            // this unit came from DRAM: write it through to its slot (512 bytes per token)
            unsigned char *slot = const_cast<unsigned char *>(p.prefix) +
                                  ((size_t)h * p.prefix_head_stride + (size_t)base * 2 * D) * E;
            for (int i = lane; i < ntok * (2 * ROWB / 16); i += 32) {
                const int t = i / (2 * ROWB / 16), c = i % (2 * ROWB / 16);
                reinterpret_cast<uint4 *>(slot + (size_t)t * 2 * ROWB)[c] =
                    reinterpret_cast<const uint4 *>(sb + t * PITCH)[c];
            }
        }
        if (ntok < kUnitTokens) {
            // rows past the end hold stale bytes: zero the value rows so that 0 * garbage
            // cannot produce NaN (their logits are masked below)
            for (int i = lane; i < (kUnitTokens - ntok) * (ROWB / 16); i += 32) {
                const int r = ntok + i / (ROWB / 16);
                reinterpret_cast<uint4 *>(sb + ROWB + r * PITCH)[i % (ROWB / 16)] = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // ---- S = Q K^T for 16 tokens (two n-tiles of 8) --------------------------------
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kp = 0; kp < KSTEPS / 2; ++kp) {
            uint32_t b[4];
            ldmatrix_x4(b, sb + k_off + kp * 64);                 // tokens 0..7, channels 32kp .. 32kp+31
            MmaTraits<T>::mma(s0, qa0[2 * kp], qa2[2 * kp], b[0], b[1]);
            MmaTraits<T>::mma(s0, qa0[2 * kp + 1], qa2[2 * kp + 1], b[2], b[3]);
            ldmatrix_x4(b, sb + k_off + 8 * PITCH + kp * 64);     // tokens 8..15
            MmaTraits<T>::mma(s1, qa0[2 * kp], qa2[2 * kp], b[0], b[1]);
            MmaTraits<T>::mma(s1, qa0[2 * kp + 1], qa2[2 * kp + 1], b[2], b[3]);
        }
        // this lane: row `row`, tokens 2qd, 2qd+1, 8+2qd, 9+2qd
        float v0 = s0[0] * p.scale_log2, v1 = s0[1] * p.scale_log2;
        float v2 = s1[0] * p.scale_log2, v3 = s1[1] * p.scale_log2;
        if (2 * qd >= ntok) v0 = NEG_INF;
        if (2 * qd + 1 >= ntok) v1 = NEG_INF;
        if (8 + 2 * qd >= ntok) v2 = NEG_INF;
        if (9 + 2 * qd >= ntok) v3 = NEG_INF;

        // ---- online softmax (log2 domain) -----------------------------------------------
        float mx = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3));
        mx = fmaxf(mx, __shfl_xor_sync(DA_FULL_MASK, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(DA_FULL_MASK, mx, 2));
        const float mnew = fmaxf(m_run, mx);
        const float msafe = (mnew == NEG_INF) ? 0.f : mnew;
        const float alpha = fast_exp2(m_run - msafe);
        v0 = fast_exp2(v0 - msafe);
        v1 = fast_exp2(v1 - msafe);
        v2 = fast_exp2(v2 - msafe);
        v3 = fast_exp2(v3 - msafe);
        l_part = l_part * alpha + ((v0 + v1) + (v2 + v3));
        m_run = mnew;
#pragma unroll
        for (int d = 0; d < NT; ++d) {
            o[d][0] *= alpha;
            o[d][1] *= alpha;
        }
        const uint32_t pa0 = MmaTraits<T>::pack(v0, v1);  // tokens 0..7 block of P
        const uint32_t pa2 = MmaTraits<T>::pack(v2, v3);  // tokens 8..15 block of P

        // ---- O += P V ---------------------------------------------------------------------
#pragma unroll
        for (int dp = 0; dp < NT / 2; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, sb + v_off + dp * 32);           // channels 16dp .. 16dp+15, all 16 tokens
            MmaTraits<T>::mma(o[2 * dp], pa0, pa2, b[0], b[1]);
            MmaTraits<T>::mma(o[2 * dp + 1], pa0, pa2, b[2], b[3]);
        }

        __syncwarp();
        if (it + STAGES < n_my) issue(s, it + STAGES);
    }

    // ---- this warp's partial: finish the row sum, publish --------------------------------
    l_part += __shfl_xor_sync(DA_FULL_MASK, l_part, 1);
    l_part += __shfl_xor_sync(DA_FULL_MASK, l_part, 2);
    if (row < REP) {
#pragma unroll
        for (int d = 0; d < NT; ++d) {
            red[warp][row][8 * d + 2 * qd] = o[d][0];
            red[warp][row][8 * d + 2 * qd + 1] = o[d][1];
        }
        if (qd == 0) {
            red[warp][row][D] = m_run;
            red[warp][row][D + 1] = l_part;
        }
    }
    __syncthreads();

    // ---- merge the warps, write this CTA's partial ------------------------------------
    float *part = p.partials + ((size_t)(h * p.part_rows + p.part_offset + x) * REP) * PW;
    for (int e = tid; e < REP * PW; e += THREADS) {
        const int r = e / PW;
        const int c = e % PW;
        float mn = NEG_INF;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mn = fmaxf(mn, red[w][r][D]);
        float outv;
        if (c == D) {
            outv = mn;
        } else if (c > D + 1) {
            outv = 0.f;  // padding
        } else {
            const float ms = (mn == NEG_INF) ? 0.f : mn;
            outv = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) outv += red[w][r][c] * fast_exp2(red[w][r][D] - ms);
        }
        part[e] = outv;
    }
    if (p.phase == 1) return;   // phase 2 merges the rows of both launches
    __threadfence();
    __syncthreads();
    unsigned int *tickets = p.counters;
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&tickets[h], 1u);
        sh_last = (ticket == (unsigned int)(splits - 1));
    }
    __syncthreads();
    if (!sh_last) return;

    // ---- last CTA of this head (of this launch) ---------------------------------------------
    // Every other CTA fenced its partial row before it took its ticket, and the merge reads the
    // rows with L2 loads issued after the barrier that follows the ticket: no fence on this side.
    merge_splits<T, D, REP, THREADS>(p, h, p.merge_first, p.merge_rows, reinterpret_cast<float *>(smem), nullptr);
    // every CTA of this head is done with the split: the one the LRU update left becomes current
    if (p.phase == 2 && tid == 0) p.flip[h] ^= 1;
    if (tid == 0) tickets[h] = 0u;
}

template <typename T, int D, int REP, int WARPS>
static cudaError_t launch_mma_w(const AttnParams &p, int n_kv_heads, cudaStream_t stream) {

    constexpr int STAGEB = kUnitTokens * (2 * D * 2 + 16);
    constexpr int STAGES = STAGEB > 8192 ? 3 : 4;
    constexpr int SMEM = WARPS * STAGES * STAGEB;
    auto kern = decode_attention_mma_kernel<T, D, REP, STAGES, WARPS>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    dim3 grid(p.phase == 1 ? attn_splits_phase1(n_kv_heads) : attn_splits(n_kv_heads), n_kv_heads);
    kern<<<grid, WARPS * 32, SMEM, stream>>>(p);
    return cudaGetLastError();
}

template <typename T, int D, int REP>
static cudaError_t launch_mma(const AttnParams &p, int n_kv_heads, cudaStream_t stream) {
    if (p.phase == 1) return launch_mma_w<T, D, REP, kAttnPhase1Warps>(p, n_kv_heads, stream);
    return launch_mma_w<T, D, REP, kAttnWarps>(p, n_kv_heads, stream);
}

template <typename T>
static cudaError_t dispatch_mma(const AttnParams &p, int n_kv_heads, int rep, int head_dim, cudaStream_t s) {
#define DA_MMA_CASE(DD, RR) \
    if (head_dim == DD && rep == RR) return launch_mma<T, DD, RR>(p, n_kv_heads, s);
    DA_MMA_CASE(128, 1) DA_MMA_CASE(128, 2) DA_MMA_CASE(128, 4) DA_MMA_CASE(128, 8)
    DA_MMA_CASE(64, 1) DA_MMA_CASE(64, 2) DA_MMA_CASE(64, 4) DA_MMA_CASE(64, 8)
#undef DA_MMA_CASE
    return cudaErrorInvalidValue;
}

cudaError_t launch_attention_mma(const AttnParams &p, int n_kv_heads, int rep, int head_dim, int dtype,
                                 cudaStream_t stream) {
    if (dtype == DA_BF16) return dispatch_mma<__nv_bfloat16>(p, n_kv_heads, rep, head_dim, stream);
    if (dtype == DA_F16) return dispatch_mma<__half>(p, n_kv_heads, rep, head_dim, stream);
    return cudaErrorInvalidValue;
}

}  // namespace da

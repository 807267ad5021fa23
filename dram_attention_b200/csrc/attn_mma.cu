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

#include "attn_body.cuh"

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
    __device__ __forceinline__ static void mma16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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
    __device__ __forceinline__ static void mma16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

// Arithmetic of a 16-token unit on tensor cores.  FULL = false: at most 8 query rows (rows 8..15
// of the A operand are zero and their accumulators are never read); FULL = true: up to 16 rows
// (several query tokens per call).
template <typename T, int D_, bool FULL>
struct MmaMath {
    using Elem = T;
    static constexpr int kD = D_;
    static constexpr int ROWB = kD * 2;                   // one key (or value) row in HBM
    static constexpr int kPitch = 2 * ROWB + 16;          // padded token (key row, value row) in shared memory
    static constexpr int STAGEB = kUnitTokens * kPitch;
    static constexpr bool kPerTokenCopy = true;
    static constexpr int KSTEPS = kD / 16;                // k-steps of the QK contraction
    static constexpr int NT = kD / 8;                     // n-tiles of the PV contraction
    static constexpr int NR = FULL ? 2 : 1;               // query rows per lane: lane / 4 (and + 8)
    static_assert(sizeof(T) == 2 && kD % 32 == 0, "16-bit element types");

    struct State {
        uint32_t qa[NR][2][KSTEPS];   // A fragments of Q: [row half][k half][k-step]
        float m_run[NR];              // row max (quad-uniform)
        float l_part[NR];             // this lane's share of the row sum
        float o[NT][4];
        int back[NR];                 // tokens at the end of a unit's range that the row must not see
    };

    __device__ __forceinline__ static void init(State &st, const AttnParams &p, int h, int lane, int rows) {
        const int qd = lane & 3;
        const int hq = p.n_kv_heads * p.rep;
#pragma unroll
        for (int half = 0; half < NR; ++half) {
            const int r = (lane >> 2) + 8 * half;
            const bool live = r < rows;
            const int tok = p.q_tok0 + (live ? r / p.rep : 0);
            const unsigned char *qrow = p.q + ((size_t)tok * hq + (size_t)h * p.rep + (live ? r % p.rep : 0)) * ROWB;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                const uint32_t w0 = *reinterpret_cast<const uint32_t *>(qrow + (16 * ks + 2 * qd) * 2);
                const uint32_t w2 = *reinterpret_cast<const uint32_t *>(qrow + (16 * ks + 8 + 2 * qd) * 2);
                st.qa[half][0][ks] = live ? w0 : 0u;
                st.qa[half][1][ks] = live ? w2 : 0u;
            }
            st.back[half] = live ? p.s_total - 1 - tok : 0;
            st.m_run[half] = -INFINITY;
            st.l_part[half] = 0.f;
        }
#pragma unroll
        for (int d = 0; d < NT; ++d) st.o[d][0] = st.o[d][1] = st.o[d][2] = st.o[d][3] = 0.f;
    }

    __device__ __forceinline__ static void mma(float (&d)[4], const State &st, int ks, uint32_t b0, uint32_t b1) {
        if constexpr (FULL) MmaTraits<T>::mma16(d, st.qa[0][0][ks], st.qa[1][0][ks], st.qa[0][1][ks], st.qa[1][1][ks], b0, b1);
        else MmaTraits<T>::mma(d, st.qa[0][0][ks], st.qa[0][1][ks], b0, b1);
    }

    // `avail` = tokens that exist from the unit's first token on; a row sees the first avail - back
    __device__ __forceinline__ static void consume(State &st, const unsigned char *sb, int avail, int lane,
                                                   float scale_log2) {
        constexpr float NEG_INF = -INFINITY;
        const int qd = lane & 3;
        // ldmatrix row addresses of this lane inside a stage
        const int lm = lane >> 3;   // which 8x8 tile of the x4 load
        const int lr = lane & 7;    // row inside the tile
        const int k_off = lr * kPitch + lm * 16;                               // key tile: rows lr, 16-byte column block lm
        const int v_off = ROWB + ((lm & 1) * 8 + lr) * kPitch + (lm >> 1) * 16;    // value tile (transposed load)

        // ---- S = Q K^T for 16 tokens (two n-tiles of 8) --------------------------------
        // four independent accumulation chains (even / odd k-steps of each n-tile), added at the end
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        float s0b[4] = {0.f, 0.f, 0.f, 0.f}, s1b[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kp = 0; kp < KSTEPS / 2; ++kp) {
            uint32_t b[4], c[4];
            ldmatrix_x4(b, sb + k_off + kp * 64);                 // tokens 0..7, channels 32kp .. 32kp+31
            ldmatrix_x4(c, sb + k_off + 8 * kPitch + kp * 64);    // tokens 8..15
            mma(s0, st, 2 * kp, b[0], b[1]);
            mma(s1, st, 2 * kp, c[0], c[1]);
            mma(s0b, st, 2 * kp + 1, b[2], b[3]);
            mma(s1b, st, 2 * kp + 1, c[2], c[3]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s0[i] += s0b[i];
            s1[i] += s1b[i];
        }
        uint32_t pa[NR][2];
#pragma unroll
        for (int half = 0; half < NR; ++half) {
            // this lane: row lane/4 + 8*half, tokens 2qd, 2qd+1, 8+2qd, 9+2qd
            const int lim = avail - st.back[half];
            float v0 = s0[2 * half] * scale_log2, v1 = s0[2 * half + 1] * scale_log2;
            float v2 = s1[2 * half] * scale_log2, v3 = s1[2 * half + 1] * scale_log2;
            if (2 * qd >= lim) v0 = NEG_INF;
            if (2 * qd + 1 >= lim) v1 = NEG_INF;
            if (8 + 2 * qd >= lim) v2 = NEG_INF;
            if (9 + 2 * qd >= lim) v3 = NEG_INF;

            // ---- online softmax (log2 domain) -----------------------------------------------
            float mx = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3));
            mx = fmaxf(mx, __shfl_xor_sync(DA_FULL_MASK, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(DA_FULL_MASK, mx, 2));
            const float mnew = fmaxf(st.m_run[half], mx);
            const float msafe = (mnew == NEG_INF) ? 0.f : mnew;
            const float alpha = fast_exp2(st.m_run[half] - msafe);
            v0 = fast_exp2(v0 - msafe);
            v1 = fast_exp2(v1 - msafe);
            v2 = fast_exp2(v2 - msafe);
            v3 = fast_exp2(v3 - msafe);
            st.l_part[half] = st.l_part[half] * alpha + ((v0 + v1) + (v2 + v3));
            st.m_run[half] = mnew;
            // once the running maxima have settled alpha is exactly 1 for every row: skip the rescale
            if (__any_sync(DA_FULL_MASK, alpha != 1.f)) {
#pragma unroll
                for (int d = 0; d < NT; ++d) {
                    st.o[d][2 * half] *= alpha;
                    st.o[d][2 * half + 1] *= alpha;
                }
            }
            pa[half][0] = MmaTraits<T>::pack(v0, v1);  // tokens 0..7 block of P
            pa[half][1] = MmaTraits<T>::pack(v2, v3);  // tokens 8..15 block of P
        }

        // ---- O += P V ---------------------------------------------------------------------
#pragma unroll
        for (int dp = 0; dp < NT / 2; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, sb + v_off + dp * 32);           // channels 16dp .. 16dp+15, all 16 tokens
            if constexpr (FULL) {
                MmaTraits<T>::mma16(st.o[2 * dp], pa[0][0], pa[1][0], pa[0][1], pa[1][1], b[0], b[1]);
                MmaTraits<T>::mma16(st.o[2 * dp + 1], pa[0][0], pa[1][0], pa[0][1], pa[1][1], b[2], b[3]);
            } else {
                MmaTraits<T>::mma(st.o[2 * dp], pa[0][0], pa[0][1], b[0], b[1]);
                MmaTraits<T>::mma(st.o[2 * dp + 1], pa[0][0], pa[0][1], b[2], b[3]);
            }
        }
    }

    // finish the row sums, write this warp's rows
    __device__ __forceinline__ static void publish(State &st, float *red, int lane, int rows) {
        constexpr int PW = PartialRow<kD>::kWidth;
        const int qd = lane & 3;
#pragma unroll
        for (int half = 0; half < NR; ++half) {
            float l = st.l_part[half];
            l += __shfl_xor_sync(DA_FULL_MASK, l, 1);
            l += __shfl_xor_sync(DA_FULL_MASK, l, 2);
            const int r = (lane >> 2) + 8 * half;
            if (r < rows) {
#pragma unroll
                for (int d = 0; d < NT; ++d) {
                    red[r * PW + 8 * d + 2 * qd] = st.o[d][2 * half];
                    red[r * PW + 8 * d + 2 * qd + 1] = st.o[d][2 * half + 1];
                }
                if (qd == 0) {
                    red[r * PW + kD] = st.m_run[half];
                    red[r * PW + kD + 1] = l;
                }
            }
        }
    }
};

// WARPS per CTA, STAGES per warp, at least MINB CTAs per SM.
template <typename T, int D, bool FULL, int WARPS, int STAGES, int MINB>
__global__ void __launch_bounds__(WARPS * 32, MINB) decode_attention_mma_kernel(const AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    decode_attention_body<MmaMath<T, D, FULL>, WARPS, STAGES>(p, smem);
}

template <typename T, int D, bool FULL, int WARPS, int STAGES, int MINB>
static cudaError_t launch_mma_w(const AttnParams &p, int n_kv_heads, int splits, cudaStream_t stream) {
    using M = MmaMath<T, D, FULL>;
    constexpr int SMEM = WARPS * STAGES * M::STAGEB;
    auto kern = decode_attention_mma_kernel<T, D, FULL, WARPS, STAGES, MINB>;
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
    dim3 grid(splits, n_kv_heads);
    // phase 1 runs on a stream of its own beside the kernels of the step; the other launches follow
    // the LRU update in their stream and may move onto the SMs while it is still running
    if (p.phase != 1) return launch_dependent(kern, grid, dim3(WARPS * 32), (size_t)SMEM, stream, p);
    kern<<<grid, WARPS * 32, SMEM, stream>>>(p);
    return cudaGetLastError();
}

// Geometry.  The loop of a warp is a chain of dependent instructions (wait, ldmatrix, mma,
// softmax, issue), so an SM needs many warps to keep its copies flowing: 12 warps with two
// stages each (203 KB of stages per SM for head_dim 128).  The single launch and phase 2 use
// three 4-warp CTAs per SM; phase 1 one 12-warp CTA that fills its SM.
template <typename T, int D, bool FULL>
static cudaError_t launch_mma(const AttnParams &p, int n_kv_heads, int splits, cudaStream_t stream) {
    if (p.phase == 1) return launch_mma_w<T, D, FULL, kAttnPhase1Warps, 2, 1>(p, n_kv_heads, splits, stream);
    return launch_mma_w<T, D, FULL, kAttnWarps, 2, 3>(p, n_kv_heads, splits, stream);
}

template <typename T, int D>
static cudaError_t launch_mma_d(const AttnParams &p, int n_kv_heads, int splits, cudaStream_t stream) {
    if (p.n_q * p.rep > 8) return launch_mma<T, D, true>(p, n_kv_heads, splits, stream);
    return launch_mma<T, D, false>(p, n_kv_heads, splits, stream);
}

template <typename T>
static cudaError_t dispatch_mma(const AttnParams &p, int n_kv_heads, int head_dim, int splits, cudaStream_t s) {
    if (head_dim == 128) return launch_mma_d<T, 128>(p, n_kv_heads, splits, s);
    if (head_dim == 64) return launch_mma_d<T, 64>(p, n_kv_heads, splits, s);
    return cudaErrorInvalidValue;
}

cudaError_t launch_attention_mma(const AttnParams &p, int n_kv_heads, int head_dim, int dtype, int splits,
                                 cudaStream_t stream) {
    if (dtype == DA_BF16) return dispatch_mma<__nv_bfloat16>(p, n_kv_heads, head_dim, splits, stream);
    if (dtype == DA_F16) return dispatch_mma<__half>(p, n_kv_heads, head_dim, splits, stream);
    return cudaErrorInvalidValue;
}

}  // namespace da

DA_DEFINE_TRACE_SETTER(trace_set_attn_mma)

// Decode attention of one query token over the whole slot table plus the local
// window: split-K flash-decode with the append of the new key/value and the final
// merge in the same launch.
//
// Work unit = 16 consecutive tokens (8 KiB for head_dim 128 in 16-bit types).  A
// unit of the slot table is one contiguous block (token-major, key then value), so
// one untiled bulk copy (TMA) brings it into shared memory; a unit of the local
// window is gathered row by row with small bulk copies into the same layout.  Every
// warp owns a private ring of stages with one mbarrier each, so there is no
// CTA-wide synchronisation in the main loop.
//
// Arithmetic mapping: 8 lanes share a token (each owns D/8 channels, as two
// chunks that make conflict-free 128-bit shared-memory reads), 4 tokens per warp
// pass, all `rep` query heads of the KV head at once.  The dot products finish
// with a 3-step shuffle tree; softmax is online in the log2 domain with float32
// state; partial (m, l, acc) of the 4 token groups and the 4 warps are merged
// through shuffles and shared memory, written to the workspace, and the last CTA
// of a head (atomic ticket) merges the splits and writes the output.

#include "attn_common.cuh"

namespace da {

template <typename T, int D, int REP, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 4 ? 2 : 1) decode_attention_kernel(const AttnParams p) {
    constexpr int E = (int)sizeof(T);
    constexpr int ROWB = D * E;                 // one key (or value) row
    constexpr int TOKB = 2 * ROWB;              // one token: key row then value row
    constexpr int UNITB = kUnitTokens * TOKB;   // one stage
    constexpr int NPL = D / 8;                  // channels per lane
    constexpr int CH = NPL / 2;                 // channels per chunk
    constexpr int CHB = CH * E;                 // bytes per chunk
    constexpr int PW = PartialRow<D>::kWidth;   // floats per partial row: acc[D], m, l, pad
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
    const int g = lane >> 3;  // token group inside the warp
    const int j = lane & 7;   // channel block inside the token

    // ---- position and unit range ------------------------------------------------
    const int pos = p.start_pos_dev ? *p.start_pos_dev : p.start_pos_host;
    int t_new = pos - p.dram_tokens;  // index of the new token in the local window
    bool pos_ok = true;
    if (t_new < 0 || t_new >= p.local_capacity) {
        pos_ok = false;
        if (tid == 0 && x == 0) atomicOr(p.status, DA_STATUS_BAD_POSITION);
        t_new = t_new < 0 ? 0 : p.local_capacity - 1;
    }
    const int n_local = t_new + 1;
    const int n_prefix = p.n_prefix_tokens;
    // Units are dealt round-robin to the (CTA, warp) workers of this head, so every
    // worker sees the same mix of slot-table units (one bulk copy) and local-window
    // units (a row gather).
    const int n_workers = splits * WARPS;
    const int worker = x * WARPS + warp;
    const UnitPlan plan = plan_units(p, h, n_local, worker, n_workers, lane);
    const int units_prefix = plan.units_slots;   // units of this launch that come from the slot table
    const int n_my = plan.n_my;

    unsigned char *my_stages = smem + (size_t)warp * STAGES * UNITB;
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

    // ---- query rows of this KV head, pre-scaled by log2(e) / sqrt(D) ----------------
    float qr[REP][NPL];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        const unsigned char *qrow = p.q + ((size_t)(h * REP + r)) * ROWB;
        load_elems<T, CH>(qrow + j * CHB, &qr[r][0]);
        load_elems<T, CH>(qrow + ROWB / 2 + j * CHB, &qr[r][CH]);
#pragma unroll
        for (int i = 0; i < NPL; ++i) qr[r][i] *= p.scale_log2;
    }

    float m[REP], l[REP], acc[REP][NPL];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = NEG_INF;
        l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) acc[r][i] = 0.f;
    }

    // tokens of unit u
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

    // start the copies of unit u into stage s of this warp
    auto issue = [&](int s, int it) {
        const int idx = unit_index(it);
        const int u = worker + idx * n_workers;
        uint64_t *bar = &bars[warp][s];
        unsigned char *dst = my_stages + (size_t)s * UNITB;
        const int base = unit_base(u, idx);
        const int src_page = unit_src(idx);
        const int ntok = unit_tokens(u, base);
        if (u < units_prefix) {
            if (lane == 0) {
                const uint32_t bytes = (uint32_t)ntok * TOKB;
                mbar_arrive_expect_tx(bar, bytes);
                const size_t tok = (size_t)base;
                const unsigned char *src =
                    src_page < 0 ? p.prefix + ((size_t)h * p.prefix_head_stride + tok * 2 * D) * E
                                 : p.dram + ((size_t)h * p.dram_head_stride +
                                             ((size_t)src_page * p.page_tokens + tok % p.page_tokens) * 2 * D) * E;
                bulk_copy_g2s(dst, src, bytes, bar);
            }
        } else {
            const int t0 = (u - units_prefix) * kUnitTokens;
            if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)ntok * TOKB);
            __syncwarp();
            const int tl = lane & 15;
            const int is_v = lane >> 4;
            if (tl < ntok) {
                const int t = t0 + tl;
                const unsigned char *src;
                if (t == t_new) {
                    src = (is_v ? p.new_v : p.new_k) + (size_t)h * ROWB;
                } else {
                    src = (is_v ? p.local_v : p.local_k) +
                          ((size_t)t * p.local_tok_stride + (size_t)h * p.local_head_stride) * E;
                }
                bulk_copy_g2s(dst + tl * TOKB + is_v * ROWB, src, ROWB, bar);
            }
        }
    };

    for (int it = 0; it < STAGES && it < n_my; ++it) issue(it, it);

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
        const unsigned char *sb = my_stages + (size_t)s * UNITB;
        if (unit_src(idx) >= 0 && u < units_prefix) {
            // this unit came from DRAM: write it through to its slot
            uint4 *slot = reinterpret_cast<uint4 *>(
                const_cast<unsigned char *>(p.prefix) +
                ((size_t)h * p.prefix_head_stride + (size_t)base * 2 * D) * E);
            for (int i = lane; i < ntok * (TOKB / 16); i += 32) slot[i] = reinterpret_cast<const uint4 *>(sb)[i];
        }

        // logits (log2 domain) of 4 tokens x REP heads
        float sc[4][REP];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            const unsigned char *kp = sb + (g + 4 * tt) * TOKB;
            float kf[NPL];
            load_elems<T, CH>(kp + j * CHB, &kf[0]);
            load_elems<T, CH>(kp + ROWB / 2 + j * CHB, &kf[CH]);
#pragma unroll
            for (int r = 0; r < REP; ++r) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < NPL; ++i) a = fmaf(qr[r][i], kf[i], a);
                sc[tt][r] = a;
            }
        }
#pragma unroll
        for (int off = 1; off <= 4; off <<= 1)
#pragma unroll
            for (int tt = 0; tt < 4; ++tt)
#pragma unroll
                for (int r = 0; r < REP; ++r) sc[tt][r] += __shfl_xor_sync(DA_FULL_MASK, sc[tt][r], off);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)
            if (g + 4 * tt >= ntok) {
#pragma unroll
                for (int r = 0; r < REP; ++r) sc[tt][r] = NEG_INF;
            }

        // online softmax update
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            const float mx = fmaxf(fmaxf(sc[0][r], sc[1][r]), fmaxf(sc[2][r], sc[3][r]));
            const float mnew = fmaxf(m[r], mx);
            const float msafe = (mnew == NEG_INF) ? 0.f : mnew;
            const float alpha = fast_exp2(m[r] - msafe);
            float psum = 0.f;
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
                sc[tt][r] = fast_exp2(sc[tt][r] - msafe);
                psum += sc[tt][r];
            }
            l[r] = l[r] * alpha + psum;
            m[r] = mnew;
#pragma unroll
            for (int i = 0; i < NPL; ++i) acc[r][i] *= alpha;
        }

        // values
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            if (g + 4 * tt < ntok) {
                const unsigned char *vp = sb + (g + 4 * tt) * TOKB + ROWB;
                float vf[NPL];
                load_elems<T, CH>(vp + j * CHB, &vf[0]);
                load_elems<T, CH>(vp + ROWB / 2 + j * CHB, &vf[CH]);
#pragma unroll
                for (int r = 0; r < REP; ++r)
#pragma unroll
                    for (int i = 0; i < NPL; ++i) acc[r][i] = fmaf(sc[tt][r], vf[i], acc[r][i]);
            }
        }

        __syncwarp();
        if (it + STAGES < n_my) issue(s, it + STAGES);
    }

    // ---- merge the 4 token groups of the warp ---------------------------------------
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            const float mo = __shfl_xor_sync(DA_FULL_MASK, m[r], off);
            const float lo = __shfl_xor_sync(DA_FULL_MASK, l[r], off);
            const float mn = fmaxf(m[r], mo);
            const float ms = (mn == NEG_INF) ? 0.f : mn;
            const float a = fast_exp2(m[r] - ms);
            const float b = fast_exp2(mo - ms);
            l[r] = l[r] * a + lo * b;
            m[r] = mn;
#pragma unroll
            for (int i = 0; i < NPL; ++i) {
                const float ao = __shfl_xor_sync(DA_FULL_MASK, acc[r][i], off);
                acc[r][i] = acc[r][i] * a + ao * b;
            }
        }
    }
    if (g == 0) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                red[warp][r][j * CH + i] = acc[r][i];
                red[warp][r][D / 2 + j * CH + i] = acc[r][CH + i];
            }
            if (j == 0) {
                red[warp][r][D] = m[r];
                red[warp][r][D + 1] = l[r];
            }
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
        part[e] = outv;  // c < D: weighted acc; c == D: max; c == D+1: weighted l
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
static cudaError_t launch_attn_w(const AttnParams &p, int n_kv_heads, cudaStream_t stream) {

    constexpr int UNITB = kUnitTokens * 2 * D * (int)sizeof(T);
    constexpr int STAGES = UNITB >= 16384 ? 2 : (UNITB >= 8192 ? 3 : 4);
    constexpr int SMEM = WARPS * STAGES * UNITB;
    auto kern = decode_attention_kernel<T, D, REP, STAGES, WARPS>;
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
static cudaError_t launch_attn(const AttnParams &p, int n_kv_heads, cudaStream_t stream) {
    if (p.phase == 1) return launch_attn_w<T, D, REP, kAttnPhase1Warps>(p, n_kv_heads, stream);
    return launch_attn_w<T, D, REP, kAttnWarps>(p, n_kv_heads, stream);
}

template <typename T>
static cudaError_t dispatch_attn(const AttnParams &p, int n_kv_heads, int rep, int head_dim, cudaStream_t s) {
#define DA_ATTN_CASE(DD, RR) \
    if (head_dim == DD && rep == RR) return launch_attn<T, DD, RR>(p, n_kv_heads, s);
    DA_ATTN_CASE(128, 1) DA_ATTN_CASE(128, 2) DA_ATTN_CASE(128, 4) DA_ATTN_CASE(128, 8)
    DA_ATTN_CASE(64, 1) DA_ATTN_CASE(64, 2) DA_ATTN_CASE(64, 4) DA_ATTN_CASE(64, 8)
#undef DA_ATTN_CASE
    return cudaErrorInvalidValue;
}

}  // namespace da

extern "C" size_t da_decode_attention_workspace_bytes(int n_kv_heads, int rep, int head_dim) {
    if (n_kv_heads < 1 || rep < 1 || head_dim < 1) return 0;
    return (size_t)da::kCounterBytes +
           (size_t)n_kv_heads * da::attn_splits(n_kv_heads) * rep * (head_dim + 4) * sizeof(float);
}

extern "C" size_t da_decode_attention_phased_workspace_bytes(int n_kv_heads, int rep, int head_dim);

static int decode_attention_common(const void *q, const void *prefix_kv, long long prefix_head_stride,
                                   int n_prefix_tokens, void *local_k, void *local_v,
                                   long long local_token_stride, long long local_head_stride,
                                   int local_capacity, const void *new_k, const void *new_v,
                                   const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                   void *out, float *lse_out, void *workspace, size_t workspace_bytes,
                                   int32_t *status, int n_kv_heads, int rep, int head_dim, int dtype,
                                   const void *dram_pages, int n_dram_pages, const int32_t *slot_source,
                                   int n_slots, int page_size, int phase, const int32_t *order, const int32_t *n_evictable,
                                   int32_t *flip, da_stream_t stream) {
    if (!q || !prefix_kv || !local_k || !local_v || !new_k || !new_v || !out || !workspace || !status)
        return DA_ERR_NULL;
    if (n_kv_heads < 1 || n_prefix_tokens < 1 || local_capacity < 1 || dram_tokens < 0) return DA_ERR_SHAPE;
    if (head_dim != 64 && head_dim != 128) return DA_ERR_UNSUPPORTED;
    if (rep != 1 && rep != 2 && rep != 4 && rep != 8) return DA_ERR_UNSUPPORTED;
    if (n_kv_heads * 4 > da::kCounterBytes || n_kv_heads > 65535) return DA_ERR_UNSUPPORTED;
    if (dtype != DA_F32 && dtype != DA_F16 && dtype != DA_BF16) return DA_ERR_DTYPE;
    const size_t esz = dtype == DA_F32 ? 4 : 2;
    const uintptr_t ptrs = (uintptr_t)q | (uintptr_t)prefix_kv | (uintptr_t)local_k | (uintptr_t)local_v |
                           (uintptr_t)new_k | (uintptr_t)new_v | (uintptr_t)out;
    if ((ptrs & 15) || ((uintptr_t)workspace & 255)) return DA_ERR_ALIGN;
    if (((size_t)prefix_head_stride * esz) % 16 || ((size_t)local_token_stride * esz) % 16 ||
        ((size_t)local_head_stride * esz) % 16)
        return DA_ERR_ALIGN;
    if (phase < 0 || phase > 2) return DA_ERR_SHAPE;
    const size_t ws_need = phase == 0 ? da_decode_attention_workspace_bytes(n_kv_heads, rep, head_dim)
                                      : da_decode_attention_phased_workspace_bytes(n_kv_heads, rep, head_dim);
    if (workspace_bytes < ws_need) return DA_ERR_WORKSPACE;

    da::AttnParams p{};
    p.q = static_cast<const unsigned char *>(q);
    p.prefix = static_cast<const unsigned char *>(prefix_kv);
    p.prefix_head_stride = prefix_head_stride;
    p.n_prefix_tokens = n_prefix_tokens;
    p.local_k = static_cast<unsigned char *>(local_k);
    p.local_v = static_cast<unsigned char *>(local_v);
    p.local_tok_stride = local_token_stride;
    p.local_head_stride = local_head_stride;
    p.local_capacity = local_capacity;
    p.new_k = static_cast<const unsigned char *>(new_k);
    p.new_v = static_cast<const unsigned char *>(new_v);
    p.start_pos_dev = start_pos_dev;
    p.start_pos_host = start_pos_host;
    p.dram_tokens = dram_tokens;
    p.out = static_cast<unsigned char *>(out);
    p.lse_out = lse_out;
    p.counters = static_cast<unsigned int *>(workspace);
    p.partials = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + da::kCounterBytes);
    p.status = status;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)head_dim);
    if (slot_source) {
        // units (16 tokens) must not straddle pages, the slot table must be exactly the prefix,
        // and a warp keeps the sources of its units in its 32 lanes
        if (!dram_pages) return DA_ERR_NULL;
        if (page_size < 1 || n_slots < 1 || n_dram_pages < 1) return DA_ERR_SHAPE;
        if (page_size % da::kUnitTokens != 0 || (long long)n_slots * page_size != n_prefix_tokens)
            return DA_ERR_UNSUPPORTED;
        if ((uintptr_t)dram_pages & 15) return DA_ERR_ALIGN;
        const int units_max = (n_prefix_tokens + da::kUnitTokens - 1) / da::kUnitTokens +
                              (local_capacity + da::kUnitTokens - 1) / da::kUnitTokens;
        const int workers = phase == 1 ? da::attn_splits_phase1(n_kv_heads) * da::kAttnPhase1Warps
                                       : da::attn_splits(n_kv_heads) * da::kAttnWarps;
        if ((units_max + workers - 1) / workers > da::kMaxUnitsPerWarp) return DA_ERR_UNSUPPORTED;
        p.dram = static_cast<const unsigned char *>(dram_pages);
        p.dram_head_stride = (long long)n_dram_pages * page_size * 2 * head_dim;
        p.slot_source = slot_source;
        p.n_slots = n_slots;
        p.page_tokens = page_size;
    }
    p.phase = phase;
    p.n_kv_heads = n_kv_heads;
    p.counters1 = p.counters + da::kCounterBytes / 8;
    p.part_rows = da::attn_splits(n_kv_heads);
    p.part_offset = 0;
    p.merge_first = 0;
    p.merge_rows = p.part_rows;
    if (phase != 0) {
        if (!slot_source || !order || !n_evictable || !flip) return DA_ERR_NULL;
        if (n_kv_heads * 8 > da::kCounterBytes) return DA_ERR_UNSUPPORTED;
        const int sa = da::attn_splits_phase1(n_kv_heads), sb = da::attn_splits(n_kv_heads);
        p.order = order;
        p.n_evictable = n_evictable;
        p.flip = flip;
        p.part_rows = sa + sb;                // phase-1 rows, then phase-2 rows
        p.part_offset = phase == 2 ? sa : 0;
        p.merge_first = 0;
        p.merge_rows = sa + sb;
    }

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == DA_F32) e = da::dispatch_attn<float>(p, n_kv_heads, rep, head_dim, s);
    else e = da::launch_attention_mma(p, n_kv_heads, rep, head_dim, dtype, s);
    return (int)e;
}

extern "C" int da_decode_attention(const void *q, const void *prefix_kv, long long prefix_head_stride,
                                   int n_prefix_tokens, void *local_k, void *local_v,
                                   long long local_token_stride, long long local_head_stride,
                                   int local_capacity, const void *new_k, const void *new_v,
                                   const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                   void *out, float *lse_out, void *workspace, size_t workspace_bytes,
                                   int32_t *status, int n_kv_heads, int rep, int head_dim, int dtype,
                                   da_stream_t stream) {
    return decode_attention_common(q, prefix_kv, prefix_head_stride, n_prefix_tokens, local_k, local_v,
                                   local_token_stride, local_head_stride, local_capacity, new_k, new_v,
                                   start_pos_dev, start_pos_host, dram_tokens, out, lse_out, workspace,
                                   workspace_bytes, status, n_kv_heads, rep, head_dim, dtype, nullptr, 0,
                                   nullptr, 0, 0, 0, nullptr, nullptr, nullptr, stream);
}

extern "C" int da_decode_attention_fetch(const void *q, void *slots, long long slots_head_stride, int n_slots,
                                         int page_size, const void *dram_pages, int n_dram_pages,
                                         const int32_t *slot_source, void *local_k, void *local_v,
                                         long long local_token_stride, long long local_head_stride,
                                         int local_capacity, const void *new_k, const void *new_v,
                                         const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                         void *out, float *lse_out, void *workspace, size_t workspace_bytes,
                                         int32_t *status, int n_kv_heads, int rep, int head_dim, int dtype,
                                         da_stream_t stream) {
    if (!slot_source) return DA_ERR_NULL;
    if (n_slots < 1 || page_size < 1 || (long long)n_slots * page_size > 0x7fffffffLL) return DA_ERR_SHAPE;
    return decode_attention_common(q, slots, slots_head_stride, n_slots * page_size, local_k, local_v,
                                   local_token_stride, local_head_stride, local_capacity, new_k, new_v,
                                   start_pos_dev, start_pos_host, dram_tokens, out, lse_out, workspace,
                                   workspace_bytes, status, n_kv_heads, rep, head_dim, dtype, dram_pages,
                                   n_dram_pages, slot_source, n_slots, page_size, 0, nullptr, nullptr, nullptr, stream);
}

extern "C" int da_decode_attention_phased_supported(int n_kv_heads, int rep, int head_dim, int dtype, int n_slots,
                                                    int page_size, int local_capacity) {
    if (n_kv_heads < 1 || n_slots < 1 || page_size < 1 || local_capacity < 1) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    if (rep != 1 && rep != 2 && rep != 4 && rep != 8) return 0;
    if (dtype != DA_F32 && dtype != DA_F16 && dtype != DA_BF16) return 0;
    if (page_size % da::kUnitTokens != 0 || (long long)n_slots * page_size > 0x7fffffffLL) return 0;
    const int units = n_slots * (page_size / da::kUnitTokens) +
                      (local_capacity + da::kUnitTokens - 1) / da::kUnitTokens;
    const int w1 = da::attn_splits_phase1(n_kv_heads) * da::kAttnPhase1Warps;
    const int w2 = da::attn_splits(n_kv_heads) * da::kAttnWarps;
    if ((units + w1 - 1) / w1 > da::kMaxUnitsPerWarp || (units + w2 - 1) / w2 > da::kMaxUnitsPerWarp) return 0;
    // shared memory of a phase-1 CTA: 8 warps x stages x stage bytes + the warp-merge scratch
    const size_t esz = dtype == DA_F32 ? 4 : 2;
    size_t stage = (size_t)da::kUnitTokens * (2 * head_dim * esz + (esz == 2 ? 16 : 0));
    const int stages = esz == 2 ? (stage > 8192 ? 3 : 4) : (stage >= 16384 ? 2 : (stage >= 8192 ? 3 : 4));
    const size_t smem = (size_t)da::kAttnPhase1Warps * stages * stage +
                        (size_t)da::kAttnPhase1Warps * rep * (head_dim + 4) * sizeof(float) + 2048;
    return smem <= 227 * 1024 ? 1 : 0;
}

extern "C" size_t da_decode_attention_phased_workspace_bytes(int n_kv_heads, int rep, int head_dim) {
    if (n_kv_heads < 1 || rep < 1 || head_dim < 1) return 0;
    return (size_t)da::kCounterBytes + (size_t)n_kv_heads *
                                           (da::attn_splits_phase1(n_kv_heads) + da::attn_splits(n_kv_heads)) * rep *
                                           (head_dim + 4) * sizeof(float);
}

extern "C" int da_decode_attention_phased(int phase, const int32_t *order, const int32_t *n_evictable,
                                          int32_t *split_flip, const void *q, void *slots, long long slots_head_stride, int n_slots,
                                          int page_size, const void *dram_pages, int n_dram_pages,
                                          const int32_t *slot_source, void *local_k, void *local_v,
                                          long long local_token_stride, long long local_head_stride,
                                          int local_capacity, const void *new_k, const void *new_v,
                                          const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                          void *out, float *lse_out, void *workspace, size_t workspace_bytes,
                                          int32_t *status, int n_kv_heads, int rep, int head_dim, int dtype,
                                          da_stream_t stream) {
    if (phase != 1 && phase != 2) return DA_ERR_SHAPE;
    if (!slot_source || !order || !n_evictable || !split_flip) return DA_ERR_NULL;
    if (!da_decode_attention_phased_supported(n_kv_heads, rep, head_dim, dtype, n_slots, page_size, local_capacity))
        return DA_ERR_UNSUPPORTED;
    if (n_slots < 1 || page_size < 1 || (long long)n_slots * page_size > 0x7fffffffLL) return DA_ERR_SHAPE;
    return decode_attention_common(q, slots, slots_head_stride, n_slots * page_size, local_k, local_v,
                                   local_token_stride, local_head_stride, local_capacity, new_k, new_v,
                                   start_pos_dev, start_pos_host, dram_tokens, out, lse_out, workspace,
                                   workspace_bytes, status, n_kv_heads, rep, head_dim, dtype, dram_pages,
                                   n_dram_pages, slot_source, n_slots, page_size, phase, order, n_evictable,
                                   split_flip, stream);
}

// ---- entry point with built-in scratch ------------------------------------------------

namespace da {
// Scratch for da_decode_attention_static: the same layout da_decode_attention expects in
// its workspace (ticket counters, then the per-CTA partials).  2 MiB covers every shape
// the kernels accept with head_dim <= 128 and rep <= 8 (the largest needs about 1.2 MiB).
// The array is part of the loaded module: every GPU that loads this library keeps it
// until the process exits, and it starts out zero-filled.
constexpr size_t kStaticScratchBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
}  // namespace da

extern "C" size_t da_decode_attention_static_capacity(void) { return da::kStaticScratchBytes; }

extern "C" int da_decode_attention_static(const void *q, const void *prefix_kv, long long prefix_head_stride,
                                          int n_prefix_tokens, void *local_k, void *local_v,
                                          long long local_token_stride, long long local_head_stride,
                                          int local_capacity, const void *new_k, const void *new_v,
                                          const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                          void *out, float *lse_out, int32_t *status, int n_kv_heads, int rep,
                                          int head_dim, int dtype, da_stream_t stream) {
    if (n_kv_heads < 1 || rep < 1 || head_dim < 1) return DA_ERR_SHAPE;
    const size_t need = da_decode_attention_workspace_bytes(n_kv_heads, rep, head_dim);
    if (need > da::kStaticScratchBytes) return DA_ERR_STATIC_SCRATCH;

    // In host code the array's name is only a handle for the runtime, not a device
    // address: ask the runtime for the address once per device, with that device
    // current (it is: the caller's stream belongs to it), and hand that to the kernel.
    static void *scratch_of_device[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DA_ERR_UNSUPPORTED;
    if (scratch_of_device[dev] == nullptr) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, da::g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        scratch_of_device[dev] = ptr;
    }
    void *scratch = scratch_of_device[dev];

    // All calls share the array and it keeps what the last call left.  The kernel only
    // needs the ticket counters to be zero on entry; clear them on the caller's stream
    // (a call that was cut short could have left them half counted).
    e = cudaMemsetAsync(scratch, 0, da::kCounterBytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return (int)e;
    return da_decode_attention(q, prefix_kv, prefix_head_stride, n_prefix_tokens, local_k, local_v,
                               local_token_stride, local_head_stride, local_capacity, new_k, new_v,
                               start_pos_dev, start_pos_host, dram_tokens, out, lse_out, scratch,
                               da::kStaticScratchBytes, status, n_kv_heads, rep, head_dim, dtype, stream);
}

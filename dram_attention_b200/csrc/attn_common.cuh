// Pieces shared by the decode-attention kernels (float32 on CUDA cores, 16-bit
// types on tensor cores): launch geometry, the parameter block, the unit plan and
// the final merge of the per-CTA partials.
#pragma once

#include "da_common.cuh"

namespace da {

constexpr int kAttnWarps = 4;          // warps per CTA of the single launch and of phase 2
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kUnitTokens = 16;
constexpr int kCounterBytes = 1024;
constexpr int kAttnTargetCtas = 296;   // 2 per SM on 148 SMs
constexpr int kAttnMaxSplits = 148;
constexpr int kAttnMaxRows = 16;       // query rows (tokens x GQA group) of one KV head per launch
constexpr int kRoundUnits = 64;        // units a warp plans at a time (two per lane)

// Phase 1 runs beside the selection kernels, whose CTAs need a whole SM each.  Its CTAs are
// therefore built to fill an SM on their own (8 warps, twice the shared memory), and by default
// there are at most 116 of them: wherever the hardware places them, 32 of the 148 SMs stay empty.
// Phase 2 normally covers only the few slots the LRU update could evict; 64 CTAs (two per SM on
// those 32 SMs) are plenty.
constexpr int kAttnPhase1Warps = 8;
constexpr int kAttnPhase1Ctas = 116;
constexpr int kAttnPhase2Ctas = 64;

__host__ __device__ inline int attn_splits(int n_kv_heads) {
    int s = kAttnTargetCtas / n_kv_heads;
    if (s > kAttnMaxSplits) s = kAttnMaxSplits;
    if (s < 1) s = 1;
    return s;
}

__host__ __device__ inline int attn_splits_phase1(int n_kv_heads) {
    int s = kAttnPhase1Ctas / n_kv_heads;
    if (s < 1) s = 1;
    return s;
}

__host__ __device__ inline int attn_splits_phase2(int n_kv_heads) {
    int s = kAttnPhase2Ctas / n_kv_heads;
    if (s < 1) s = 1;
    return s;
}

struct AttnParams {
    const unsigned char *q;        // (s_total, n_kv_heads * rep, D)
    const unsigned char *prefix;
    long long prefix_head_stride;  // elements
    int n_prefix_tokens;
    unsigned char *local_k, *local_v;
    long long local_tok_stride, local_head_stride;  // elements
    int local_capacity;
    const unsigned char *new_k, *new_v;   // (s_total, n_kv_heads, D)
    const int32_t *start_pos_dev;
    int start_pos_host;
    int dram_tokens;
    unsigned char *out;            // (s_total, n_kv_heads * rep, D)
    float *lse_out;                // (s_total, n_kv_heads * rep) or null
    float *partials;
    unsigned int *counters;
    int32_t *status;
    float scale_log2;
    // optional: pages that da_lru_update just assigned to slots are read from DRAM (pinned
    // host memory) by the warp that owns the unit, and written through to the slot
    const unsigned char *dram;       // (n_kv_heads, n_dram_pages, page_tokens, 2, D) or null
    long long dram_head_stride;      // elements
    const int32_t *slot_source;      // (n_kv_heads, n_slots): DRAM page to read instead, or -1
    int n_slots;
    int page_tokens;                 // multiple of 16 when slot_source is set
    // optional: two launches per step.  Phase 1 attends over the local window and the slots
    // outside the eviction front (it runs beside selection and LRU update); phase 2 attends over
    // the front after the update; the CTA of either launch that finishes last merges both.  The
    // front is order[h][0 .. n_evictable[h]) of the copy flip[h] names.  redo[h] != 0 (set by the
    // LRU update when it had to evict a slot outside the front): phase 2 covers the whole head
    // and the merge leaves out the rows of phase 1.
    int phase;                       // 0: one launch over everything
    const int32_t *order;            // [2][n_kv_heads][n_slots]
    const int32_t *n_evictable;      // [2][n_kv_heads]
    int32_t *flip;                   // [n_kv_heads]
    const int32_t *redo;             // [n_kv_heads]
    int part_rows;                   // partial rows (CTAs) per head in the workspace
    int part_offset;                 // first row this launch writes
    int ticket_target;               // CTAs of a head that take a ticket before the merge
    int splits1;                     // rows of phase 1 (first in the workspace)
    int n_kv_heads;
    int rep;
    // query tokens: the call has s_total of them (appended at consecutive positions); this
    // launch computes tokens [q_tok0, q_tok0 + n_q), i.e. n_q * rep query rows per KV head
    int s_total, q_tok0, n_q;
};

// Units of a head this launch covers.
struct LaunchUnits {
    int units_slots;      // units from the slot table
    int units_local;      // units from the local window
    const int32_t *order; // slot order to walk (null: slot-table tokens in place)
    int order_off;        // first entry of `order` that belongs to this launch
    int ups;              // units per slot page
};

__device__ __forceinline__ LaunchUnits launch_units(const AttnParams &p, int h, int n_local) {
    LaunchUnits lu;
    lu.order = nullptr;
    lu.order_off = 0;
    lu.ups = p.phase != 0 ? p.page_tokens / kUnitTokens : 1;
    bool local = true;
    if (p.phase == 0) {
        lu.units_slots = (p.n_prefix_tokens + kUnitTokens - 1) / kUnitTokens;
    } else {
        const int cur = p.flip[h] & 1;
        const int32_t *order = p.order + ((size_t)cur * p.n_kv_heads + h) * p.n_slots;
        const int n_ev = min(max(p.n_evictable[cur * p.n_kv_heads + h], 0), p.n_slots);
        if (p.phase == 1) {
            lu.units_slots = (p.n_slots - n_ev) * lu.ups;
            lu.order = order;
            lu.order_off = n_ev;
        } else if (p.redo[h] != 0) {
            lu.units_slots = p.n_slots * lu.ups;   // the whole head, slots in place
        } else {
            lu.units_slots = n_ev * lu.ups;
            lu.order = order;
            local = false;
        }
    }
    lu.units_local = local ? (n_local + kUnitTokens - 1) / kUnitTokens : 0;
    return lu;
}

// Where each unit of one round of a warp comes from (two per lane).
struct UnitPlan {
    int n_round;       // units of this round: positions round * 64 .. round * 64 + n_round - 1 of the warp
    int base[2];       // lane i: first token (inside the head's slot table) of unit i and 32 + i, or -1
    int src[2];        // lane i: DRAM page to read that unit from instead, or -1
};

__device__ __forceinline__ UnitPlan plan_round(const AttnParams &p, const LaunchUnits &lu, int h, int worker,
                                               int n_workers, int lane, int round, int total_my) {
    UnitPlan pl;
    pl.n_round = min(kRoundUnits, total_my - round * kRoundUnits);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        pl.base[k] = -1;
        pl.src[k] = -1;
        const int i = 32 * k + lane;
        const int u = worker + (round * kRoundUnits + i) * n_workers;
        if (i < pl.n_round && u < lu.units_slots) {
            int base = u * kUnitTokens;
            if (lu.order) {
                int slot = lu.order[lu.order_off + u / lu.ups];
                slot = min(max(slot, 0), p.n_slots - 1);
                base = slot * p.page_tokens + (u % lu.ups) * kUnitTokens;
            }
            pl.base[k] = base;
            if (p.slot_source && p.phase != 1)
                pl.src[k] = p.slot_source[(size_t)h * p.n_slots + base / p.page_tokens];
        }
    }
    return pl;
}

// Order in which a warp walks the units of a round: the ones that have to come from DRAM first,
// so that their host-link latency overlaps everything else the warp does.  perm = position ->
// unit index (two per lane, like the plan); `scratch` is 64 bytes of shared memory of this warp.
__device__ __forceinline__ void plan_order(const UnitPlan &pl, int lane, int (&perm)[2], unsigned char *scratch) {
    const unsigned lt = (1u << lane) - 1;
    const unsigned f0 = __ballot_sync(DA_FULL_MASK, pl.src[0] >= 0);
    const unsigned f1 = __ballot_sync(DA_FULL_MASK, pl.src[1] >= 0);
    const int nf = __popc(f0) + __popc(f1);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = 32 * k + lane;
        if (i < pl.n_round) {
            const int fresh_before = k == 0 ? __popc(f0 & lt) : __popc(f0) + __popc(f1 & lt);
            const bool fresh = pl.src[k] >= 0;
            scratch[fresh ? fresh_before : nf + (i - fresh_before)] = (unsigned char)i;
        }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 2; ++k) perm[k] = (32 * k + lane < pl.n_round) ? scratch[32 * k + lane] : 0;
    __syncwarp();
}

// value of lane (it % 32)'s entry (it / 32) of a two-deep per-lane table
__device__ __forceinline__ int plan_lookup(const int (&tab)[2], int it) {
    const int v0 = __shfl_sync(DA_FULL_MASK, tab[0], it & 31);
    const int v1 = __shfl_sync(DA_FULL_MASK, tab[1], it & 31);
    return (it & 32) ? v1 : v0;
}


// Floats per partial row: acc[D], max, l, padded to a multiple of 4 so that rows can
// be read with 128-bit loads.
template <int D> struct PartialRow { static constexpr int kWidth = D + 4; };

// Final merge of the per-CTA partials of one head by one CTA of THREADS threads.  A CTA's
// partial = `rows` rows of (acc[D] already weighted to the row's max, max, l).  `scratch` holds
// at least 2 * splits * rows floats of shared memory (the idle stage buffers).  Loads bypass L1
// (the rows were written by other SMs).  The first batch of accumulator rows is requested
// together with the (max, l) pairs.
template <typename T, int D, int THREADS>
__device__ __forceinline__ void merge_splits(const AttnParams &p, int h, int first_row, int splits, int rows,
                                             float *scratch) {
    constexpr int PW = PartialRow<D>::kWidth;
    constexpr int VPR = D / 4;          // float4 per accumulator row
    constexpr int BATCH = 40;
    constexpr float NEG_INF = -INFINITY;
    __shared__ float sh_m[kAttnMaxRows], sh_l[kAttnMaxRows];
    const int tid = threadIdx.x;
    const float *hp = p.partials + ((size_t)(h * p.part_rows + first_row) * rows) * PW;
    const int n = splits * rows;
    const int RS = rows * PW / 4;  // float4 stride between the partials of two CTAs
    float *wgt = scratch;        // [n] max, then weight
    float *lsum = scratch + n;   // [n] l of every partial row

    for (int e0 = 0; e0 < rows * VPR; e0 += THREADS) {
        const int e = e0 + tid;
        const bool live = e < rows * VPR;
        const int r = live ? e / VPR : 0;
        const int c4 = live ? e % VPR : 0;
        const float4 *col = reinterpret_cast<const float4 *>(hp + (size_t)r * PW) + c4;
        float4 v[BATCH];
        // first batch of accumulator loads goes out before anything is waited on
#pragma unroll
        for (int u = 0; u < BATCH; ++u)
            if (u < splits) v[u] = __ldcg(col + (size_t)u * RS);
        if (e0 == 0) {
            for (int i = tid; i < n; i += THREADS) {
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(hp + (size_t)i * PW + D));
                wgt[i] = ml.x;
                lsum[i] = ml.y;
            }
            __syncthreads();
            // one warp per query row: common max, weights exp2(max_s - max), weighted row sum
            const int lane = tid & 31;
            for (int rr = tid >> 5; rr < rows; rr += THREADS / 32) {
                float mn = NEG_INF;
                for (int s = lane; s < splits; s += 32) mn = fmaxf(mn, wgt[s * rows + rr]);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) mn = fmaxf(mn, __shfl_xor_sync(DA_FULL_MASK, mn, off));
                const float ms = (mn == NEG_INF) ? 0.f : mn;
                float ll = 0.f;
                for (int s = lane; s < splits; s += 32) {
                    const float w = fast_exp2(wgt[s * rows + rr] - ms);
                    wgt[s * rows + rr] = w;
                    ll = fmaf(lsum[s * rows + rr], w, ll);
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) ll += __shfl_xor_sync(DA_FULL_MASK, ll, off);
                if (lane == 0) {
                    sh_m[rr] = ms;
                    sh_l[rr] = ll;
                }
            }
            __syncthreads();
        }
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < splits; s0 += BATCH) {
            if (s0 > 0) {
#pragma unroll
                for (int u = 0; u < BATCH; ++u)
                    if (s0 + u < splits) v[u] = __ldcg(col + (size_t)(s0 + u) * RS);
            }
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                if (s0 + u < splits) {
                    const float w = wgt[(s0 + u) * rows + r];
                    a.x = fmaf(v[u].x, w, a.x);
                    a.y = fmaf(v[u].y, w, a.y);
                    a.z = fmaf(v[u].z, w, a.z);
                    a.w = fmaf(v[u].w, w, a.w);
                }
            }
        }
        if (live) {
            const float ll = sh_l[r];
            const float inv = ll > 0.f ? 1.f / ll : 0.f;
            // row r = (query token, head of the group)
            const int tok = p.q_tok0 + r / p.rep;
            const size_t orow = (size_t)tok * p.n_kv_heads * p.rep + (size_t)h * p.rep + r % p.rep;
            T *dst = reinterpret_cast<T *>(p.out) + orow * D + 4 * c4;
            dst[0] = from_float<T>(a.x * inv);
            dst[1] = from_float<T>(a.y * inv);
            dst[2] = from_float<T>(a.z * inv);
            dst[3] = from_float<T>(a.w * inv);
            if (c4 == 0 && p.lse_out) p.lse_out[orow] = (sh_m[r] + log2f(ll)) * 0.6931471805599453f;
        }
    }
}

// 16-bit element types: tensor-core kernel (attn_mma.cu).
cudaError_t launch_attention_mma(const AttnParams &p, int n_kv_heads, int head_dim, int dtype, int splits,
                                 cudaStream_t stream);

}  // namespace da

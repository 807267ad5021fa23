// Pieces shared by the two decode-attention kernels (float32 on CUDA cores,
// 16-bit types on tensor cores): launch geometry, the parameter block, and the
// final merge of the per-CTA partials.
#pragma once

#include "da_common.cuh"

namespace da {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kUnitTokens = 16;
constexpr int kCounterBytes = 1024;
constexpr int kAttnTargetCtas = 296;  // 2 per SM on 148 SMs
constexpr int kAttnMaxSplits = 148;

__host__ __device__ inline int attn_splits(int n_kv_heads) {
    int s = kAttnTargetCtas / n_kv_heads;
    if (s > kAttnMaxSplits) s = kAttnMaxSplits;
    if (s < 1) s = 1;
    return s;
}

struct AttnParams {
    const unsigned char *q;
    const unsigned char *prefix;
    long long prefix_head_stride;  // elements
    int n_prefix_tokens;
    unsigned char *local_k, *local_v;
    long long local_tok_stride, local_head_stride;  // elements
    int local_capacity;
    const unsigned char *new_k, *new_v;
    const int32_t *start_pos_dev;
    int start_pos_host;
    int dram_tokens;
    unsigned char *out;
    float *lse_out;
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
    // optional: two launches per step.  phase 1 attends over the local window and the slots
    // that the coming LRU update cannot evict (it runs beside selection and LRU update);
    // phase 2 attends over the evictable slots after the update and merges both.  The split
    // is order[h][0 .. n_evictable[h]) = evictable, the rest not (left by da_lru_update).
    int phase;                       // 0: one launch over everything
    const int32_t *order;            // [2][n_kv_heads][n_slots]: two copies of the split; flip[h] names the
    const int32_t *n_evictable;      // [2][n_kv_heads]            one both phases of this step use, the LRU
    int32_t *flip;                   // [n_kv_heads]               update writes the other, phase 2 flips
    unsigned int *counters1;         // ticket counters of phase 1 (second half of the counter block)
    int part_rows;                   // partial rows per head in the workspace
    int part_offset;                 // first row this launch writes
    int merge_first, merge_rows;     // rows the last CTA of a head merges
    int n_kv_heads;
};

constexpr int kMaxUnitsPerWarp = 64;   // two per lane: where each unit of a warp comes from
// Phase 1 runs beside the selection kernels, whose CTAs need a whole SM each.  Its CTAs are
// therefore built to fill an SM on their own (8 warps, twice the shared memory), and there
// are at most 116 of them: wherever the hardware places them, 32 of the 148 SMs stay empty.
constexpr int kAttnPhase1Warps = 8;
constexpr int kAttnPhase1Ctas = 116;

__host__ __device__ inline int attn_splits_phase1(int n_kv_heads) {
    int s = kAttnPhase1Ctas / n_kv_heads;
    if (s < 1) s = 1;
    return s;
}

// Which units a launch covers and where each of this warp's units comes from.
struct UnitPlan {
    int units_slots;   // units from the slot table in this launch
    int units_local;   // units from the local window in this launch
    int n_my;          // units of this warp: worker, worker + n_workers, ...
    int base[2];       // lane i: first token (inside the head's slot table) of unit i and 32 + i
    int src[2];        // lane i: DRAM page to read that unit from instead, or -1
};

__device__ __forceinline__ UnitPlan plan_units(const AttnParams &p, int h, int n_local, int worker,
                                               int n_workers, int lane) {
    UnitPlan pl;
    const int ups = p.order ? p.page_tokens / kUnitTokens : 1;
    int n_ev = 0;
    const int32_t *order = nullptr;
    if (p.order) {
        const int cur = p.flip[h] & 1;
        order = p.order + ((size_t)cur * p.n_kv_heads + h) * p.n_slots;
        n_ev = min(max(p.n_evictable[cur * p.n_kv_heads + h], 0), p.n_slots);
    }
    if (p.phase == 0) pl.units_slots = (p.n_prefix_tokens + kUnitTokens - 1) / kUnitTokens;
    else if (p.phase == 1) pl.units_slots = (p.n_slots - n_ev) * ups;
    else pl.units_slots = n_ev * ups;
    pl.units_local = p.phase == 2 ? 0 : (n_local + kUnitTokens - 1) / kUnitTokens;
    const int units = pl.units_slots + pl.units_local;
    pl.n_my = units > worker ? (units - worker + n_workers - 1) / n_workers : 0;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        pl.base[k] = -1;
        pl.src[k] = -1;
        const int i = 32 * k + lane;
        const int u = worker + i * n_workers;
        if (i < pl.n_my && u < pl.units_slots) {
            int base = u * kUnitTokens;
            if (p.phase != 0) {
                int slot = order[(p.phase == 1 ? n_ev : 0) + u / ups];
                slot = min(max(slot, 0), p.n_slots - 1);
                base = slot * p.page_tokens + (u % ups) * kUnitTokens;
            }
            pl.base[k] = base;
            if (p.slot_source && p.phase != 1)
                pl.src[k] = p.slot_source[(size_t)h * p.n_slots + base / p.page_tokens];
        }
    }
    return pl;
}

// Order in which a warp walks its units: the ones that have to come from DRAM first, so that
// their host-link latency overlaps everything else the warp does.  perm = position -> unit
// index (two per lane, like the plan); `scratch` is 64 bytes of shared memory of this warp.
__device__ __forceinline__ void plan_order(const UnitPlan &pl, int lane, int (&perm)[2], unsigned char *scratch) {
    const unsigned lt = (1u << lane) - 1;
    const unsigned f0 = __ballot_sync(DA_FULL_MASK, pl.src[0] >= 0);
    const unsigned f1 = __ballot_sync(DA_FULL_MASK, pl.src[1] >= 0);
    const int nf = __popc(f0) + __popc(f1);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = 32 * k + lane;
        if (i < pl.n_my) {
            const int fresh_before = k == 0 ? __popc(f0 & lt) : __popc(f0) + __popc(f1 & lt);
            const bool fresh = pl.src[k] >= 0;
            scratch[fresh ? fresh_before : nf + (i - fresh_before)] = (unsigned char)i;
        }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 2; ++k) perm[k] = (32 * k + lane < pl.n_my) ? scratch[32 * k + lane] : 0;
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

// Final merge of the per-CTA partials of one head by one CTA of THREADS threads.
// partial row = acc[D] (already weighted to the row's max), max, l.  `scratch` holds
// at least 2 * splits * REP floats of shared memory (the idle stage buffers).  Loads bypass L1 (the rows were
// written by other SMs).  The first batch of accumulator rows is requested together
// with the (max, l) pairs; up to 52 rows make a batch (the accumulators of the main loop are dead by then).  With `partial_out` the result is
// written as one more partial row instead of the output (phase 1 folds its rows this way).
template <typename T, int D, int REP, int THREADS>
__device__ __forceinline__ void merge_splits(const AttnParams &p, int h, int first_row, int splits, float *scratch,
                                             float *partial_out) {
    constexpr int PW = PartialRow<D>::kWidth;
    constexpr int VPR = D / 4;          // float4 per accumulator row
    constexpr int BATCH = 52;
    constexpr float NEG_INF = -INFINITY;
    __shared__ float sh_m[REP], sh_l[REP];
    const int tid = threadIdx.x;
    const float *hp = p.partials + ((size_t)(h * p.part_rows + first_row) * REP) * PW;
    const int n = splits * REP;
    float *wgt = scratch;        // [n] max, then weight
    float *lsum = scratch + n;   // [n] l of every partial row

    for (int e0 = 0; e0 < REP * VPR; e0 += THREADS) {
        const int e = e0 + tid;
        const bool live = e < REP * VPR;
        const int r = live ? e / VPR : 0;
        const int c4 = live ? e % VPR : 0;
        const float4 *col = reinterpret_cast<const float4 *>(hp + (size_t)r * PW) + c4;
        constexpr int RS = REP * PW / 4;  // float4 stride between splits
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
            for (int r = tid >> 5; r < REP; r += THREADS / 32) {
                float mn = NEG_INF;
                for (int s = lane; s < splits; s += 32) mn = fmaxf(mn, wgt[s * REP + r]);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) mn = fmaxf(mn, __shfl_xor_sync(DA_FULL_MASK, mn, off));
                const float ms = (mn == NEG_INF) ? 0.f : mn;
                float ll = 0.f;
                for (int s = lane; s < splits; s += 32) {
                    const float w = fast_exp2(wgt[s * REP + r] - ms);
                    wgt[s * REP + r] = w;
                    ll = fmaf(lsum[s * REP + r], w, ll);
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) ll += __shfl_xor_sync(DA_FULL_MASK, ll, off);
                if (lane == 0) {
                    sh_m[r] = ms;
                    sh_l[r] = ll;
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
                    const float w = wgt[(s0 + u) * REP + r];
                    a.x = fmaf(v[u].x, w, a.x);
                    a.y = fmaf(v[u].y, w, a.y);
                    a.z = fmaf(v[u].z, w, a.z);
                    a.w = fmaf(v[u].w, w, a.w);
                }
            }
        }
        if (live && partial_out) {
            // not the end yet: one partial row (acc weighted to the common max, max, l)
            float *dst = partial_out + (size_t)r * PW;
            reinterpret_cast<float4 *>(dst)[c4] = a;
            if (c4 == 0) {
                dst[D] = sh_m[r];
                dst[D + 1] = sh_l[r];
            }
        } else if (live) {
            const float ll = sh_l[r];
            const float inv = ll > 0.f ? 1.f / ll : 0.f;
            T *dst = reinterpret_cast<T *>(p.out) + (size_t)(h * REP + r) * D + 4 * c4;
            dst[0] = from_float<T>(a.x * inv);
            dst[1] = from_float<T>(a.y * inv);
            dst[2] = from_float<T>(a.z * inv);
            dst[3] = from_float<T>(a.w * inv);
            if (c4 == 0 && p.lse_out) p.lse_out[h * REP + r] = (sh_m[r] + log2f(ll)) * 0.6931471805599453f;
        }
    }
}

// 16-bit element types: tensor-core kernel (attn_mma.cu).
cudaError_t launch_attention_mma(const AttnParams &p, int n_kv_heads, int rep, int head_dim, int dtype,
                                 cudaStream_t stream);

}  // namespace da

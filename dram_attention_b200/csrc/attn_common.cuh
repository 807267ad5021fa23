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
constexpr int kAttnTargetCtas = 444;   // 3 per SM on 148 SMs
constexpr int kAttnMaxSplits = 148;
constexpr int kAttnMaxRows = 16;       // query rows (tokens x GQA group) of one KV head per launch
constexpr int kRoundUnits = 32;        // units a warp plans at a time (one per lane)

// Phase 1 runs beside the selection kernels, whose CTAs need a whole SM each.  Its CTAs are
// therefore built to fill an SM on their own (12 warps, all of the shared memory), and by default
// there are at most 116 of them: wherever the hardware places them, 32 of the 148 SMs stay empty.
// Phase 2 normally covers only the few slots the LRU update could evict; 64 CTAs on those 32 SMs
// are plenty.
constexpr int kAttnPhase1Warps = 12;
constexpr int kAttnPhase1Ctas = 116;
constexpr int kAttnPhase1MaxPerHead = 20;  // a shard of 1 to 4 KV heads: beyond 20 CTAs a head, every further partial
                                           // row costs the final merge (which is on the step's critical path) more
                                           // than the CTA adds in bandwidth (phase 1 is not on that path)
constexpr int kAttnPhase2Ctas = 64;
constexpr int kAttnPhase2MaxPerHead = 8;   // the front is small: more CTAs only lengthen the merge

__host__ __device__ inline int attn_splits(int n_kv_heads) {
    int s = kAttnTargetCtas / n_kv_heads;
    if (s > kAttnMaxSplits) s = kAttnMaxSplits;
    if (s < 1) s = 1;
    return s;
}

__host__ __device__ inline int attn_splits_phase1(int n_kv_heads) {
    int s = kAttnPhase1Ctas / n_kv_heads;
    if (s > kAttnPhase1MaxPerHead) s = kAttnPhase1MaxPerHead;
    if (s < 1) s = 1;
    return s;
}

__host__ __device__ inline int attn_splits_phase2(int n_kv_heads) {
    int s = kAttnPhase2Ctas / n_kv_heads;
    if (s > kAttnPhase2MaxPerHead) s = kAttnPhase2MaxPerHead;
    if (s < 1) s = 1;
    return s;
}

constexpr int kAttnMaxPeers = 16;

struct AttnParams {
    // KV-head sharding: the CTA that merges a head also sends the head's output rows to every rank's gather
    // buffer (see gather.cu for the layout and the tag); null when the caller gathers itself
    // (the pointers travel in the kernel's parameters, so that the store loop at the end of a merge has no
    // dependent load in it; peer_world == 0: nothing is sent)
    uint2 *peer_buf[kAttnMaxPeers];
    const int32_t *peer_seq;
    int peer_rank, peer_world, peer_words;   // words (4 bytes of payload each) per rank
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
    int head_dim;
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

// The words of the eviction queue's state a launch plans from: read together, early (see the kernel body).
struct FrontWords {
    int flip, nf0, nf1;
};
__device__ __forceinline__ FrontWords load_front(const AttnParams &p, int h) {
    FrontWords f = {0, 0, 0};
    if (p.phase != 0) {
        f.nf0 = p.n_evictable[h];
        f.nf1 = p.n_evictable[p.n_kv_heads + h];
        f.flip = p.flip[h];
    }
    return f;
}

// `redo`: the LRU update had to evict beyond the front (second launch only).
__device__ __forceinline__ LaunchUnits launch_units(const AttnParams &p, int h, int n_local, bool redo,
                                                    const FrontWords &fw) {
    LaunchUnits lu;
    lu.order = nullptr;
    lu.order_off = 0;
    lu.ups = p.phase != 0 ? p.page_tokens / kUnitTokens : 1;
    bool local = true;
    if (p.phase == 0) {
        lu.units_slots = (p.n_prefix_tokens + kUnitTokens - 1) / kUnitTokens;
    } else {
        // (the front sizes of both queue copies were read beside the flip word, not after it)
        const int cur = fw.flip & 1;
        const int32_t *order = p.order + ((size_t)cur * p.n_kv_heads + h) * p.n_slots;
        const int n_ev = min(max(cur ? fw.nf1 : fw.nf0, 0), p.n_slots);
        if (p.phase == 1) {
            lu.units_slots = (p.n_slots - n_ev) * lu.ups;
            lu.order = order;
            lu.order_off = n_ev;
        } else if (redo) {
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

// One entry of a warp's plan table (shared memory, in the order the warp visits its units):
//   x, y  global address of the unit's first token (slot table, or the DRAM page to read instead)
//   z     slot-table units: first token inside the head's slot table (>= 0);
//         local-window units: -1 - first token of the unit in the local window
//   w     DRAM page the unit is read from (it is then written through to its slot), or -1
// A round covers the warp's units at positions round * 32 .. round * 32 + n_round - 1; lane i plans
// unit i.  Planning has two halves, so that the second launch of a step can do the first before
// the LRU update has finished: plan_base() needs only the eviction queue as it was BEFORE the
// update, plan_commit() the marks the update leaves (which slots must be read from DRAM).

// First slot-table token of lane's unit of this round, or -1 (a local-window unit, or none).
__device__ __forceinline__ int plan_base(const AttnParams &p, const LaunchUnits &lu, int worker, int n_workers,
                                         int lane, int round, int total_my) {
    const int n_round = min(kRoundUnits, total_my - round * kRoundUnits);
    const int u = worker + (round * kRoundUnits + lane) * n_workers;
    int base = -1;
    if (lane < n_round && u < lu.units_slots) {
        base = u * kUnitTokens;
        if (lu.order) {
            int slot = lu.order[lu.order_off + u / lu.ups];
            slot = min(max(slot, 0), p.n_slots - 1);
            base = slot * p.page_tokens + (u % lu.ups) * kUnitTokens;
        }
    }
    return base;
}

// Writes the round's table.  Units that have to come from DRAM are visited first, so that their
// host-link latency overlaps everything else the warp does.  Returns n_round.
__device__ __forceinline__ int plan_commit(const AttnParams &p, const LaunchUnits &lu, int h, int worker,
                                           int n_workers, int lane, int round, int total_my, int base,
                                           uint4 *tab, size_t elem_bytes) {
    const int n_round = min(kRoundUnits, total_my - round * kRoundUnits);
    const int u = worker + (round * kRoundUnits + lane) * n_workers;
    const bool valid = lane < n_round;
    int src = -1;
    if (base >= 0 && p.slot_source && p.phase != 1)
        src = p.slot_source[(size_t)h * p.n_slots + base / p.page_tokens];
    const unsigned fresh = __ballot_sync(DA_FULL_MASK, valid && src >= 0);
    if (valid) {
        const int before = __popc(fresh & ((1u << lane) - 1));
        const int pos = src >= 0 ? before : __popc(fresh) + (lane - before);
        uint4 e;
        unsigned long long addr = 0;
        if (base >= 0) {
            const size_t tok_bytes = (size_t)2 * p.head_dim * elem_bytes;
            const unsigned char *a =
                src < 0 ? p.prefix + (size_t)h * p.prefix_head_stride * elem_bytes + (size_t)base * tok_bytes
                        : p.dram + (size_t)h * p.dram_head_stride * elem_bytes +
                              ((size_t)src * p.page_tokens + base % p.page_tokens) * tok_bytes;
            addr = (unsigned long long)a;
            e.z = (unsigned)base;
        } else {
            e.z = (unsigned)(-1 - (u - lu.units_slots) * kUnitTokens);
        }
        e.x = (unsigned)(addr & 0xffffffffull);
        e.y = (unsigned)(addr >> 32);
        e.w = (unsigned)src;
        tab[pos] = e;
    }
    __syncwarp();
    return n_round;
}

// Floats per partial row: acc[D], max, l, padded to a multiple of 4 so that rows can
// be read with 128-bit loads.
template <int D> struct PartialRow { static constexpr int kWidth = D + 4; };

__device__ __forceinline__ void cp_async_16(void *dst_smem, const void *src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst_smem)), "l"(src_gmem) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most N of this thread's committed groups are still in flight
template <int N> __device__ __forceinline__ void cp_async_wait_group() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Final merge of the per-CTA partials of one head by one CTA of THREADS threads.  A CTA's
// partial = `rows` rows of (acc[D] already weighted to the row's max, max, l); the partials of
// consecutive CTAs are contiguous in the workspace.  They are brought into shared memory (the
// idle stage buffers, `smem_bytes` of them) with 16-byte asynchronous copies that bypass L1 (the
// rows were written by other SMs) and need no registers.  When they do not all fit, the buffer
// is used as two halves: the next batch is on its way while the current one is added up.  The
// first batch is requested before anything else is looked at.  `skip_flag` (may be null):
// when the word it points to is non-zero the first `skip` CTAs' rows are left out (they get
// weight zero); it is read together with the (max, l) pairs, so it costs no round trip.
template <typename T, int D, int THREADS>
__device__ __forceinline__ void merge_splits(const AttnParams &p, int h, int splits, int rows, const int32_t *skip_flag,
                                             int skip, unsigned char *smem, int smem_bytes) {
    constexpr int PW = PartialRow<D>::kWidth;
    constexpr int VPR = D / 4;          // float4 per accumulator row
    constexpr float NEG_INF = -INFINITY;
    constexpr int MAXE = (kAttnMaxRows * VPR + THREADS - 1) / THREADS;   // output float4 per thread
    __shared__ float sh_m[kAttnMaxRows], sh_l[kAttnMaxRows];
    const int tid = threadIdx.x;
    const int32_t peer_step = p.peer_world > 0 ? __ldcg(p.peer_seq) : 0;   // (needed at the very end: read now)
    const float *hp = p.partials + ((size_t)h * p.part_rows * rows) * PW;
    const int n = splits * rows;
    float *wgt = reinterpret_cast<float *>(smem);   // [n] max, then weight
    float *lsum = wgt + n;                          // [n] l of every partial row
    const int head_bytes = ((2 * n * (int)sizeof(float)) + 15) & ~15;
    float4 *buf0 = reinterpret_cast<float4 *>(smem + head_bytes);
    const int cta_f4 = rows * PW / 4;               // float4 per CTA's partial
    int chunk = (smem_bytes - head_bytes) / (cta_f4 * 16);
    if (chunk < splits) chunk = max(chunk / 2, 1);  // two halves in flight
    chunk = min(chunk, splits);
    float4 *buf1 = buf0 + (size_t)chunk * cta_f4;

    // one commit group per batch (also when this thread has nothing to copy in it)
    auto request = [&](int s0, float4 *buf) {
        const int cnt = min(chunk, splits - s0);
        const float4 *src = reinterpret_cast<const float4 *>(hp) + (size_t)s0 * cta_f4;
        for (int i = tid; i < cnt * cta_f4; i += THREADS) cp_async_16(buf + i, src + i);
        cp_async_commit();
    };
    request(0, buf0);
    if (chunk < splits) request(chunk, buf1);
    const int n_skip = (skip_flag != nullptr && __ldcg(skip_flag) != 0) ? skip * rows : 0;
    for (int i = tid; i < n; i += THREADS) {
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(hp + (size_t)i * PW + D));
        wgt[i] = i < n_skip ? NEG_INF : ml.x;
        lsum[i] = ml.y;
    }
    __syncthreads();
    {   // one warp per query row: common max, weights exp2(max_s - max), weighted row sum
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
    }
    float4 a[MAXE];
#pragma unroll
    for (int k = 0; k < MAXE; ++k) a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    int which = 0;
    for (int s0 = 0; s0 < splits; s0 += chunk, which ^= 1) {
        const int cnt = min(chunk, splits - s0);
        const float4 *buf = which ? buf1 : buf0;
        if (s0 + chunk < splits) cp_async_wait_group<1>(); else cp_async_wait_group<0>();   // this batch has landed
        __syncthreads();      // the batch and (first time round) the weights are in shared memory
#pragma unroll
        for (int k = 0; k < MAXE; ++k) {
            const int e = k * THREADS + tid;
            if (e < rows * VPR) {
                const int r = e / VPR, c4 = e % VPR;
                const float4 *col = buf + r * (PW / 4) + c4;
                for (int s = 0; s < cnt; ++s) {
                    const float4 v = col[s * cta_f4];
                    const float w = wgt[(s0 + s) * rows + r];
                    a[k].x = fmaf(v.x, w, a[k].x);
                    a[k].y = fmaf(v.y, w, a[k].y);
                    a[k].z = fmaf(v.z, w, a[k].z);
                    a[k].w = fmaf(v.w, w, a[k].w);
                }
            }
        }
        if (s0 + 2 * chunk < splits) {
            __syncthreads();  // everybody is done with this half: the batch after the next goes into it
            request(s0 + 2 * chunk, which ? buf1 : buf0);
        }
    }
#pragma unroll
    for (int k = 0; k < MAXE; ++k) {
        const int e = k * THREADS + tid;
        if (e < rows * VPR) {
            const int r = e / VPR, c4 = e % VPR;
            const float ll = sh_l[r];
            const float inv = ll > 0.f ? 1.f / ll : 0.f;
            // row r = (query token, head of the group)
            const int tok = p.q_tok0 + r / p.rep;
            const size_t orow = (size_t)tok * p.n_kv_heads * p.rep + (size_t)h * p.rep + r % p.rep;
            T *dst = reinterpret_cast<T *>(p.out) + orow * D + 4 * c4;
            const T v0 = from_float<T>(a[k].x * inv), v1 = from_float<T>(a[k].y * inv),
                    v2 = from_float<T>(a[k].z * inv), v3 = from_float<T>(a[k].w * inv);
            dst[0] = v0;
            dst[1] = v1;
            dst[2] = v2;
            dst[3] = v3;
            if (c4 == 0 && p.lse_out) p.lse_out[orow] = (sh_m[r] + log2f(ll)) * 0.6931471805599453f;
            if (p.peer_world > 0) {
                // these four values as payload words {payload, tag} into slot (seq & 1) of every rank's buffer,
                // at this rank's place (one query token per call: orow is the head row)
                const int32_t sq = peer_step;
                const uint32_t tag = (uint32_t)(sq + 1);
                constexpr int NW = (int)(4 * sizeof(T) / 4);
                uint32_t w[NW];
                if constexpr (sizeof(T) == 4) {
                    w[0] = __float_as_uint((float)v0);
                    w[1] = __float_as_uint((float)v1);
                    w[NW - 2] = __float_as_uint((float)v2);
                    w[NW - 1] = __float_as_uint((float)v3);
                } else {
                    auto bits = [](T v) -> uint32_t { return (uint32_t)(*reinterpret_cast<const unsigned short *>(&v)); };
                    w[0] = bits(v0) | (bits(v1) << 16);
                    w[NW - 1] = bits(v2) | (bits(v3) << 16);
                }
                const size_t word0 = (size_t)(sq & 1) * p.peer_world * p.peer_words + (size_t)p.peer_rank * p.peer_words +
                                     (orow * D + 4 * c4) * sizeof(T) / 4;
#pragma unroll
                for (int g = 0; g < kAttnMaxPeers; ++g) {
                    if (g < p.peer_world) {
                        uint2 *pd = p.peer_buf[g] + word0;
#pragma unroll
                        for (int i = 0; i < NW; ++i) st_word_sys(pd + i, w[i], tag);
                    }
                }
            }
        }
    }
}

// 16-bit element types: tensor-core kernel (attn_mma.cu).
cudaError_t launch_attention_mma(const AttnParams &p, int n_kv_heads, int head_dim, int dtype, int splits,
                                 cudaStream_t stream);

}  // namespace da

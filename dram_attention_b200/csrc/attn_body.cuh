// The decode-attention kernel without its arithmetic: unit scheduling, the asynchronous copies
// into per-warp stage rings, the append of the new keys/values, the publication of the partials
// and the ticket that elects the merging CTA.  The arithmetic (how a 16-token unit in shared
// memory updates the running softmax state) comes from a `Math` policy: CUDA-core FMAs for
// float32 (attn.cu), warp-level tensor-core MMAs for 16-bit types (attn_mma.cu).
//
// Work unit = 16 consecutive tokens of one KV head.  A warp owns a private ring of stages with
// one mbarrier each, so the main loop has no CTA-wide synchronisation.  Units are dealt
// round-robin to the (CTA, warp) workers of a head; a warp plans 32 of its units at a time
// (one per lane: where the unit lies, whether it has to come from DRAM) into a small table in
// shared memory and walks a round with the DRAM-sourced units first.
//
// Math policy interface:
//   Elem, kD, kPitch (bytes between two tokens of a stage), kPerTokenCopy
//   struct State; init(State&, p, h, lane, rows); consume(State&, stage, avail, lane);
//   publish(State&, red, lane, rows)   red = float [rows][D + 4] of this warp
#pragma once

#include "attn_common.cuh"

namespace da {

template <typename Math, int WARPS, int STAGES>
__device__ __forceinline__ void decode_attention_body(const AttnParams &p, unsigned char *smem) {
    using T = typename Math::Elem;
    constexpr int D = Math::kD;
    constexpr int E = (int)sizeof(T);
    constexpr int ROWB = D * E;                  // one key (or value) row in HBM
    constexpr int TOKB = 2 * ROWB;               // one token of the slot table: key row, value row
    constexpr int PITCH = Math::kPitch;          // the same token in a stage
    constexpr int STAGEB = kUnitTokens * PITCH;
    constexpr int PW = PartialRow<D>::kWidth;
    constexpr int THREADS = WARPS * 32;
    constexpr float NEG_INF = -INFINITY;
    static_assert(STAGES * STAGEB >= kAttnMaxRows * PW * (int)sizeof(float), "a warp's ring holds its partial");

    __shared__ __align__(8) uint64_t bars[WARPS][STAGES];
    __shared__ __align__(16) uint4 plan_tab[WARPS][kRoundUnits];
    __shared__ int sh_last;

    const int h = blockIdx.y;
    const int x = blockIdx.x;
    const int splits = gridDim.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int rows = p.n_q * p.rep;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(&bars[warp][s], 1);
    }
    mbar_fence_init();
    __syncthreads();
    // Launched as a dependent of the kernel before it in the stream, i.e. possibly while that kernel
    // is still at work.  The single launch reads nothing in global memory before the wait.  The
    // second launch of a step (phase 2) always follows the LRU update, whose results it needs only
    // late: it reads its inputs, the eviction queue as it was before the update and its query rows
    // first (all of them complete before the update began) and waits further down.
    const int trace_kernel = p.phase == 2 ? 4 : 3;
    const int trace_cta = h * splits + x;
    if (tid == 0) trace_stamp(trace_kernel, trace_cta, 0);
    if (p.phase != 2) {
        griddep_wait();
        griddep_launch_dependents();   // a dependent launch after this one (the gather of the head shards) may move in
    }

    // ---- everything the CTA has to read before it can plan sets out together: the position, the state of the
    //      eviction queue, the query rows (the first instruction that needs any of them is in Math::init);
    //      one round trip to memory instead of one after the other ------------------------------------
    const int pos = p.start_pos_dev ? *p.start_pos_dev : p.start_pos_host;
    const FrontWords fw = load_front(p, h);
    typename Math::State st;
    Math::init(st, p, h, lane, rows);

    // ---- position and unit range ------------------------------------------------
    int t0 = pos - p.dram_tokens;   // index of the first new token in the local window
    bool pos_ok = true;
    if (t0 < 0 || t0 + p.s_total > p.local_capacity) {
        pos_ok = false;
        if (tid == 0 && x == 0) atomicOr(p.status, DA_STATUS_BAD_POSITION);
        t0 = t0 < 0 ? 0 : p.local_capacity - p.s_total;
    }
    const int n_local = t0 + p.s_total;
    const int n_prefix = p.n_prefix_tokens;
    const int n_workers = splits * WARPS;
    // warp-major worker ids: the workers that get one unit more than the others are spread over all CTAs of
    // the head (one or two per SM), not packed into the first CTAs (twelve on the same SM)
    const int worker = warp * splits + x;
    LaunchUnits lu = launch_units(p, h, n_local, false, fw);
    int units = lu.units_slots + lu.units_local;
    int total_my = units > worker ? (units - worker + n_workers - 1) / n_workers : 0;

    unsigned char *my_stages = smem + (size_t)warp * STAGES * STAGEB;
    uint4 *tab = plan_tab[warp];

    // ---- append the new keys/values to the local window ----------------------------
    if (x == 0 && warp == 0 && pos_ok && p.phase != 2 && p.q_tok0 == 0) {
        for (int i = 0; i < p.s_total; ++i) {
            const size_t srco = ((size_t)i * p.n_kv_heads + h) * ROWB;
            const uint4 *sk = reinterpret_cast<const uint4 *>(p.new_k + srco);
            const uint4 *sv = reinterpret_cast<const uint4 *>(p.new_v + srco);
            const size_t off = ((size_t)(t0 + i) * p.local_tok_stride + (size_t)h * p.local_head_stride) * E;
            uint4 *dk = reinterpret_cast<uint4 *>(p.local_k + off);
            uint4 *dv = reinterpret_cast<uint4 *>(p.local_v + off);
            for (int c = lane; c < ROWB / 16; c += 32) {
                dk[c] = sk[c];
                dv[c] = sv[c];
            }
        }
    }

    const uint64_t stream_policy = l2_policy_evict_first();   // the KV stream is read once per step
    bool dead = false;

    int base0 = plan_base(p, lu, worker, n_workers, lane, 0, total_my);
    if (p.phase == 2) {
        griddep_wait();   // from here on the LRU update is complete
        griddep_launch_dependents();
        if (p.redo[h] != 0) {
            // it evicted beyond the front: this launch covers the whole head
            lu = launch_units(p, h, n_local, true, fw);
            units = lu.units_slots + lu.units_local;
            total_my = units > worker ? (units - worker + n_workers - 1) / n_workers : 0;
            base0 = plan_base(p, lu, worker, n_workers, lane, 0, total_my);
        }
    }

    for (int round = 0; round * kRoundUnits < total_my && !dead; ++round) {
        const int base = round == 0 ? base0 : plan_base(p, lu, worker, n_workers, lane, round, total_my);
        const int n_round = plan_commit(p, lu, h, worker, n_workers, lane, round, total_my, base, tab, (size_t)E);
        const int g0 = round * kRoundUnits;   // units this warp has consumed before this round

        // start the copies of the unit at position `it` of this round into stage s
        auto issue = [&](int s, int it) {
            const uint4 e = tab[it];
            uint64_t *bar = &bars[warp][s];
            unsigned char *dst = my_stages + (size_t)s * STAGEB;
            const int z = (int)e.z;
            if (z >= 0) {
                // slot-table unit (from its slot, or from the DRAM page that was just assigned to it)
                const int ntok = min(kUnitTokens, n_prefix - z);
                const unsigned char *src =
                    reinterpret_cast<const unsigned char *>(((unsigned long long)e.y << 32) | e.x);
                if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)ntok * TOKB);
                __syncwarp();
                if constexpr (Math::kPerTokenCopy) {
                    // a token's key and value rows are contiguous in HBM: one copy per token
                    if (lane < ntok)
                        bulk_copy_g2s_hint(dst + lane * PITCH, src + (size_t)lane * TOKB, TOKB, bar, stream_policy);
                } else {
                    if (lane == 0) bulk_copy_g2s_hint(dst, src, (uint32_t)ntok * TOKB, bar, stream_policy);
                }
            } else {
                // local window: one copy per row, key rows by lanes 0..15, value rows by lanes 16..31
                const int tfirst = -1 - z;
                const int ntok = min(kUnitTokens, n_local - tfirst);
                if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)ntok * TOKB);
                __syncwarp();
                const int tl = lane & 15;
                const int is_v = lane >> 4;
                if (tl < ntok) {
                    const int t = tfirst + tl;
                    const unsigned char *src;
                    if (t >= t0) {   // one of this call's new tokens: straight from the inputs
                        src = (is_v ? p.new_v : p.new_k) + ((size_t)(t - t0) * p.n_kv_heads + h) * ROWB;
                    } else {
                        src = (is_v ? p.local_v : p.local_k) +
                              ((size_t)t * p.local_tok_stride + (size_t)h * p.local_head_stride) * E;
                    }
                    bulk_copy_g2s_hint(dst + tl * PITCH + is_v * ROWB, src, ROWB, bar, stream_policy);
                }
            }
        };

        for (int it = 0; it < STAGES && it < n_round; ++it) issue((g0 + it) % STAGES, it);

        for (int it = 0; it < n_round; ++it) {
            const int g = g0 + it;
            const int s = g % STAGES;
            const uint4 e = tab[it];
            const int z = (int)e.z;
            // tokens that exist from the unit's first token on (before any causal cut)
            const int avail = z >= 0 ? n_prefix - z : n_local - (-1 - z);
            const int ntok = min(kUnitTokens, avail);
            unsigned char *sb = my_stages + (size_t)s * STAGEB;
            const bool arrived = mbar_wait_bounded(&bars[warp][s], (uint32_t)((g / STAGES) & 1));
            if (!__all_sync(DA_FULL_MASK, arrived)) {
                if (lane == 0) atomicOr(p.status, DA_STATUS_WAIT_TIMEOUT);
                dead = true;
                break;
            }
            if (z >= 0 && (int)e.w >= 0) {
                // this unit came from DRAM: write it through to its slot
                unsigned char *slot = const_cast<unsigned char *>(p.prefix) +
                                      ((size_t)h * p.prefix_head_stride + (size_t)z * 2 * D) * E;
                for (int i = lane; i < ntok * (TOKB / 16); i += 32) {
                    const int t = i / (TOKB / 16), c = i % (TOKB / 16);
                    reinterpret_cast<uint4 *>(slot + (size_t)t * TOKB)[c] =
                        reinterpret_cast<const uint4 *>(sb + t * PITCH)[c];
                }
            }
            if (ntok < kUnitTokens) {
                // rows past the end hold stale bytes: zero the value rows so that 0 * garbage
                // cannot produce NaN (their logits are masked)
                for (int i = lane; i < (kUnitTokens - ntok) * (ROWB / 16); i += 32) {
                    const int r = ntok + i / (ROWB / 16);
                    reinterpret_cast<uint4 *>(sb + ROWB + r * PITCH)[i % (ROWB / 16)] = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }

            Math::consume(st, sb, avail, lane, p.scale_log2);

            __syncwarp();
            if (it + STAGES < n_round) issue(s, it + STAGES);
        }
        __syncwarp();   // the table is rewritten by the next round
    }

    // ---- this warp's partial into its own (now idle) ring ----------------------------------
    float *red = reinterpret_cast<float *>(my_stages);
    Math::publish(st, red, lane, rows);
    __syncthreads();
    if (tid == 0) trace_stamp(trace_kernel, trace_cta, 2);

    // ---- merge the warps, write this CTA's partial ------------------------------------
    float *part = p.partials + ((size_t)(h * p.part_rows + p.part_offset + x) * rows) * PW;
    for (int e = tid; e < rows * PW; e += THREADS) {
        const int r = e / PW;
        const int c = e % PW;
        float mn = NEG_INF;
#pragma unroll
        for (int w = 0; w < WARPS; ++w)
            mn = fmaxf(mn, reinterpret_cast<const float *>(smem + (size_t)w * STAGES * STAGEB)[r * PW + D]);
        float outv;
        if (c == D) {
            outv = mn;
        } else if (c > D + 1) {
            outv = 0.f;  // padding
        } else {
            const float ms = (mn == NEG_INF) ? 0.f : mn;
            outv = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float *rw = reinterpret_cast<const float *>(smem + (size_t)w * STAGES * STAGEB) + r * PW;
                outv += rw[c] * fast_exp2(rw[D] - ms);
            }
        }
        part[e] = outv;  // c < D: weighted acc; c == D: max; c == D + 1: weighted l
    }
    __syncthreads();
    if (tid == 0) {
        // The ticket releases this CTA's rows (ordered before this thread by the barrier) and acquires the rows
        // of every CTA that took a ticket before: one acq_rel read-modify-write at GPU scope instead of a fence
        // on either side.  The barrier below carries the acquire to the other threads of the CTA.
        unsigned int ticket;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.counters + h) : "memory");
        sh_last = (ticket == (unsigned int)(p.ticket_target - 1));
    }
    __syncthreads();
    if (tid == 0) {
        trace_stamp(trace_kernel, trace_cta, 3);
        if (!sh_last) trace_stamp(trace_kernel, trace_cta, 1);
    }
    if (!sh_last) return;

    // ---- the CTA of this head that finished last (of both launches, when there are two) --------
    // a head that phase 2 redid: phase 1's rows (the first in the workspace) are left out
    merge_splits<T, D, THREADS>(p, h, p.part_rows, rows, p.phase != 0 ? p.redo + h : nullptr, p.splits1, smem,
                                WARPS * STAGES * STAGEB);
    // every CTA of this head is done with the eviction front: the one the LRU update left becomes current
    if (p.phase != 0 && tid == 0) atomicXor(p.flip + h, 1);   // (no result wanted: the CTA does not wait for it)
    if (tid == 0) p.counters[h] = 0u;
    if (tid == 0) trace_stamp(trace_kernel, trace_cta, 1);
}

}  // namespace da

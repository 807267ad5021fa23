// Per-query-head top-k page selection: radix select on order-preserving 32-bit
// keys, exact lowest-index tie-break, then the k survivors are ranked by
// (score descending, page id ascending).  One CTA per (token, query head) row, or a cluster of
// four CTAs for rows of more than 16 384 pages; the result is written straight into the
// per-KV-head page list.

#include "da_common.cuh"

namespace da {

constexpr int kTopkThreads = 1024;
constexpr int kTopkWarps = kTopkThreads / 32;
constexpr int kTopkMaxK = 4096;

// Candidates the ranking step can take: k plus half as many again (the selection stops
// refining its threshold as soon as the keys above it and its whole bucket fit).
__host__ __device__ inline int topk_candidate_capacity(int k) { return k + (k >> 1); }

// Ascending unsigned order of the key == ascending float order; -0.0 is folded
// onto +0.0 so that the two compare equal (ties then go by page id).
__device__ __forceinline__ uint32_t score_key(float x) {
    uint32_t b = __float_as_uint(x);
    if ((b << 1) == 0) b = 0;
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

__device__ __forceinline__ float key_score(uint32_t key) {
    return __uint_as_float(key ^ ((key >> 31) ? 0x80000000u : 0xffffffffu));
}

// Bucket 0..255 of a score in a linear division of [lo, lo + 256 / scale).  Monotone
// non-decreasing in x (subtraction of a constant, multiplication by a positive constant,
// truncation and clamping all are), which is all the selection needs: a key in a higher
// bucket is strictly larger than a key in a lower one, equal keys share a bucket.
__device__ __forceinline__ int linear_bucket(float x, float lo, float scale) {
    const int b = (int)((x - lo) * scale);
    return min(max(b, 0), 255);
}

// Where the keys of a row live while the kernel runs.  IPT > 0: n_pages <= IPT * 1024
// and every thread keeps its IPT keys in registers after one coalesced read (key j of
// thread t is page j * 1024 + t).  IPT == 0: any length; the row is re-read from
// global memory (L2) in batches of 8 loads per thread.
template <int IPT> struct RowKeys {
    uint32_t k[IPT > 0 ? IPT : 1];

    __device__ __forceinline__ void load(const float *__restrict__ srow, int n, int tid) {
        if constexpr (IPT > 0) {
            float v[IPT];
#pragma unroll
            for (int j = 0; j < IPT; ++j) {
                const int i = j * kTopkThreads + tid;
                v[j] = i < n ? srow[i] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < IPT; ++j) k[j] = score_key(v[j]);
        }
    }

    // f(page, key, valid) for every chunk of 1024 pages in ascending order; every thread
    // of the block calls f the same number of times.
    template <typename F>
    __device__ __forceinline__ void for_each(const float *__restrict__ srow, int n, int tid, F f) const {
        if constexpr (IPT > 0) {
#pragma unroll
            for (int j = 0; j < IPT; ++j) {
                const int i = j * kTopkThreads + tid;
                if (j * kTopkThreads < n) f(i, k[j], i < n);
            }
        } else {
            for (int base = 0; base < n; base += 8 * kTopkThreads) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = base + j * kTopkThreads + tid;
                    v[j] = i < n ? srow[i] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = base + j * kTopkThreads + tid;
                    if (base + j * kTopkThreads < n) f(i, score_key(v[j]), i < n);
                }
            }
        }
    }
};

// Warp 0: over 256 counters taken from the highest index down, the index where the running
// count reaches `need`, the count above it, and its own count.  Lane l owns indices
// 255-8l .. 248-8l.  With `above_of` every index also gets the count above it.
__device__ __forceinline__ void descending_crossing(const int *hist, int need, int lane, int *digit_out,
                                                    int *above_out, int *count_out, int *above_of = nullptr) {
    int c[8], tot = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        c[j] = hist[255 - (lane * 8 + j)];
        tot += c[j];
    }
    int incl = tot;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        int v = __shfl_up_sync(DA_FULL_MASK, incl, off);
        if (lane >= off) incl += v;
    }
    int above = incl - tot;  // keys at higher indices than this lane's block
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int idx = 255 - (lane * 8 + j);
        if (above_of) above_of[idx] = above;
        if (above < need && above + c[j] >= need) {
            *digit_out = idx;
            *above_out = above;
            *count_out = c[j];
        }
        above += c[j];
    }
}

// Orders m candidates (composite keys: ~score key in the high word, page id in the low word, so that
// ascending composite order is score descending, page id ascending): rank = number of smaller
// composite keys; the first k leave.  The candidate array is read two entries per 128-bit load; with
// m odd the pad entry is the largest possible key and counts for nobody.  `rank` is scratch of m ints.
__device__ __forceinline__ void rank_candidates(unsigned long long *cand, int *rank, int m, int k,
                                                int32_t *__restrict__ dst, int tid) {
    for (int e = tid; e < m; e += kTopkThreads) rank[e] = 0;
    if (tid == 0 && (m & 1)) cand[m] = ~0ull;
    __syncthreads();
    {
        // with m < 1024 the comparisons of one element are split over several threads
        const int n_pairs = (m + 1) >> 1;
        int segs = kTopkThreads / m;
        if (segs < 1) segs = 1;
        const int per_sweep = kTopkThreads / segs;
        const int seg_pairs = (n_pairs + segs - 1) / segs;
        const ulonglong2 *pairs = reinterpret_cast<const ulonglong2 *>(cand);
        for (int e0 = 0; e0 < m; e0 += per_sweep) {
            const int e = e0 + tid % per_sweep;
            const int seg = tid / per_sweep;
            if (e < m && seg < segs) {
                const unsigned long long v = cand[e];
                const int j0 = seg * seg_pairs;
                const int j1 = min(n_pairs, j0 + seg_pairs);
                int c = 0;
#pragma unroll 4
                for (int j = j0; j < j1; ++j) {
                    const ulonglong2 w = pairs[j];
                    c += (w.x < v) + (w.y < v);
                }
                if (c) atomicAdd(&rank[e], c);
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < m; e += kTopkThreads) {
        const int rk = rank[e];
        if (rk < k) dst[rk] = (int32_t)(cand[e] & 0xffffffffu);
    }
}

// One row, one CTA: the whole selection.  `dst` receives the k page ids in (score descending,
// page id ascending) order.
template <int IPT>
__device__ __forceinline__ void topk_row(const float *__restrict__ srow, int n_pages, int k, int32_t *__restrict__ dst,
                                         unsigned char *smem_raw) {
    const int cap = topk_candidate_capacity(k);
    unsigned long long *cand = reinterpret_cast<unsigned long long *>(smem_raw);  // [cap + 2]
    int *rank = reinterpret_cast<int *>(cand + cap + 2);                          // [cap]
    __shared__ int hist2[2][256];   // the histogram of pass p is hist2[p & 1]; the other one is cleared meanwhile
    __shared__ int warp_tot[kTopkWarps];
    __shared__ int sh_digit, sh_above, sh_count, sh_taken;
    __shared__ uint32_t sh_kmin, sh_kmax;
    __shared__ int above_of[256];   // linear level 1: candidates in higher buckets, per bucket

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    if (tid < 256) {
        hist2[0][tid] = 0;
        hist2[1][tid] = 0;
    }
    if (tid == 0) {
        sh_kmin = 0xffffffffu;
        sh_kmax = 0u;
    }
    RowKeys<IPT> keys;
    keys.load(srow, n_pages, tid);
    __syncthreads();

    // ---- fast path: one or two histograms over LINEAR buckets of the row's value range ----
    // The radix digits of a float cluster (a row's scores share a few exponents), which makes
    // the first radix passes both slow (every thread hits the same few counters) and weak
    // (the k-th key's bucket still holds thousands).  256 equal-width buckets between the
    // row's minimum and maximum spread the keys out: the bucket of the k-th key typically
    // holds a few dozen, so the keys above it plus that bucket already fit the ranking step.
    // If they do not, the bucket is divided once more; if that fails too (extreme outliers,
    // massive ties) the exact radix select below takes over from scratch.
    int lin_levels = 0;        // 0: radix select decides; 1, 2: candidates = linear buckets
    float lin_lo = 0.f, lin_scale = 0.f, lin_lo2 = 0.f, lin_scale2 = 0.f;
    int lin_b = 0, lin_b2 = 0, lin_m = 0;
    {
        uint32_t kmn = 0xffffffffu, kmx = 0u;
        keys.for_each(srow, n_pages, tid, [&](int, uint32_t key, bool valid) {
            if (valid) {
                kmn = min(kmn, key);
                kmx = max(kmx, key);
            }
        });
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            kmn = min(kmn, __shfl_xor_sync(DA_FULL_MASK, kmn, off));
            kmx = max(kmx, __shfl_xor_sync(DA_FULL_MASK, kmx, off));
        }
        if (lane == 0) {
            atomicMin(&sh_kmin, kmn);
            atomicMax(&sh_kmax, kmx);
        }
        __syncthreads();
        const float lo = key_score(sh_kmin), hi = key_score(sh_kmax);
        const float width = hi - lo;
        if (width > 0.f && width < 3.0e38f) {   // also false for NaN
            lin_lo = lo;
            lin_scale = 256.f / width;
            int need_lin = k, above_total = 0;
            for (int level = 1; level <= 2; ++level) {
                int *hist = hist2[level - 1];
                keys.for_each(srow, n_pages, tid, [&](int, uint32_t key, bool valid) {
                    if (!valid) return;
                    const float x = key_score(key);
                    const int b1 = linear_bucket(x, lin_lo, lin_scale);
                    if (level == 1) atomicAdd(&hist[b1], 1);
                    else if (b1 == lin_b) atomicAdd(&hist[linear_bucket(x, lin_lo2, lin_scale2)], 1);
                });
                __syncthreads();
                if (warp == 0)
                    descending_crossing(hist, need_lin, lane, &sh_digit, &sh_above, &sh_count,
                                        level == 1 ? above_of : nullptr);
                __syncthreads();
                const int b = sh_digit, above = sh_above, cnt = sh_count;
                if (level == 1) {
                    lin_b = b;
                    lin_lo2 = lin_lo + (float)b / lin_scale;
                    lin_scale2 = lin_scale * 256.f;
                } else {
                    lin_b2 = b;
                }
                above_total += above;
                need_lin -= above;
                if (above_total + cnt <= cap) {
                    lin_levels = level;
                    lin_m = above_total + cnt;
                    break;
                }
            }
        }
        if (lin_levels == 0) {
            // the radix select starts from clean histograms
            __syncthreads();
            if (tid < 256) {
                hist2[0][tid] = 0;
                hist2[1][tid] = 0;
            }
            __syncthreads();
        }
    }

    // ---- radix select: key of the k-th largest score -----------------------
    uint32_t prefix = 0, mask = 0;
    int need = k;  // how many still to take among keys that match the prefix
    int count_eq = 0;
    bool early = false;
    for (int pass = 0; pass < 4 && lin_levels == 0; ++pass) {
        const int shift = 24 - 8 * pass;
        int *hist = hist2[pass & 1];
        // the other histogram was last read before the previous pass's final barrier: clear it for
        // the next pass now, so that a pass costs two barriers
        if (tid < 256) hist2[(pass + 1) & 1][tid] = 0;
        keys.for_each(srow, n_pages, tid, [&](int, uint32_t key, bool valid) {
            const bool in = valid && (key & mask) == prefix;
            // Scores cluster in a few exponent buckets, so most lanes of a warp share a
            // digit: the lanes that agree with the first participating lane are counted
            // with one ballot and one atomic, the rest add one by one.
            const uint32_t digit = (key >> shift) & 255u;
            const uint32_t act = __ballot_sync(DA_FULL_MASK, in);
            if (act) {
                const int first = __ffs(act) - 1;
                const uint32_t d0 = __shfl_sync(DA_FULL_MASK, digit, first);
                const uint32_t same = __ballot_sync(DA_FULL_MASK, in && digit == d0);
                if (lane == first) atomicAdd(&hist[d0], __popc(same));
                else if (in && digit != d0) atomicAdd(&hist[digit], 1);
            }
        });
        __syncthreads();
        if (warp == 0) descending_crossing(hist, need, lane, &sh_digit, &sh_above, &sh_count);
        __syncthreads();
        prefix |= (uint32_t)sh_digit << shift;
        mask |= 255u << shift;
        need -= sh_above;
        count_eq = sh_count;
        // (no barrier here: sh_* are next written after the next pass's histogram barrier, which no
        // thread passes before it has read them)
        // The keys above this bucket (k - need of them) are in; if the bucket itself is small, all
        // of it can go to the ranking step, which then decides - no need to refine the threshold.
        if (pass < 3 && k - need + count_eq <= cap) {
            early = true;
            break;
        }
    }
    // Without the early exit: prefix = key of the k-th largest; `need` of the `count_eq` keys equal
    // to it are taken.  With it: every key whose masked bits are >= prefix is a candidate.
    if (lin_levels == 1) {
        // ---- candidates sorted by bucket as they are gathered, then ranked inside their bucket ----
        // Bucket b's candidates go to cand[above_of[b] ...] (a counter per bucket hands out the
        // places; hist2[1] is still all zero), so a candidate's final rank is above_of[b] plus
        // its rank among the handful of keys of its own bucket.
        const int *count_of = hist2[0];
        int *fill = hist2[1];
        keys.for_each(srow, n_pages, tid, [&](int i, uint32_t key, bool valid) {
            if (!valid) return;
            const int b = linear_bucket(key_score(key), lin_lo, lin_scale);
            if (b >= lin_b) {
                const int at = above_of[b] + atomicAdd(&fill[b], 1);
                cand[at] = ((unsigned long long)(~key) << 32) | (uint32_t)i;
            }
        });
        __syncthreads();
        for (int e = tid; e < lin_m; e += kTopkThreads) {
            const unsigned long long v = cand[e];
            const int b = linear_bucket(key_score(~(uint32_t)(v >> 32)), lin_lo, lin_scale);
            const int first = above_of[b];
            const int last = first + count_of[b];
            int c = first;
            for (int j = first; j < last; ++j) c += cand[j] < v;
            if (c < k) dst[c] = (int32_t)(v & 0xffffffffu);
        }
        return;
    }

    const uint32_t thr = prefix;
    const int m = lin_levels ? lin_m : (early ? k - need + count_eq : k);   // candidates that get ranked

    // ---- gather the survivors ------------------------------------------------
    // Two sweeps over the keys instead of a shared counter: every warp first counts what it
    // will take, a scan over the 32 warp totals gives each warp its range of `cand`, and the
    // second sweep writes without atomics.
    const bool take_all_ties = lin_levels != 0 || early || (count_eq == need);
    auto taken = [&](uint32_t key) -> bool {
        if (lin_levels) {
            const float x = key_score(key);
            const int b1 = linear_bucket(x, lin_lo, lin_scale);
            if (lin_levels == 1 || b1 != lin_b) return b1 >= lin_b;
            return linear_bucket(x, lin_lo2, lin_scale2) >= lin_b2;
        }
        if (early) return (key & mask) >= thr;
        return key > thr || (take_all_ties && key == thr);
    };
    int warp_count = 0;
    keys.for_each(srow, n_pages, tid, [&](int, uint32_t key, bool valid) {
        const bool take = valid && taken(key);
        warp_count += __popc(__ballot_sync(DA_FULL_MASK, take));
    });
    if (lane == 0) warp_tot[warp] = warp_count;
    __syncthreads();
    int warp_base;
    {
        const int wt = warp_tot[lane];
        int incl = wt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(DA_FULL_MASK, incl, off);
            if (lane >= off) incl += v;
        }
        warp_base = __shfl_sync(DA_FULL_MASK, incl - wt, warp);
        const int all = __shfl_sync(DA_FULL_MASK, incl, 31);
        if (tid == 0) sh_taken = all;
    }
    keys.for_each(srow, n_pages, tid, [&](int i, uint32_t key, bool valid) {
        const bool take = valid && taken(key);
        const uint32_t bal = __ballot_sync(DA_FULL_MASK, take);
        if (take) cand[warp_base + __popc(bal & ((1u << lane) - 1))] = ((unsigned long long)(~key) << 32) | (uint32_t)i;
        warp_base += __popc(bal);
    });
    __syncthreads();
    if (!take_all_ties) {
        // the `need` lowest page ids among keys == thr, by an ordered block scan
        int taken_ties = 0;  // uniform across the block
        const int first_slot = sh_taken;
        __syncthreads();
        keys.for_each(srow, n_pages, tid, [&](int i, uint32_t key, bool valid) {
            if (taken_ties >= need) return;  // uniform
            const bool f = valid && key == thr;
            const uint32_t bal = __ballot_sync(DA_FULL_MASK, f);
            if (lane == 0) warp_tot[warp] = __popc(bal);
            __syncthreads();
            int before = 0, total = 0;
            for (int w = 0; w < kTopkWarps; ++w) {
                const int c = warp_tot[w];
                if (w < warp) before += c;
                total += c;
            }
            const int my = taken_ties + before + __popc(bal & ((1u << lane) - 1));
            if (f && my < need) cand[first_slot + my] = ((unsigned long long)(~thr) << 32) | (uint32_t)i;
            taken_ties += total;
            __syncthreads();
        });
    }
    __syncthreads();

    rank_candidates(cand, rank, m, k, dst, tid);
}

// Where row `row` of the launch ((token * n_kv_heads + hk) * rep + r) goes in the per-KV-head page list.
__device__ __forceinline__ int32_t *row_destination(int32_t *page_list, int row, int rows, int n_kv_heads, int rep, int k) {
    const int r = row % rep;
    const int hk = (row / rep) % n_kv_heads;
    const int tok = row / (rep * n_kv_heads);
    const int n_tokens = rows / (n_kv_heads * rep);
    return page_list + (size_t)hk * n_tokens * rep * k + (size_t)(tok * rep + r) * k;
}

template <int IPT>
__global__ void __launch_bounds__(kTopkThreads)
topk_pages_kernel(const float *__restrict__ scores, int32_t *__restrict__ page_list, int n_kv_heads, int rep,
                  int n_pages, int k) {
    if (threadIdx.x == 0) trace_stamp(1, blockIdx.x, 0);
    // on whichever path the kernel leaves: thread 0's end stamp
    struct EndStamp {
        __device__ ~EndStamp() {
            if (threadIdx.x == 0) trace_stamp(1, blockIdx.x, 1);
        }
    } end_stamp;
    griddep_wait();                // the scores come from the kernel before this one
    if (threadIdx.x == 0) trace_stamp(1, blockIdx.x, 2);
    griddep_launch_dependents();   // the LRU update may move onto the SMs and wait there
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int row = blockIdx.x;
    topk_row<IPT>(scores + (size_t)row * n_pages, n_pages, k,
                  row_destination(page_list, row, gridDim.x, n_kv_heads, rep, k), smem_raw);
}

// ---- long rows: one row per cluster of kTopkCluster CTAs ---------------------------------------
// A single CTA spends its time walking the row (64 keys per thread at 65 536 pages, several
// sweeps).  Here every CTA of a cluster keeps a quarter of the row in registers (16 keys per
// thread); the row's value range and the bucket counts are summed over the cluster through
// distributed shared memory, every CTA finds the same threshold bucket, and the candidates of
// all CTAs meet in CTA 0's shared memory (remote atomics hand out the places), where they are
// ranked as in the one-CTA kernel.  Rows that the two linear levels cannot resolve (extreme
// outliers, massive ties, a constant row) fall back to the one-CTA selection, run by CTA 0.
constexpr int kTopkCluster = 4;
constexpr int kTopkClusterIpt = 16;
constexpr int kTopkClusterMaxPages = kTopkCluster * kTopkClusterIpt * kTopkThreads;   // 65 536

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t dsmem_addr(const void *local, uint32_t rank) {
    uint32_t a = smem_addr(local), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ int dsmem_ld_s32(uint32_t addr) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ int dsmem_atomic_add_s32(uint32_t addr, int v) {
    int old;
    asm volatile("atom.shared::cluster.add.s32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void dsmem_st_u64(uint32_t addr, unsigned long long v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}

// The fall-back of the cluster kernel, kept out of line so that the common path stays small in the
// instruction cache.
__device__ __noinline__ void topk_row_fallback(const float *__restrict__ srow, int n_pages, int k,
                                               int32_t *__restrict__ dst, unsigned char *smem_raw) {
    topk_row<0>(srow, n_pages, k, dst, smem_raw);
}

__global__ void __launch_bounds__(kTopkThreads)
topk_pages_cluster_kernel(const float *__restrict__ scores, int32_t *__restrict__ page_list, int n_kv_heads, int rep,
                          int n_pages, int k) {
    if (threadIdx.x == 0) trace_stamp(1, blockIdx.x, 0);
    struct EndStamp {
        __device__ ~EndStamp() {
            if (threadIdx.x == 0) trace_stamp(1, blockIdx.x, 1);
        }
    } end_stamp;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int cap = topk_candidate_capacity(k);
    unsigned long long *cand = reinterpret_cast<unsigned long long *>(smem_raw);  // [cap + 2], used in CTA 0
    int *rank = reinterpret_cast<int *>(cand + cap + 2);                          // [cap]
    __shared__ int hist[2][256];      // this CTA's bucket counts of level 1 and level 2
    __shared__ int total[256];        // the cluster's counts of the level at hand
    __shared__ int above_of[256];     // level 1: candidates in higher buckets, per bucket
    __shared__ int fill[256];         // CTA 0: places handed out per bucket (level 1) / in all ([0], level 2)
    __shared__ uint32_t sh_kmin, sh_kmax;
    __shared__ int sh_digit, sh_above, sh_count;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t crank = cluster_ctarank();
    const int row = blockIdx.x / kTopkCluster;
    const int rows = gridDim.x / kTopkCluster;
    const float *srow = scores + (size_t)row * n_pages;
    int32_t *dst = row_destination(page_list, row, rows, n_kv_heads, rep, k);
    // this CTA's part of the row: `per` pages from `base` (a multiple of 4 pages, so that every part starts aligned)
    const int per = (((n_pages + kTopkCluster - 1) / kTopkCluster) + 3) & ~3;
    const int base = min((int)crank * per, n_pages);
    const int n_mine = min(per, n_pages - base);

    if (tid < 256) {
        hist[0][tid] = 0;
        hist[1][tid] = 0;
        fill[tid] = 0;
    }
    if (tid == 0) {
        sh_kmin = 0xffffffffu;
        sh_kmax = 0u;
    }
    griddep_wait();                // the scores come from the kernel before this one
    if (tid == 0) trace_stamp(1, blockIdx.x, 2);
    griddep_launch_dependents();   // the LRU update may move onto the SMs and wait there
    RowKeys<kTopkClusterIpt> keys;
    keys.load(srow + base, n_mine, tid);
    __syncthreads();

    // ---- the row's value range ------------------------------------------------------------------
    {
        uint32_t kmn = 0xffffffffu, kmx = 0u;
        keys.for_each(srow + base, n_mine, tid, [&](int, uint32_t key, bool valid) {
            if (valid) {
                kmn = min(kmn, key);
                kmx = max(kmx, key);
            }
        });
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            kmn = min(kmn, __shfl_xor_sync(DA_FULL_MASK, kmn, off));
            kmx = max(kmx, __shfl_xor_sync(DA_FULL_MASK, kmx, off));
        }
        if (lane == 0) {
            atomicMin(&sh_kmin, kmn);
            atomicMax(&sh_kmax, kmx);
        }
    }
    cluster_sync_all();   // every CTA's range (and its cleared counters) can be read
    uint32_t gmin = 0xffffffffu, gmax = 0u;
#pragma unroll
    for (uint32_t c = 0; c < kTopkCluster; ++c) {
        gmin = min(gmin, (uint32_t)dsmem_ld_s32(dsmem_addr(&sh_kmin, c)));
        gmax = max(gmax, (uint32_t)dsmem_ld_s32(dsmem_addr(&sh_kmax, c)));
    }
    const float lo = key_score(gmin), hi = key_score(gmax);
    const float width = hi - lo;
    int lin_levels = 0, lin_b = 0, lin_b2 = 0, lin_m = 0;
    const float lin_lo = lo, lin_scale = 256.f / width;
    float lin_lo2 = 0.f, lin_scale2 = 0.f;
    if (width > 0.f && width < 3.0e38f) {   // also false for NaN; uniform over the cluster
        int need_lin = k, above_total = 0;
        for (int level = 1; level <= 2; ++level) {
            int *h = hist[level - 1];
            keys.for_each(srow + base, n_mine, tid, [&](int, uint32_t key, bool valid) {
                if (!valid) return;
                const float x = key_score(key);
                const int b1 = linear_bucket(x, lin_lo, lin_scale);
                if (level == 1) atomicAdd(&h[b1], 1);
                else if (b1 == lin_b) atomicAdd(&h[linear_bucket(x, lin_lo2, lin_scale2)], 1);
            });
            cluster_sync_all();
            if (tid < 256) {
                int t = 0;
#pragma unroll
                for (uint32_t c = 0; c < kTopkCluster; ++c) t += dsmem_ld_s32(dsmem_addr(&h[tid], c));
                total[tid] = t;
            }
            __syncthreads();
            if (warp == 0)
                descending_crossing(total, need_lin, lane, &sh_digit, &sh_above, &sh_count,
                                    level == 1 ? above_of : nullptr);
            __syncthreads();
            const int b = sh_digit, above = sh_above, cnt = sh_count;
            if (level == 1) {
                lin_b = b;
                lin_lo2 = lin_lo + (float)b / lin_scale;
                lin_scale2 = lin_scale * 256.f;
            } else {
                lin_b2 = b;
            }
            above_total += above;
            need_lin -= above;
            if (above_total + cnt <= cap) {
                lin_levels = level;
                lin_m = above_total + cnt;
                break;
            }
            __syncthreads();   // sh_* and total are rewritten by the next level
        }
    }
    if (lin_levels == 0) {
        // the one-CTA selection over the whole row, by CTA 0 (nobody reads anybody's shared memory from here on)
        cluster_sync_all();
        if (crank == 0) topk_row_fallback(srow, n_pages, k, dst, smem_raw);
        return;
    }

    // ---- the candidates meet in CTA 0 -------------------------------------------------------------
    // Level 1: bucket b's candidates go to cand[above_of[b] ...], so that a candidate's final rank is
    // above_of[b] plus its rank among the few keys of its own bucket.  Level 2: places in arrival order.
    const uint32_t cand0 = dsmem_addr(cand, 0);
    keys.for_each(srow + base, n_mine, tid, [&](int i, uint32_t key, bool valid) {
        if (!valid) return;
        const float x = key_score(key);
        const int b1 = linear_bucket(x, lin_lo, lin_scale);
        bool take;
        int counter, first;
        if (lin_levels == 1) {
            take = b1 >= lin_b;
            counter = b1;
            first = above_of[b1];
        } else {
            take = b1 > lin_b || (b1 == lin_b && linear_bucket(x, lin_lo2, lin_scale2) >= lin_b2);
            counter = 0;
            first = 0;
        }
        if (take) {
            const int at = first + dsmem_atomic_add_s32(dsmem_addr(&fill[counter], 0), 1);
            dsmem_st_u64(cand0 + (uint32_t)at * 8u, ((unsigned long long)(~key) << 32) | (uint32_t)(base + i));
        }
    });
    cluster_sync_all();   // all candidates are in place; the other CTAs are done
    if (crank != 0) return;
    if (lin_levels == 1) {
        for (int e = tid; e < lin_m; e += kTopkThreads) {
            const unsigned long long v = cand[e];
            const int b = linear_bucket(key_score(~(uint32_t)(v >> 32)), lin_lo, lin_scale);
            const int first = above_of[b];
            const int last = first + total[b];
            int c = first;
            for (int j = first; j < last; ++j) c += cand[j] < v;
            if (c < k) dst[c] = (int32_t)(v & 0xffffffffu);
        }
        return;
    }
    rank_candidates(cand, rank, lin_m, k, dst, tid);
}
template <int IPT>
static cudaError_t launch_topk(const float *scores, int32_t *page_list, int rows, int n_kv_heads, int rep,
                               int n_pages, int k, cudaStream_t stream) {
    // opt in to > 48 KB of dynamic shared memory once per device
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(topk_pages_kernel<IPT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 topk_candidate_capacity(kTopkMaxK) * 12 + 16);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int cap = topk_candidate_capacity(k);
    const size_t smem = (size_t)(cap + 2) * sizeof(unsigned long long) + (size_t)cap * sizeof(int);
    const cudaError_t le = launch_dependent(topk_pages_kernel<IPT>, dim3(rows), dim3(kTopkThreads), (size_t)smem, stream,
                                            scores, page_list, n_kv_heads, rep, n_pages, k);
    if (le != cudaSuccess) return le;
    return cudaGetLastError();
}

static cudaError_t launch_topk_cluster(const float *scores, int32_t *page_list, int rows, int n_kv_heads, int rep,
                                       int n_pages, int k, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(topk_pages_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 topk_candidate_capacity(kTopkMaxK) * 12 + 16);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int cap = topk_candidate_capacity(k);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * kTopkCluster);
    cfg.blockDim = dim3(kTopkThreads);
    cfg.dynamicSmemBytes = (size_t)(cap + 2) * sizeof(unsigned long long) + (size_t)cap * sizeof(int);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = kTopkCluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    e = cudaLaunchKernelEx(&cfg, topk_pages_cluster_kernel, scores, page_list, n_kv_heads, rep, n_pages, k);
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

}  // namespace da

extern "C" int da_topk_pages_wide(const float *scores, int32_t *page_list, int n_tokens, int n_kv_heads, int rep,
                                  int n_pages, int k, int sm_budget, da_stream_t stream) {
    if (!scores || !page_list) return DA_ERR_NULL;
    if (n_tokens < 1 || n_kv_heads < 1 || rep < 1 || n_pages < 1 || k < 1 || k > n_pages || sm_budget < 0)
        return DA_ERR_SHAPE;
    if (k > da::kTopkMaxK) return DA_ERR_UNSUPPORTED;
    const int rows = n_tokens * n_kv_heads * rep;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (sm_budget == 0) sm_budget = 148;
    // long rows are split over a cluster when all clusters find an SM per CTA at once; otherwise the
    // clusters would run in turns and one CTA per row is as fast
    if (n_pages > 16 * da::kTopkThreads && n_pages <= da::kTopkClusterMaxPages && rows * da::kTopkCluster <= sm_budget)
        e = da::launch_topk_cluster(scores, page_list, rows, n_kv_heads, rep, n_pages, k, s);
    else if (n_pages <= 4 * da::kTopkThreads) e = da::launch_topk<4>(scores, page_list, rows, n_kv_heads, rep, n_pages, k, s);
    else if (n_pages <= 8 * da::kTopkThreads) e = da::launch_topk<8>(scores, page_list, rows, n_kv_heads, rep, n_pages, k, s);
    else if (n_pages <= 16 * da::kTopkThreads) e = da::launch_topk<16>(scores, page_list, rows, n_kv_heads, rep, n_pages, k, s);
    else e = da::launch_topk<0>(scores, page_list, rows, n_kv_heads, rep, n_pages, k, s);
    return (int)e;
}

extern "C" int da_topk_pages(const float *scores, int32_t *page_list, int n_tokens, int n_kv_heads, int rep,
                             int n_pages, int k, da_stream_t stream) {
    return da_topk_pages_wide(scores, page_list, n_tokens, n_kv_heads, rep, n_pages, k, 0, stream);
}

DA_DEFINE_TRACE_SETTER(trace_set_topk)

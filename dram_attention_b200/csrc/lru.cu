// LRU slot-table update: one CTA per KV head does, in one launch, what the
// reference does with a marking kernel, a library sort and a serial walk.
//
//   1. hits: every listed page that is resident gets time = step.
//   2. misses: the first appearance (in list order) of every non-resident page is
//      found with an atomicMin of the list index into the page's own table entry
//      (entries of non-resident pages are negative, so codes below -1 are free),
//      and ranked by a block prefix sum.
//   3. victims: slots ordered by (time, slot) with a stable LSD radix sort on the
//      time in shared memory; only as many 8-bit passes as the step counter has
//      bytes.
//   4. the j-th miss takes the j-th victim; tables updated; (page, slot) pairs
//      emitted for the payload copy.

#include "da_common.cuh"

namespace da {

constexpr int kLruThreads = 1024;
constexpr int kLruWarps = kLruThreads / 32;
constexpr int kLruMaxSlots = 8192;
constexpr int kLruMaxList = 8192;
constexpr int kLruMaxRounds = kLruMaxSlots / kLruThreads;  // items per lane in the sort

// Exclusive prefix sum over the block of one int per thread; returns the
// exclusive value and writes the block total to *total.  `wsum` is 32 ints of
// shared memory.  Contains two __syncthreads().
__device__ __forceinline__ int block_exclusive_scan(int v, int *wsum, int *total) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        int t = __shfl_up_sync(DA_FULL_MASK, incl, off);
        if (lane >= off) incl += t;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    int before = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kLruWarps; ++w) {
        const int c = wsum[w];
        if (w < warp) before += c;
        tot += c;
    }
    *total = tot;
    __syncthreads();
    return before + incl - v;
}

__global__ void __launch_bounds__(kLruThreads)
lru_update_kernel(const int32_t *__restrict__ page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                  int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step_counters,
                  int32_t *__restrict__ miss_pages, int32_t *__restrict__ miss_slots,
                  int32_t *__restrict__ n_miss_out, int32_t *status) {
    extern __shared__ __align__(16) int smem_i[];
    int *keyA = smem_i;                  // [n_slots] sort keys (access time)
    int *valA = keyA + n_slots;          // [n_slots] slot ids
    int *keyB = valA + n_slots;
    int *valB = keyB + n_slots;
    int *mpage = valB + n_slots;         // [list_len] miss pages in list order
    int *hist = mpage + list_len;        // [256 * 32] digit-major, warp-minor
    __shared__ int wsum[kLruWarps];
    __shared__ int sh_max;

    const int h = blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int32_t *list = page_list + (size_t)h * list_len;
    int32_t *d2s = dram_to_slot + (size_t)h * n_dram_pages;
    int32_t *s2d = slot_to_dram + (size_t)h * n_slots;
    int32_t *tim = access_time + (size_t)h * n_slots;
    int32_t *mp_out = miss_pages + (size_t)h * list_len;
    int32_t *ms_out = miss_slots + (size_t)h * list_len;

    const int step = step_counters[h] + 1;
    if (tid == 0) sh_max = step;
    for (int s = tid; s < n_slots; s += kLruThreads) {
        keyA[s] = tim[s];
        valA[s] = s;
    }
    __syncthreads();

    // ---- 1. hits, and first-appearance marks for non-resident pages -----------
    // code(i) = i - list_len - 1 is in [-list_len-1, -2]; the smallest list index wins.
    int bad = 0;
    for (int i = tid; i < list_len; i += kLruThreads) {
        const int p = list[i];
        if (p < 0 || p >= n_dram_pages) { bad = 1; continue; }
        const int s = __ldcg(&d2s[p]);
        if (s >= 0) {
            if (s < n_slots) { keyA[s] = step; tim[s] = step; }
        } else {
            atomicMin(&d2s[p], i - list_len - 1);
        }
    }
    if (bad) atomicOr(status, DA_STATUS_BAD_PAGE_ID);
    __syncthreads();

    // ---- 2. rank the first appearances in list order ---------------------------
    int n_miss = 0;
    for (int base = 0; base < list_len; base += kLruThreads) {
        const int i = base + tid;
        int p = -1, f = 0;
        if (i < list_len) {
            p = list[i];
            if (p >= 0 && p < n_dram_pages) f = (__ldcg(&d2s[p]) == i - list_len - 1);
        }
        int total;
        const int j = n_miss + block_exclusive_scan(f, wsum, &total);
        if (f) mpage[j] = p;
        n_miss += total;
    }
    __syncthreads();

    if (n_miss > 0) {
        // ---- 3. stable radix sort of the slots by access time --------------------
        for (int s = tid; s < n_slots; s += kLruThreads) atomicMax(&sh_max, keyA[s]);
        __syncthreads();
        const int bits = 32 - __clz(sh_max | 1);
        const int passes = (bits + 7) / 8;
        // warp w owns the contiguous items [w * per_warp, (w + 1) * per_warp)
        const int per_warp = (((n_slots + kLruWarps - 1) / kLruWarps) + 31) / 32 * 32;
        const int rounds = per_warp / 32;  // <= kLruMaxRounds
        int *kin = keyA, *vin = valA, *kout = keyB, *vout = valB;
        for (int pass = 0; pass < passes; ++pass) {
            const int shift = 8 * pass;
            for (int x = tid; x < 256 * kLruWarps; x += kLruThreads) hist[x] = 0;
            __syncthreads();
            int off[kLruMaxRounds], dig[kLruMaxRounds];
#pragma unroll
            for (int r = 0; r < kLruMaxRounds; ++r) {
                off[r] = 0;
                dig[r] = -1;
                if (r < rounds) {
                    const int i = warp * per_warp + r * 32 + lane;
                    const bool valid = i < n_slots;
                    const int d = valid ? ((kin[i] >> shift) & 255) : 256;
                    const uint32_t peers = __match_any_sync(DA_FULL_MASK, d);
                    const int leader = __ffs(peers) - 1;
                    const int pos = __popc(peers & ((1u << lane) - 1));
                    int base = 0;
                    if (valid && lane == leader) {
                        base = hist[d * kLruWarps + warp];
                        hist[d * kLruWarps + warp] = base + __popc(peers);
                    }
                    base = __shfl_sync(DA_FULL_MASK, base, leader);
                    if (valid) {
                        off[r] = base + pos;
                        dig[r] = d;
                    }
                    __syncwarp();
                }
            }
            __syncthreads();
            // exclusive scan of hist in (digit, warp) order: 8 consecutive entries per thread
            {
                int c[8], tot = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    c[j] = hist[tid * 8 + j];
                    tot += c[j];
                }
                int total;
                int run = block_exclusive_scan(tot, wsum, &total);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    hist[tid * 8 + j] = run;
                    run += c[j];
                }
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < kLruMaxRounds; ++r) {
                if (r < rounds && dig[r] >= 0) {
                    const int i = warp * per_warp + r * 32 + lane;
                    const int dst = hist[dig[r] * kLruWarps + warp] + off[r];
                    kout[dst] = kin[i];
                    vout[dst] = vin[i];
                }
            }
            __syncthreads();
            int *t = kin; kin = kout; kout = t;
            t = vin; vin = vout; vout = t;
        }
        // kin/vin now hold the slots in eviction order.

        // ---- 4. overflow check, then assignment ------------------------------------
        const bool overflow = (n_miss > n_slots) || (kin[min(n_miss, n_slots) - 1] >= step);
        if (overflow) {
            // undo the marks; tables stay as after the hit marking
            for (int j = tid; j < n_miss; j += kLruThreads) d2s[mpage[j]] = -1;
            if (tid == 0) atomicOr(status, DA_STATUS_LRU_OVERFLOW);
            n_miss = 0;
        } else {
            for (int j = tid; j < n_miss; j += kLruThreads) {
                const int p = mpage[j];
                const int v = vin[j];
                const int old = s2d[v];
                if (old >= 0 && old < n_dram_pages) d2s[old] = -1;
                s2d[v] = p;
                d2s[p] = v;
                tim[v] = step;
                mp_out[j] = p;
                ms_out[j] = v;
            }
        }
    }
    if (tid == 0) {
        n_miss_out[h] = n_miss;
        step_counters[h] = step;
    }
}

static size_t lru_smem_bytes(int n_slots, int list_len) {
    return ((size_t)4 * n_slots + list_len + 256 * kLruWarps) * sizeof(int);
}

}  // namespace da

extern "C" int da_lru_update(const int32_t *page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                             int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step,
                             int n_kv_heads, int32_t *miss_pages, int32_t *miss_slots, int32_t *n_miss,
                             int32_t *status, da_stream_t stream) {
    if (!page_list || !dram_to_slot || !slot_to_dram || !access_time || !step || !miss_pages || !miss_slots ||
        !n_miss || !status)
        return DA_ERR_NULL;
    if (list_len < 1 || n_dram_pages < 1 || n_slots < 1 || n_kv_heads < 1) return DA_ERR_SHAPE;
    if (n_slots > da::kLruMaxSlots || list_len > da::kLruMaxList) return DA_ERR_UNSUPPORTED;
    const size_t smem = da::lru_smem_bytes(n_slots, list_len);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DA_ERR_UNSUPPORTED;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(da::lru_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)da::lru_smem_bytes(da::kLruMaxSlots, da::kLruMaxList));
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    da::lru_update_kernel<<<n_kv_heads, da::kLruThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        page_list, list_len, dram_to_slot, n_dram_pages, slot_to_dram, access_time, n_slots, step, miss_pages,
        miss_slots, n_miss, status);
    return (int)cudaGetLastError();
}

// LRU slot-table update: one CTA per KV head does, in one launch, what the
// reference does with a marking kernel, a library sort and a serial walk.
//
//   1. hits: every listed page that is resident gets time = step.
//   2. misses: the first appearance (in list order) of every non-resident page is
//      found with a shared-memory hash table keyed by page id that keeps the
//      smallest list index, and ranked by a block prefix sum.
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
    // every warp scans the 32 warp totals with shuffles (one read per lane)
    const int wt = wsum[lane];
    int wincl = wt;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        int t = __shfl_up_sync(DA_FULL_MASK, wincl, off);
        if (lane >= off) wincl += t;
    }
    const int before = __shfl_sync(DA_FULL_MASK, wincl - wt, warp);
    *total = __shfl_sync(DA_FULL_MASK, wincl, 31);
    __syncthreads();
    return before + incl - v;
}

constexpr int kLruMaxListRounds = kLruMaxList / kLruThreads;

// Shared-memory plan (ints): keyA[n_slots] valA[n_slots] | X[2 * max(n_slots, table)] |
// mpage[list_len] | hist[256 * 32] | s2d[n_slots].  X is the page hash table
// (keys, first list index) while misses are found and the sort's second buffer after.
__host__ __device__ inline int lru_table_size(int list_len) {
    int t = 64;
    while (t < 2 * list_len) t <<= 1;
    return t;
}

__global__ void __launch_bounds__(kLruThreads)
lru_update_kernel(const int32_t *__restrict__ page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                  int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step_counters,
                  int32_t *__restrict__ miss_pages, int32_t *__restrict__ miss_slots,
                  int32_t *__restrict__ n_miss_out, int32_t *slot_source, int32_t *order_out,
                  int32_t *n_evictable_out, int32_t *status) {
    extern __shared__ __align__(16) int smem_i[];
    const int table = lru_table_size(list_len);
    const int xhalf = n_slots > table ? n_slots : table;
    int *keyA = smem_i;                  // [n_slots] sort keys (access time)
    int *valA = keyA + n_slots;          // [n_slots] slot ids
    int *xbuf = valA + n_slots;          // [2 * xhalf]
    int *tkey = xbuf;                    // [table] page id or -1
    int *tval = xbuf + table;            // [table] smallest list index of that page
    int *keyB = xbuf;                    // [n_slots]   (after the table is dead)
    int *valB = xbuf + n_slots;          // [n_slots]
    int *mpage = xbuf + 2 * xhalf;       // [list_len] miss pages in list order
    int *hist = mpage + list_len;        // [256 * 32] digit-major, warp-minor
    int *s2d_s = hist + 256 * kLruWarps; // [n_slots] slot -> page before this step
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

    // slot_source[slot] = DRAM page whose payload still has to be brought into the slot, -1
    // otherwise: forget the marks of the previous call (its miss list is still in ms_out)
    int32_t *src_map = slot_source ? slot_source + (size_t)h * n_slots : nullptr;
    if (src_map) {
        const int prev = min(n_miss_out[h], list_len);
        for (int j = tid; j < prev; j += kLruThreads) {
            const int v = ms_out[j];
            if (v >= 0 && v < n_slots) src_map[v] = -1;
        }
    }

    // ---- independent global reads first: list, its table entries, times, slot map ------
    int pg[kLruMaxListRounds], sl[kLruMaxListRounds];
    int bad = 0;
#pragma unroll
    for (int r = 0; r < kLruMaxListRounds; ++r) {
        const int i = r * kLruThreads + tid;
        pg[r] = -1;
        if (r * kLruThreads < list_len && i < list_len) {
            const int p = list[i];
            if (p < 0 || p >= n_dram_pages) bad = 1; else pg[r] = p;
        }
    }
    const int step = step_counters[h] + 1;
#pragma unroll
    for (int r = 0; r < kLruMaxListRounds; ++r) sl[r] = pg[r] >= 0 ? d2s[pg[r]] : 0;
    for (int s = tid; s < n_slots; s += kLruThreads) {
        keyA[s] = tim[s];
        valA[s] = s;
        s2d_s[s] = s2d[s];
    }
    for (int x = tid; x < table; x += kLruThreads) {
        tkey[x] = -1;
        tval[x] = 0x7fffffff;
    }
    if (tid == 0) sh_max = step;
    if (bad) atomicOr(status, DA_STATUS_BAD_PAGE_ID);
    __syncthreads();

    // ---- 1. hits get the step; non-resident pages go into the hash table -------------
    const int tmask = table - 1;
    const int tshift = 32 - (__ffs(table) - 1);
#pragma unroll
    for (int r = 0; r < kLruMaxListRounds; ++r) {
        const int p = pg[r];
        if (p < 0) { sl[r] = -1; continue; }   // sl[r] becomes the table position of a miss, -1 otherwise
        const int s = sl[r];
        sl[r] = -1;
        if (s >= 0) {
            if (s < n_slots) { keyA[s] = step; tim[s] = step; }
        } else {
            int pos = (int)(((uint32_t)p * 2654435761u) >> tshift) & tmask;
            for (int probe = 0; probe < table; ++probe) {
                const int prev = atomicCAS(&tkey[pos], -1, p);
                if (prev == -1 || prev == p) {
                    atomicMin(&tval[pos], r * kLruThreads + tid);
                    sl[r] = pos;
                    break;
                }
                pos = (pos + 1) & tmask;
            }
        }
    }
    __syncthreads();

    // ---- 2. first appearances, ranked in list order -----------------------------------
    int n_miss = 0;
#pragma unroll
    for (int r = 0; r < kLruMaxListRounds; ++r) {
        if (r * kLruThreads < list_len) {
            const int f = (sl[r] >= 0) && (tval[sl[r]] == r * kLruThreads + tid);
            int total;
            const int j = n_miss + block_exclusive_scan(f, wsum, &total);
            if (f) mpage[j] = pg[r];
            n_miss += total;
        }
    }
    __syncthreads();  // the table is dead from here on; xbuf becomes keyB/valB

    const bool want_order = order_out != nullptr;
    const int n_miss_found = n_miss;
    if (n_miss > 0 || want_order) {
        // ---- 3. stable radix sort of the slots by access time --------------------
        {
            int mx = 0;
            for (int s = tid; s < n_slots; s += kLruThreads) mx = max(mx, keyA[s]);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) mx = max(mx, __shfl_xor_sync(DA_FULL_MASK, mx, off));
            if (lane == 0) atomicMax(&sh_max, mx);
        }
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
        const bool overflow =
            n_miss > 0 && ((n_miss > n_slots) || (kin[min(n_miss, n_slots) - 1] >= step));
        if (overflow) {
            if (tid == 0) atomicOr(status, DA_STATUS_LRU_OVERFLOW);
            n_miss = 0;  // tables stay as after the hit marking
        } else {
            for (int j = tid; j < n_miss; j += kLruThreads) {
                const int p = mpage[j];
                const int v = vin[j];
                const int old = s2d_s[v];
                if (old >= 0 && old < n_dram_pages) d2s[old] = -1;
                s2d[v] = p;
                d2s[p] = v;
                tim[v] = step;
                mp_out[j] = p;
                ms_out[j] = v;
                if (src_map) src_map[v] = p;
            }
        }

        // ---- 5. which slots can be evicted by the NEXT call -------------------------------
        // Sorted order now: [victims | untouched slots by (time, slot) | slots hit this call].
        // After this call victims and hits carry the newest stamp, so the next call's victims
        // come from the front of the untouched run, and no further in than the next list is
        // long (every list entry is either a hit, which removes a slot from the front, or a
        // miss, which takes one).  If the untouched run is at least list_len long, those
        // list_len slots are the only candidates; order_out = that run first, everything else
        // after it (a rotation of the sorted order by n_miss).  Otherwise every slot is a
        // candidate.
        if (want_order) {
            int touched = 0;  // slots hit by this call (sorted keys still hold the pre-assignment times)
            for (int i = tid; i < n_slots; i += kLruThreads) touched += (kin[i] >= step);
            int total;
            block_exclusive_scan(touched, wsum, &total);
            const int untouched = n_slots - total - n_miss;
            const int cap = min(list_len, n_slots);
            const bool bounded = !overflow && n_miss_found == n_miss && untouched >= cap;
            int32_t *ord = order_out + (size_t)h * n_slots;
            for (int i = tid; i < n_slots; i += kLruThreads) {
                int src = i + n_miss;
                if (src >= n_slots) src -= n_slots;
                ord[i] = vin[src];
            }
            if (tid == 0) n_evictable_out[h] = bounded ? cap : n_slots;
        }
    }
    if (tid == 0) {
        n_miss_out[h] = n_miss;
        step_counters[h] = step;
    }
}

static size_t lru_smem_bytes(int n_slots, int list_len) {
    const int table = lru_table_size(list_len);
    const int xhalf = n_slots > table ? n_slots : table;
    return ((size_t)3 * n_slots + 2 * (size_t)xhalf + list_len + 256 * kLruWarps) * sizeof(int);
}

constexpr size_t kLruMaxSmem = 227 * 1024 - 1024;

}  // namespace da

extern "C" int da_lru_update(const int32_t *page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                             int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step,
                             int n_kv_heads, int32_t *miss_pages, int32_t *miss_slots, int32_t *n_miss,
                             int32_t *slot_source, int32_t *order_out, int32_t *n_evictable_out,
                             int32_t *status, da_stream_t stream) {
    if (!page_list || !dram_to_slot || !slot_to_dram || !access_time || !step || !miss_pages || !miss_slots ||
        !n_miss || !status)
        return DA_ERR_NULL;
    if (list_len < 1 || n_dram_pages < 1 || n_slots < 1 || n_kv_heads < 1) return DA_ERR_SHAPE;
    if ((order_out == nullptr) != (n_evictable_out == nullptr)) return DA_ERR_NULL;
    if (n_slots > da::kLruMaxSlots || list_len > da::kLruMaxList) return DA_ERR_UNSUPPORTED;
    const size_t smem = da::lru_smem_bytes(n_slots, list_len);
    if (smem > da::kLruMaxSmem) return DA_ERR_UNSUPPORTED;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DA_ERR_UNSUPPORTED;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(da::lru_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)da::kLruMaxSmem);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    da::lru_update_kernel<<<n_kv_heads, da::kLruThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        page_list, list_len, dram_to_slot, n_dram_pages, slot_to_dram, access_time, n_slots, step, miss_pages,
        miss_slots, n_miss, slot_source, order_out, n_evictable_out, status);
    return (int)cudaGetLastError();
}

// LRU slot-table update: one CTA per KV head does, in one launch, what the
// reference does with a marking kernel, a library sort and a serial walk.
//
//   1. hits: every listed page that is resident gets time = step.
//   2. misses: the first appearance (in list order) of every non-resident page is
//      found with a shared-memory hash table keyed by page id that keeps the
//      smallest list index, and ranked by a block prefix sum.
//   3. victims: the n_miss slots with the smallest (time, slot).  No sort: a radix
//      select on the time finds the time T of the n_miss-th slot, every slot with
//      time < T is a victim, and the slots with time == T fill the rest in slot order
//      (an ordered block scan); the victims are then ranked among themselves by
//      counting.  One 8-bit select pass per byte of the step counter.
//   4. the j-th miss takes the j-th victim; tables updated; (page, slot) pairs
//      emitted for the payload copy.
//   5. optionally (two-launch attention) the eviction FRONT: the same select, for position
//      n_miss + split_cap, names the slots that are first in eviction order after this call;
//      and the call reports whether one of its own victims lay outside the front that was
//      current when it ran (the attention then redoes that head).

#include "da_common.cuh"

namespace da {

constexpr int kLruThreads = 1024;
constexpr int kLruWarps = kLruThreads / 32;
constexpr int kLruMaxSlots = 8192;
constexpr int kLruMaxList = 8192;

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

__host__ __device__ inline int lru_table_size(int list_len) {
    int t = 64;
    while (t < 2 * list_len) t <<= 1;
    return t;
}

// Time T of the slot at position `need` (1-based) in ascending time order, and how many slots
// have a smaller time.  tm[] holds the times of this thread's slots (slot r * 1024 + tid), -1
// for none.  8-bit radix select from the top byte of `bits` down.  hist2 = 2 x 256 ints of shared
// memory, res = 2 ints.  All threads call; contains barriers.
template <int SR>
__device__ __forceinline__ void select_time(const int (&tm)[SR], int need, int bits, int *hist2, int *res,
                                            int &t_out, int &less_out) {
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int passes = (bits + 7) / 8;
    uint32_t prefix = 0, mask = 0;
    int less = 0;
    if (tid < 256) hist2[tid] = 0;
    __syncthreads();
    for (int pass = passes - 1, buf = 0; pass >= 0; --pass, buf ^= 1) {
        const int shift = 8 * pass;
        int *hist = hist2 + 256 * buf;
        // the other histogram was last read before the previous pass's final barrier: clear it now for
        // the next pass, so that a pass costs two barriers
        if (tid < 256) hist2[256 * (buf ^ 1) + tid] = 0;
#pragma unroll
        for (int r = 0; r < SR; ++r) {
            const bool in = tm[r] >= 0 && ((uint32_t)tm[r] & mask) == prefix;
            const uint32_t digit = ((uint32_t)tm[r] >> shift) & 255u;
            // stamps cluster on the last few steps: count the lanes that share the first
            // participating lane's digit with one atomic, the others one by one
            const uint32_t act = __ballot_sync(DA_FULL_MASK, in);
            if (act) {
                const int first = __ffs(act) - 1;
                const uint32_t d0 = __shfl_sync(DA_FULL_MASK, digit, first);
                const uint32_t same = __ballot_sync(DA_FULL_MASK, in && digit == d0);
                if (lane == first) atomicAdd(&hist[d0], __popc(same));
                else if (in && digit != d0) atomicAdd(&hist[digit], 1);
            }
        }
        __syncthreads();
        if (warp == 0) {
            // lane l owns digits 8l .. 8l+7 (ascending): find where the running count reaches `need`
            int c[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                c[j] = hist[lane * 8 + j];
                tot += c[j];
            }
            int incl = tot;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int v = __shfl_up_sync(DA_FULL_MASK, incl, off);
                if (lane >= off) incl += v;
            }
            int below = incl - tot;
            const int want = need - less;
            if (below < want && incl >= want) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (below < want && below + c[j] >= want) {
                        res[0] = lane * 8 + j;
                        res[1] = below;
                        below = want;
                    } else {
                        below += c[j];
                    }
                }
            }
        }
        __syncthreads();
        prefix |= (uint32_t)res[0] << shift;
        mask |= 255u << shift;
        less += res[1];
        // (no barrier: res[] is next written after the next pass's histogram barrier)
    }
    __syncthreads();   // the caller may reuse hist2 / res right away
    t_out = (int)prefix;
    less_out = less;
}

// SR = slots per thread (n_slots <= SR * 1024), LR = list entries per thread.
template <int SR, int LR>
__global__ void __launch_bounds__(kLruThreads)
lru_update_kernel(const int32_t *__restrict__ page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                  int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step_counters,
                  int32_t *__restrict__ miss_pages, int32_t *__restrict__ miss_slots,
                  int32_t *__restrict__ n_miss_out, int32_t *slot_source, int32_t *order_out,
                  int32_t *n_evictable_out, int32_t *split_flip, int32_t *split_redo, int split_cap,
                  int split_advance, int32_t *status) {
    extern __shared__ __align__(16) int smem_i[];
    const int table = lru_table_size(list_len);
    int *tkey = smem_i;                  // [table] page id or -1; later: victim slots by rank
    int *tval = tkey + table;            // [table] smallest list index of that page
    int *tsm = tval + table;             // [n_slots] access times (hits already stamped)
    int *s2d_s = tsm + n_slots;          // [n_slots] slot -> page before this step
    int *mpage = s2d_s + n_slots;        // [list_len] miss pages in list order
    int *vtime = mpage + list_len;       // [list_len] victims: time
    int *vslot = vtime + list_len;       // [list_len] victims: slot
    unsigned char *in_front = reinterpret_cast<unsigned char *>(vslot + list_len);   // [n_slots] slot is in the current front
    __shared__ int wsum[kLruWarps];
    __shared__ int hist[512];
    __shared__ int res[2];
    __shared__ int sh_max;
    __shared__ int sh_redo;

    const int h = blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int32_t *list = page_list + (size_t)h * list_len;
    int32_t *d2s = dram_to_slot + (size_t)h * n_dram_pages;
    int32_t *s2d = slot_to_dram + (size_t)h * n_slots;
    int32_t *tim = access_time + (size_t)h * n_slots;
    int32_t *mp_out = miss_pages + (size_t)h * list_len;
    int32_t *ms_out = miss_slots + (size_t)h * list_len;

    // ---- all independent global reads first ---------------------------------------------
    int tm[SR], sd[SR];
#pragma unroll
    for (int r = 0; r < SR; ++r) {
        const int s = r * kLruThreads + tid;
        tm[r] = -1;
        sd[r] = -1;
        if (s < n_slots) {
            tm[r] = tim[s];
            sd[r] = s2d[s];
        }
    }
    int pg[LR], sl[LR];
    int bad = 0;
#pragma unroll
    for (int r = 0; r < LR; ++r) {
        const int i = r * kLruThreads + tid;
        pg[r] = -1;
        if (i < list_len) {
            const int p = list[i];
            if (p < 0 || p >= n_dram_pages) bad = 1; else pg[r] = p;
        }
    }
    const int step = step_counters[h] + 1;
    const int prev_miss = min(n_miss_out[h], list_len);
    // the eviction front the attention launch beside this update works from
    const bool want_order = order_out != nullptr;
    const int cur = want_order ? (split_flip[h] & 1) : 0;
    const int32_t *front_cur = want_order ? order_out + ((size_t)cur * gridDim.x + h) * n_slots : nullptr;
    const int n_front = want_order ? min(max(n_evictable_out[(size_t)cur * gridDim.x + h], 0), n_slots) : n_slots;
#pragma unroll
    for (int r = 0; r < LR; ++r) sl[r] = pg[r] >= 0 ? d2s[pg[r]] : 0;

    // slot_source[slot] = DRAM page whose payload still has to be brought into the slot, -1
    // otherwise: forget the marks of the previous call (its miss list is still in ms_out)
    int32_t *src_map = slot_source ? slot_source + (size_t)h * n_slots : nullptr;
    if (src_map) {
        for (int j = tid; j < prev_miss; j += kLruThreads) {
            const int v = ms_out[j];
            if (v >= 0 && v < n_slots) src_map[v] = -1;
        }
    }
#pragma unroll
    for (int r = 0; r < SR; ++r) {
        const int s = r * kLruThreads + tid;
        if (s < n_slots) {
            tsm[s] = tm[r];
            s2d_s[s] = sd[r];
        }
    }
    for (int x = tid; x < table; x += kLruThreads) {
        tkey[x] = -1;
        tval[x] = 0x7fffffff;
    }
    for (int x = tid; x < n_slots; x += kLruThreads) in_front[x] = n_front >= n_slots;
    if (tid == 0) {
        sh_max = step;
        sh_redo = 0;
    }
    if (bad) atomicOr(status, DA_STATUS_BAD_PAGE_ID);
    __syncthreads();
    if (n_front < n_slots) {
        for (int x = tid; x < n_front; x += kLruThreads) {
            const int v = front_cur[x];
            if (v >= 0 && v < n_slots) in_front[v] = 1;
        }
    }

    // ---- 1. hits get the step; non-resident pages go into the hash table -------------
    const int tmask = table - 1;
    const int tshift = 32 - (__ffs(table) - 1);
#pragma unroll
    for (int r = 0; r < LR; ++r) {
        const int p = pg[r];
        if (p < 0) { sl[r] = -1; continue; }   // sl[r] becomes the table position of a miss, -1 otherwise
        const int s = sl[r];
        sl[r] = -1;
        if (s >= 0) {
            if (s < n_slots) { tsm[s] = step; tim[s] = step; }
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

    // ---- 2. first appearances, ranked in list order; times with the hits applied --------
    int n_miss = 0;
#pragma unroll
    for (int r = 0; r < LR; ++r) {
        if (r * kLruThreads < list_len) {
            const int f = (sl[r] >= 0) && (tval[sl[r]] == r * kLruThreads + tid);
            int total;
            const int j = n_miss + block_exclusive_scan(f, wsum, &total);
            if (f) mpage[j] = pg[r];
            n_miss += total;
        }
    }
    int hits = 0, mx = 0;
#pragma unroll
    for (int r = 0; r < SR; ++r) {
        const int s = r * kLruThreads + tid;
        if (s < n_slots) {
            tm[r] = tsm[s];
            hits += (tm[r] >= step);
            mx = max(mx, tm[r]);
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mx = max(mx, __shfl_xor_sync(DA_FULL_MASK, mx, off));
    if (lane == 0) atomicMax(&sh_max, mx);
    {
        int total;
        block_exclusive_scan(hits, wsum, &total);   // also orders the atomicMax and the table's last use
        hits = total;
    }
    const int bits = 32 - __clz(sh_max | 1);
    const int n_found = n_miss;

    // ---- 3. victims ------------------------------------------------------------------------
    bool victim[SR];
#pragma unroll
    for (int r = 0; r < SR; ++r) victim[r] = false;
    bool overflow = false;
    if (n_miss > 0) {
        overflow = n_miss > n_slots - hits;   // victims must not have been touched by this call
        if (overflow) {
            if (tid == 0) atomicOr(status, DA_STATUS_LRU_OVERFLOW);
            n_miss = 0;  // tables stay as after the hit marking
        } else {
            int t1, less1;
            select_time<SR>(tm, n_miss, bits, hist, res, t1, less1);
            int run_lt = 0, run_eq = 0;   // slots seen so far (in slot order) with time < t1, == t1
#pragma unroll
            for (int r = 0; r < SR; ++r) {
                if (r * kLruThreads < n_slots) {
                    const int lt = tm[r] >= 0 && tm[r] < t1;
                    const int eq = tm[r] == t1;
                    int total;
                    const int ex = block_exclusive_scan(lt | (eq << 16), wsum, &total);
                    const int lt_rank = run_lt + (ex & 0xffff);
                    const int eq_rank = run_eq + (ex >> 16);
                    if (lt) {
                        victim[r] = true;
                        vtime[lt_rank] = tm[r];
                        vslot[lt_rank] = r * kLruThreads + tid;
                    } else if (eq && less1 + eq_rank < n_miss) {
                        victim[r] = true;
                        tkey[less1 + eq_rank] = r * kLruThreads + tid;   // already in final position
                    }
                    run_lt += total & 0xffff;
                    run_eq += total >> 16;
                }
            }
            __syncthreads();
            // the less1 victims older than t1 still have to be ordered by (time, slot)
            for (int j = tid; j < less1; j += kLruThreads) {
                const int kt = vtime[j], ks = vslot[j];
                int rank = 0;
                for (int i = 0; i < less1; ++i) {
                    const int it = vtime[i], is = vslot[i];
                    rank += (it < kt) || (it == kt && is < ks);
                }
                tkey[rank] = ks;
            }
            __syncthreads();

            // ---- 4. the j-th miss takes the j-th victim --------------------------------------
            for (int j = tid; j < n_miss; j += kLruThreads) {
                const int p = mpage[j];
                const int v = tkey[j];
                const int old = s2d_s[v];
                if (old >= 0 && old < n_dram_pages) d2s[old] = -1;
                s2d[v] = p;
                d2s[p] = v;
                tim[v] = step;
                mp_out[j] = p;
                ms_out[j] = v;
                if (src_map) src_map[v] = p;
                if (!in_front[v]) sh_redo = 1;   // evicted a slot the attention beside us is reading
            }
        }
    }

    // ---- 5. the eviction front after this call -------------------------------------------------
    // In (time, slot) order the slots are now [victims | untouched | hit by this call].  After
    // this call victims and hits carry the newest stamp, so the next call's victims come from the
    // front of the untouched run: how far in depends on how many of those slots it hits and how
    // many pages it misses.  The first split_cap slots of the run are written as the new front
    // (order_out = those first, every other slot after them); the next call checks its victims
    // against it (sh_redo above).  With fewer than split_cap untouched slots every slot is in the front.
    if (want_order) {
        // two buffers, [2][n_kv_heads][...]: the one split_flip[h] does NOT name is written
        const int wbuf = 1 - cur;
        int32_t *ord = order_out + ((size_t)wbuf * gridDim.x + h) * n_slots;
        const int cap = min(max(split_cap, 0), n_slots);
        const int untouched = n_slots - hits - n_miss;
        const bool bounded = !overflow && n_found == n_miss && untouched >= cap && cap > 0 && cap < n_slots;
        if (bounded) {
            int t2, less2;
            select_time<SR>(tm, n_miss + cap, bits, hist, res, t2, less2);   // tm: times before assignment
            int run_eq = 0, run_e = 0;
#pragma unroll
            for (int r = 0; r < SR; ++r) {
                if (r * kLruThreads < n_slots) {
                    const int s = r * kLruThreads + tid;
                    const int eq = tm[r] == t2;
                    int total;
                    const int eq_rank = run_eq + block_exclusive_scan(eq, wsum, &total);
                    run_eq += total;
                    const bool front = tm[r] >= 0 && (tm[r] < t2 || (eq && less2 + eq_rank < n_miss + cap));
                    const int e = front && !victim[r];
                    const int e_before = run_e + block_exclusive_scan(e, wsum, &total);
                    run_e += total;
                    if (s < n_slots) ord[e ? e_before : cap + (s - e_before)] = s;
                }
            }
        } else {
            for (int s = tid; s < n_slots; s += kLruThreads) ord[s] = s;
        }
        if (tid == 0) n_evictable_out[(size_t)wbuf * gridDim.x + h] = bounded ? cap : n_slots;
    }
    __syncthreads();   // sh_redo
    if (tid == 0) {
        n_miss_out[h] = n_miss;
        step_counters[h] = step;
        if (want_order) {
            split_redo[h] = sh_redo;
            if (split_advance) split_flip[h] = 1 - cur;
        }
    }
}

static size_t lru_smem_bytes(int n_slots, int list_len) {
    return ((size_t)2 * lru_table_size(list_len) + 2 * (size_t)n_slots + 3 * (size_t)list_len) * sizeof(int) +
           (((size_t)n_slots + 15) & ~(size_t)15);
}

constexpr size_t kLruMaxSmem = 227 * 1024 - 4096;

template <int SR, int LR>
static cudaError_t launch_lru(const int32_t *page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                              int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step,
                              int n_kv_heads, int32_t *miss_pages, int32_t *miss_slots, int32_t *n_miss,
                              int32_t *slot_source, int32_t *order_out, int32_t *n_evictable_out,
                              int32_t *split_flip, int32_t *split_redo, int split_cap, int split_advance,
                              int32_t *status, size_t smem, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(lru_update_kernel<SR, LR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kLruMaxSmem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    lru_update_kernel<SR, LR><<<n_kv_heads, kLruThreads, smem, stream>>>(
        page_list, list_len, dram_to_slot, n_dram_pages, slot_to_dram, access_time, n_slots, step, miss_pages,
        miss_slots, n_miss, slot_source, order_out, n_evictable_out, split_flip, split_redo, split_cap,
        split_advance, status);
    return cudaGetLastError();
}

}  // namespace da

extern "C" int da_lru_update(const int32_t *page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                             int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step,
                             int n_kv_heads, int32_t *miss_pages, int32_t *miss_slots, int32_t *n_miss,
                             int32_t *slot_source, int32_t *order_out, int32_t *n_evictable_out,
                             int32_t *split_flip, int32_t *split_redo, int split_cap, int split_advance,
                             int32_t *status, da_stream_t stream) {
    if (!page_list || !dram_to_slot || !slot_to_dram || !access_time || !step || !miss_pages || !miss_slots ||
        !n_miss || !status)
        return DA_ERR_NULL;
    if (list_len < 1 || n_dram_pages < 1 || n_slots < 1 || n_kv_heads < 1) return DA_ERR_SHAPE;
    if ((order_out == nullptr) != (n_evictable_out == nullptr) || (order_out == nullptr) != (split_flip == nullptr) ||
        (order_out == nullptr) != (split_redo == nullptr))
        return DA_ERR_NULL;
    if (n_slots > da::kLruMaxSlots || list_len > da::kLruMaxList) return DA_ERR_UNSUPPORTED;
    const size_t smem = da::lru_smem_bytes(n_slots, list_len);
    if (smem > da::kLruMaxSmem) return DA_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
#define DA_LRU_ARGS page_list, list_len, dram_to_slot, n_dram_pages, slot_to_dram, access_time, n_slots, step, \
                    n_kv_heads, miss_pages, miss_slots, n_miss, slot_source, order_out, n_evictable_out, split_flip, \
                    split_redo, split_cap, split_advance, status, smem, s
    if (n_slots <= 2048 && list_len <= 1024) e = da::launch_lru<2, 1>(DA_LRU_ARGS);
    else if (n_slots <= 4096 && list_len <= 2048) e = da::launch_lru<4, 2>(DA_LRU_ARGS);
    else e = da::launch_lru<8, 8>(DA_LRU_ARGS);
#undef DA_LRU_ARGS
    return (int)e;
}

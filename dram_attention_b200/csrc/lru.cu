// LRU slot-table update: one CTA per KV head does, in one launch, what the
// reference does with a marking kernel, a library sort and a serial walk.
//
//   1. hits: every listed page that is resident gets time = step.
//   2. misses: the first appearance (in list order) of every non-resident page is
//      found with a shared-memory hash table keyed by page id that keeps the
//      smallest list index, and ranked by a block prefix sum.
//   3. victims: the n_miss slots with the smallest (time, slot).
//   4. the j-th miss takes the j-th victim; tables updated; (page, slot) pairs
//      emitted for the payload copy.
//
// Two kernels, which differ in step 3:
//
//   lru_queue_kernel   the caller keeps the slots of every head as a QUEUE in eviction order
//       ((time, slot) ascending; two copies, the call reads one and writes the other).  Slots
//       this call does not touch keep their relative order, and the touched ones (hits and
//       victims) all get the newest stamp, i.e. go to the back in slot order.  So the victims are
//       simply the first n_miss untouched slots of the queue, and the new queue is a stable
//       partition: two rounds of block prefix sums, no sort, no select, and the timestamps are
//       never read.  The front of the new queue is what the NEXT call will evict from: the
//       two-launch attention leaves the first `split_cap` slots to its second launch, and this
//       call reports (redo) when one of its own victims lay beyond the front that was current.
//       When only a few pages miss, the kernel also copies them from DRAM (pinned host memory)
//       into their slots itself; the loads are issued before the second round of prefix sums, so
//       the host-link latency hides behind it.
//   lru_update_kernel  no queue: an 8-bit radix select on the time finds the time T of the
//       n_miss-th slot, every slot with time < T is a victim, the slots with time == T fill the
//       rest in slot order (an ordered block scan), and the victims older than T are ranked
//       among themselves by counting.

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

// Exclusive ranks of SR flags per thread, flags ordered r-major (all of r = 0 across the block, then
// r = 1, ...), two r at a time packed into one scan (counts stay below 2^16: at most 8192 slots).
template <int SR>
__device__ __forceinline__ void block_scan_flags(const int (&flag)[SR], int (&ex)[SR], int *wsum, int &total_all) {
    int run = 0;
#pragma unroll
    for (int r = 0; r < SR; r += 2) {
        const int f1 = r + 1 < SR ? flag[r + 1] : 0;
        int total;
        const int e = block_exclusive_scan(flag[r] | (f1 << 16), wsum, &total);
        ex[r] = run + (e & 0xffff);
        run += total & 0xffff;
        if (r + 1 < SR) {
            ex[r + 1] = run + (e >> 16);
            run += total >> 16;
        }
    }
    total_all = run;
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

// Without a queue.  SR = slots per thread (n_slots <= SR * 1024), LR = list entries per thread.
template <int SR, int LR>
__global__ void __launch_bounds__(kLruThreads)
lru_update_kernel(const int32_t *__restrict__ page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                  int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step_counters,
                  int32_t *__restrict__ miss_pages, int32_t *__restrict__ miss_slots,
                  int32_t *__restrict__ n_miss_out, int32_t *slot_source, int32_t *status) {
    griddep_wait();   // the page list comes from the kernel before this one
    extern __shared__ __align__(16) int smem_i[];
    const int table = lru_table_size(list_len);
    int *tkey = smem_i;                  // [table] page id or -1; later: victim slots by rank
    int *tval = tkey + table;            // [table] smallest list index of that page
    int *tsm = tval + table;             // [n_slots] access times (hits already stamped)
    int *s2d_s = tsm + n_slots;          // [n_slots] slot -> page before this step
    int *mpage = s2d_s + n_slots;        // [list_len] miss pages in list order
    int *vtime = mpage + list_len;       // [list_len] victims: time
    int *vslot = vtime + list_len;       // [list_len] victims: slot
    __shared__ int wsum[kLruWarps];
    __shared__ int hist[512];
    __shared__ int res[2];
    __shared__ int sh_max;

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
#pragma unroll
    for (int r = 0; r < LR; ++r) sl[r] = pg[r] >= 0 ? d2s[pg[r]] : 0;

    // slot_source[slot] = DRAM page whose payload still has to be brought into the slot, -1
    // otherwise.  Rewritten by every call: -1 everywhere, then (after several barriers) the marks
    // of this call's misses.
    int32_t *src_map = slot_source ? slot_source + (size_t)h * n_slots : nullptr;
    if (src_map) {
        for (int x = tid; x < n_slots; x += kLruThreads) src_map[x] = -1;
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
    if (tid == 0) sh_max = step;
    if (bad) atomicOr(status, DA_STATUS_BAD_PAGE_ID);
    __syncthreads();

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
            }
        }
    }

    if (tid == 0) {
        n_miss_out[h] = n_miss;
        step_counters[h] = step;
    }
}


// With the eviction queue.  SR = slots per thread (n_slots <= SR * 1024), LR = list entries per thread.
//   queue      [2][n_kv_heads][n_slots]: copy flip[h] is read (slots in eviction order), the other written
//   n_front    [2][n_kv_heads]: how many slots at the head of the queue the attention leaves to its
//              second launch; written for the new queue
template <int SR, int LR>
__global__ void __launch_bounds__(kLruThreads)
lru_queue_kernel(const int32_t *__restrict__ page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                 int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step_counters,
                 int32_t *__restrict__ miss_pages, int32_t *__restrict__ miss_slots,
                 int32_t *__restrict__ n_miss_out, int32_t *slot_source, int32_t *queue, int32_t *n_front_io,
                 int32_t *split_flip, int32_t *split_redo, int split_cap, int split_advance,
                 const unsigned char *dram_pages, unsigned char *slots, unsigned long long page_bytes,
                 int inline_max, unsigned int stage_off, int32_t *status) {
    if (threadIdx.x == 0) trace_stamp(2, blockIdx.x, 0);
    // The CTA is on its SM while the kernel before it still runs (programmatic dependent launch).  When the
    // caller vouches that that kernel is the selection (split_advance bit 1: it writes nothing but the page
    // list, and it has itself waited for everything before it), all this kernel needs from it is the list:
    // its own tables, both copies of the queue, the pages of the queue's slots and the cleared work areas are
    // then ready when the list is.  Otherwise the kernel before it may still be writing any of those (another
    // update, an attention launch flipping the queue) and the wait comes first.
    const bool list_only = (split_advance & 2) != 0;
    if (!list_only) griddep_wait();
    extern __shared__ __align__(16) int smem_i[];
    const int table = lru_table_size(list_len);
    int *tkey = smem_i;                  // [table] page id or -1
    int *tval = tkey + table;            // [table] smallest list index of that page
    int *mpage = tval + table;           // [list_len] miss pages in list order
    int *vslot = mpage + list_len;       // [list_len] victims in queue order
    unsigned char *touched = reinterpret_cast<unsigned char *>(vslot + list_len);   // [n_slots] hit or victim
    // [inline_max pages] where the missed pages wait between their asynchronous copy from DRAM and their slots
    uint4 *stage = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(smem_i) + stage_off);
    __shared__ int wsum[kLruWarps];
    __shared__ int sh_redo;
    __shared__ __align__(8) uint64_t stage_bar;   // completion of the page copies into the staging area

    const int h = blockIdx.x;
    const int tid = threadIdx.x;
    const int32_t *list = page_list + (size_t)h * list_len;
    int32_t *d2s = dram_to_slot + (size_t)h * n_dram_pages;
    int32_t *s2d = slot_to_dram + (size_t)h * n_slots;
    int32_t *tim = access_time + (size_t)h * n_slots;
    int32_t *mp_out = miss_pages + (size_t)h * list_len;
    int32_t *ms_out = miss_slots + (size_t)h * list_len;
    if (tid == 0) {
        mbar_init(&stage_bar, 1);
        mbar_fence_init();
    }

    // ---- all independent global reads first (both copies of the queue, so that nothing waits for
    // the flip word) --------------------------------------------------------------------------
    const int32_t *q_a = queue + (size_t)h * n_slots;
    const int32_t *q_b = queue + ((size_t)gridDim.x + h) * n_slots;
    int qa[SR], qb[SR];
#pragma unroll
    for (int r = 0; r < SR; ++r) {
        const int i = r * kLruThreads + tid;
        qa[r] = i < n_slots ? q_a[i] : -1;
        qb[r] = i < n_slots ? q_b[i] : -1;
    }
    const int nf_a = n_front_io[h], nf_b = n_front_io[(size_t)gridDim.x + h];
    const int cur = split_flip[h] & 1;
    const int step = step_counters[h] + 1;
    int32_t *q_out = queue + ((size_t)(1 - cur) * gridDim.x + h) * n_slots;
    const int n_front = min(max(cur ? nf_b : nf_a, 0), n_slots);
    int qs[SR];
#pragma unroll
    for (int r = 0; r < SR; ++r) {
        const int v = cur ? qb[r] : qa[r];
        qs[r] = r * kLruThreads + tid < n_slots ? min(max(v, 0), n_slots - 1) : -1;
    }
    // the page held by the slots at the head of the queue, where the victims come from
    int sd[SR];
#pragma unroll
    for (int r = 0; r < SR; ++r) sd[r] = qs[r] >= 0 ? s2d[qs[r]] : -1;

    // slot_source is rewritten by every call: -1 everywhere, then (after several barriers) the
    // marks of this call's misses
    int32_t *src_map = slot_source ? slot_source + (size_t)h * n_slots : nullptr;
    if (src_map) {
        for (int x = tid; x < n_slots; x += kLruThreads) src_map[x] = -1;
    }
    for (int x = tid; x < table; x += kLruThreads) {
        tkey[x] = -1;
        tval[x] = 0x7fffffff;
    }
    for (int x = tid; x < n_slots; x += kLruThreads) touched[x] = 0;
    if (tid == 0) sh_redo = 0;

    if (list_only) griddep_wait();   // the page list comes from the kernel before this one
    if (threadIdx.x == 0) trace_stamp(2, blockIdx.x, 2);
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
#pragma unroll
    for (int r = 0; r < LR; ++r) sl[r] = pg[r] >= 0 ? d2s[pg[r]] : 0;
    if (bad) atomicOr(status, DA_STATUS_BAD_PAGE_ID);
    __syncthreads();
    griddep_launch_dependents();   // the kernel after this one may move onto the SMs and wait there

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
            if (s < n_slots) { touched[s] = 1; tim[s] = step; }
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

    // ---- 2. first appearances, ranked in list order ----------------------------------------
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

    // Few misses: the update copies the pages itself.  The pages are known now (not yet the slots they go
    // to), so they set out from DRAM here, one bulk copy (TMA) per page into shared memory (no thread holds
    // or waits for them), and are moved on to their slots at the very end: the host-link latency of up to
    // inline_max pages hides behind the rest of the update.
    const bool may_copy = dram_pages != nullptr && n_miss <= inline_max;
    const int vec_per_page = (int)(page_bytes / 16);
    const unsigned char *src_h = dram_pages + (size_t)h * n_dram_pages * page_bytes;
    unsigned char *dst_h = slots + (size_t)h * n_slots * page_bytes;
    const bool in_flight = may_copy && n_miss > 0;
    if (in_flight) {
        __syncthreads();   // mpage is complete
        if (tid == 0) {
            mbar_arrive_expect_tx(&stage_bar, (uint32_t)(n_miss * page_bytes));
            for (int j = 0; j < n_miss; ++j)
                bulk_copy_g2s(reinterpret_cast<unsigned char *>(stage) + (size_t)j * page_bytes,
                              src_h + (size_t)mpage[j] * page_bytes, (uint32_t)page_bytes, &stage_bar);
        }
    }

    // ---- 3. victims = the first n_miss slots of the queue that no hit touched ------------------
    int urank[SR];        // rank of this queue position among the untouched ones, or -1
    int n_untouched = 0;
    {
        int flag[SR];
#pragma unroll
        for (int r = 0; r < SR; ++r) flag[r] = qs[r] >= 0 && !touched[qs[r]];
        block_scan_flags<SR>(flag, urank, wsum, n_untouched);   // (its barriers also publish mpage)
#pragma unroll
        for (int r = 0; r < SR; ++r)
            if (!flag[r]) urank[r] = -1;
    }
    const bool copy_here = may_copy && n_miss <= n_untouched;   // (what was loaded for nothing is dropped)
    const int n_vec = copy_here ? n_miss * vec_per_page : 0;
    if (n_miss > n_untouched) {
        // more distinct non-resident pages than slots this call may evict: tables stay as after the hits
        if (tid == 0) atomicOr(status, DA_STATUS_LRU_OVERFLOW);
        n_miss = 0;
    }

    // ---- 4. the j-th miss takes the j-th victim; the other untouched slots keep their order ------
#pragma unroll
    for (int r = 0; r < SR; ++r) {
        if (urank[r] >= 0) {
            if (urank[r] < n_miss) {
                const int j = urank[r];
                const int v = qs[r];
                const int p = mpage[j];
                const int old = sd[r];
                if (old >= 0 && old < n_dram_pages) d2s[old] = -1;
                s2d[v] = p;
                d2s[p] = v;
                tim[v] = step;
                mp_out[j] = p;
                ms_out[j] = v;
                vslot[j] = v;
                touched[v] = 1;
                if (src_map && !copy_here) src_map[v] = p;           // the attention kernel brings the page in
                if (r * kLruThreads + tid >= n_front) sh_redo = 1;   // beyond the front the attention left out
            } else {
                q_out[urank[r] - n_miss] = qs[r];
            }
        }
    }
    __syncthreads();

    // ---- 5. the touched slots go to the back of the queue, in slot order ------------------------
    {
        int flag[SR], pos[SR], n_touched;
#pragma unroll
        for (int r = 0; r < SR; ++r) {
            const int s = r * kLruThreads + tid;
            flag[r] = s < n_slots && touched[s];
        }
        block_scan_flags<SR>(flag, pos, wsum, n_touched);
#pragma unroll
        for (int r = 0; r < SR; ++r)
            if (flag[r]) q_out[n_untouched - n_miss + pos[r]] = r * kLruThreads + tid;
    }

    // ---- 6. the copied pages go from shared memory to their slots --------------------------------
    if (in_flight) {
        // (waited for also when the pages are dropped: nothing may land in shared memory after the CTA has gone)
        const bool landed = mbar_wait_bounded(&stage_bar, 0);
        if (!landed && tid == 0) atomicOr(status, DA_STATUS_WAIT_TIMEOUT);
        if (landed && n_miss > 0) {   // (not after an overflow)
            for (int i = tid; i < n_vec; i += kLruThreads)
                *reinterpret_cast<uint4 *>(dst_h + (size_t)vslot[i / vec_per_page] * page_bytes + (size_t)(i % vec_per_page) * 16) = stage[i];
        }
    }
    if (tid == 0) {
        n_miss_out[h] = n_miss;
        step_counters[h] = step;
        const int cap = split_cap > 0 ? min(split_cap, n_slots) : n_slots;
        n_front_io[(size_t)(1 - cur) * gridDim.x + h] = cap;
        split_redo[h] = sh_redo;     // (the barrier after round 4 orders its writes before this read)
        // running totals, for whoever wants to watch the cache (posted: the CTA does not wait for the old values)
        if (n_miss) atomicAdd(split_redo + gridDim.x + h, n_miss);
        if (sh_redo) atomicAdd(split_redo + 2 * gridDim.x + h, sh_redo);
        if (split_advance & 1) split_flip[h] = 1 - cur;
    }
    if (g_trace_buf != nullptr) {
        __syncthreads();
        if (tid == 0) trace_stamp(2, blockIdx.x, 1);
    }
}

static size_t lru_smem_bytes(int n_slots, int list_len) {
    return ((size_t)2 * lru_table_size(list_len) + 2 * (size_t)n_slots + 3 * (size_t)list_len) * sizeof(int);
}

static size_t lru_queue_smem_bytes(int n_slots, int list_len) {
    return ((size_t)2 * lru_table_size(list_len) + 2 * (size_t)list_len) * sizeof(int) +
           (((size_t)n_slots + 15) & ~(size_t)15);   // a multiple of 16: the page staging area follows
}

constexpr size_t kLruMaxSmem = 227 * 1024 - 4096;

struct LruArgs {
    const int32_t *page_list; int list_len; int32_t *dram_to_slot; int n_dram_pages; int32_t *slot_to_dram;
    int32_t *access_time; int n_slots; int32_t *step; int n_kv_heads; int32_t *miss_pages; int32_t *miss_slots;
    int32_t *n_miss; int32_t *slot_source; int32_t *queue; int32_t *n_front; int32_t *split_flip;
    int32_t *split_redo; int split_cap; int split_advance; const unsigned char *dram_pages; unsigned char *slots;
    unsigned long long page_bytes; int inline_max; int32_t *status;
};

template <int SR, int LR>
static cudaError_t launch_lru(const LruArgs &a, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(lru_update_kernel<SR, LR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kLruMaxSmem);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(lru_queue_kernel<SR, LR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kLruMaxSmem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    if (a.queue) {
        const size_t tables = lru_queue_smem_bytes(a.n_slots, a.list_len);
        return launch_dependent(lru_queue_kernel<SR, LR>, dim3(a.n_kv_heads), dim3(kLruThreads),
                                tables + (size_t)a.inline_max * a.page_bytes, stream, a.page_list, a.list_len,
                                a.dram_to_slot, a.n_dram_pages, a.slot_to_dram, a.access_time, a.n_slots, a.step,
                                a.miss_pages, a.miss_slots, a.n_miss, a.slot_source, a.queue, a.n_front,
                                a.split_flip, a.split_redo, a.split_cap, a.split_advance, a.dram_pages, a.slots,
                                a.page_bytes, a.inline_max, (unsigned int)tables, a.status);
    }
    return launch_dependent(lru_update_kernel<SR, LR>, dim3(a.n_kv_heads), dim3(kLruThreads),
                            lru_smem_bytes(a.n_slots, a.list_len), stream, a.page_list, a.list_len,
                            a.dram_to_slot, a.n_dram_pages, a.slot_to_dram, a.access_time, a.n_slots, a.step,
                            a.miss_pages, a.miss_slots, a.n_miss, a.slot_source, a.status);
}

}  // namespace da

DA_DEFINE_TRACE_SETTER(trace_set_lru)

extern "C" int da_lru_update(const int32_t *page_list, int list_len, int32_t *dram_to_slot, int n_dram_pages,
                             int32_t *slot_to_dram, int32_t *access_time, int n_slots, int32_t *step,
                             int n_kv_heads, int32_t *miss_pages, int32_t *miss_slots, int32_t *n_miss,
                             int32_t *slot_source, int32_t *evict_queue, int32_t *front_count,
                             int32_t *split_flip, int32_t *split_redo, int split_cap, int split_advance,
                             const void *dram_pages, void *slots, size_t page_bytes, int inline_fetch_max,
                             int32_t *status, da_stream_t stream) {
    if (!page_list || !dram_to_slot || !slot_to_dram || !access_time || !step || !miss_pages || !miss_slots ||
        !n_miss || !status)
        return DA_ERR_NULL;
    if (list_len < 1 || n_dram_pages < 1 || n_slots < 1 || n_kv_heads < 1) return DA_ERR_SHAPE;
    if ((evict_queue == nullptr) != (front_count == nullptr) || (evict_queue == nullptr) != (split_flip == nullptr) ||
        (evict_queue == nullptr) != (split_redo == nullptr))
        return DA_ERR_NULL;
    if (n_slots > da::kLruMaxSlots || list_len > da::kLruMaxList) return DA_ERR_UNSUPPORTED;
    const size_t smem = evict_queue ? da::lru_queue_smem_bytes(n_slots, list_len) : da::lru_smem_bytes(n_slots, list_len);
    if (smem > da::kLruMaxSmem) return DA_ERR_UNSUPPORTED;
    // pages are copied by the update itself only with a queue, 16-byte granularity and both ends given
    const bool can_copy = evict_queue && dram_pages && slots && inline_fetch_max > 0 && page_bytes >= 16 &&
                          page_bytes % 16 == 0 && (((uintptr_t)dram_pages | (uintptr_t)slots) & 15) == 0;
    // the pages it copies wait in shared memory beside the tables: as many as fit
    if (can_copy) {
        const size_t room = (da::kLruMaxSmem - smem) / page_bytes;
        if ((size_t)inline_fetch_max > room) inline_fetch_max = (int)room;
    }
    da::LruArgs a{page_list, list_len, dram_to_slot, n_dram_pages, slot_to_dram, access_time, n_slots, step,
                  n_kv_heads, miss_pages, miss_slots, n_miss, slot_source, evict_queue, front_count, split_flip,
                  split_redo, split_cap, split_advance,
                  can_copy ? static_cast<const unsigned char *>(dram_pages) : nullptr,
                  can_copy ? static_cast<unsigned char *>(slots) : nullptr, (unsigned long long)page_bytes,
                  can_copy && inline_fetch_max > 0 ? inline_fetch_max : 0, status};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (n_slots <= 2048 && list_len <= 1024) e = da::launch_lru<2, 1>(a, s);
    else if (n_slots <= 4096 && list_len <= 2048) e = da::launch_lru<4, 2>(a, s);
    else e = da::launch_lru<8, 8>(a, s);
    return (int)e;
}

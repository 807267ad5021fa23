/*
 * dram_attention_b200 -- C ABI of the B200 (sm_100a) kernels behind the
 * generate stage of DRAM Attention.
 *
 * The reference project (long-context/dram-attention) is pure Python: it has no
 * FFI of its own.  Each entry point below therefore names the Python-level
 * function of the reference whose GPU work it replaces (file:line inside the
 * reference project); the Python package `dram_attention_b200` binds these with
 * ctypes and mirrors the reference's classes on top of them.
 *
 * Conventions
 *   - Every pointer is a raw address: device memory unless the parameter is
 *     documented as "host".  The library never allocates or frees device memory
 *     and never synchronises; every call only enqueues work on `stream`
 *     (a cudaStream_t passed as void*), so a sequence of calls can be captured
 *     in a CUDA graph.
 *   - Return value: 0 on success, a negative DA_ERR_* for an argument the host
 *     code rejected, a positive value = cudaError_t from the launch.
 *   - Conditions only the device can see (a page id out of range, more distinct
 *     pages requested than slots, a bounded wait that ran out) set bits in a
 *     caller-provided int32 status word; the kernels skip the offending access
 *     and keep running.
 *   - dtype codes: DA_F32, DA_F16, DA_BF16 (the element type of q/k/v, of the
 *     page summaries and of the page payloads).
 *   - Heads: query head hq belongs to KV head hq / rep (contiguous GQA groups).
 */
#ifndef DRAM_ATTENTION_B200_H
#define DRAM_ATTENTION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DA_F32 0
#define DA_F16 1
#define DA_BF16 2

#define DA_OK 0
#define DA_ERR_NULL (-1)        /* a required pointer is null */
#define DA_ERR_SHAPE (-2)       /* a size is zero, negative or inconsistent */
#define DA_ERR_DTYPE (-3)       /* unknown dtype code */
#define DA_ERR_ALIGN (-4)       /* a pointer or stride breaks the stated alignment */
#define DA_ERR_UNSUPPORTED (-5) /* valid, but outside what the kernels are built for */
#define DA_ERR_WORKSPACE (-6)   /* workspace smaller than the *_workspace_bytes value */
#define DA_ERR_STATIC_SCRATCH (-7) /* shape needs more scratch than the built-in buffer holds */

/* bits of the device status word */
#define DA_STATUS_BAD_PAGE_ID 1      /* a listed page id was outside [0, n_dram_pages) */
#define DA_STATUS_LRU_OVERFLOW 2     /* more distinct non-resident pages than evictable slots */
#define DA_STATUS_BAD_POSITION 4     /* start_pos - dram_tokens outside the local window */
#define DA_STATUS_WAIT_TIMEOUT 8     /* a bounded wait on an asynchronous copy ran out */

typedef void *da_stream_t;

#if defined(__GNUC__)
#define DA_API __attribute__((visibility("default")))
#else
#define DA_API
#endif

/* Library version: major * 10000 + minor * 100 + patch. */
DA_API int da_version(void);

/* Static, human-readable text for a return code of this library. */
DA_API const char *da_error_string(int code);

/*
 * Profiling switch (no counterpart in the reference).  While a buffer of da_trace_bytes() bytes
 * of device memory is set, thread 0 of every CTA of every kernel of this library writes the
 * GPU's global nanosecond timer into it at a few points: the buffer is
 * [6 kernels][1024 CTAs (index modulo)][4 events] of uint64, kernels 0 = page scorer,
 * 1 = selection, 2 = LRU update, 3 = attention (single launch or phase 1), 4 = attention phase 2,
 * 5 = gather of the head shards; events 0 = the CTA is on its SM, 1 = it is done, and for
 * selection, LRU update and gather 2 = the kernel before it in the stream has finished (they
 * are launched early and wait), for the attention 2 = its warps are through their units, 3 = its
 * ticket is taken, for the gather 3 = its rows are sent.  A launch overwrites
 * the stamps of the launch before it, so after a step the buffer holds that step's time line,
 * including the kernels that ran side by side on different streams.  da_trace_set(NULL)
 * switches it off (the default).  Applies to the current device; call it outside stream capture.
 */
DA_API size_t da_trace_bytes(void);
DA_API int da_trace_set(void *buffer);

/*
 * Page scorer.  Replaces max_inner_product()
 * (dram_attention/max_ip_triton_kernel.py:95-124, formula :72-80 and :127-133)
 * together with the GQA reshapes around it (dram_attention/topk_selector.py:48-59).
 *
 *   score[s, hq, l] = sum_d max(q[s,hq,d] * min[hk,l,d], q[s,hq,d] * max[hk,l,d]),
 *   hk = hq / rep, products and accumulation in float32.
 *
 * q          (n_tokens, n_kv_heads * rep, head_dim), contiguous, `dtype`
 * summaries  (n_kv_heads, n_pages, 2, head_dim), contiguous, `dtype`;
 *            [.., 0, :] = per-page channel minimum, [.., 1, :] = maximum
 * scores     (n_tokens, n_kv_heads * rep, n_pages) float32, written
 * summaries_ordered  non-zero promises min <= max in every channel (true for
 *            summaries built by da_build_pages); 16-bit types then take the tensor-core
 *            path.  Zero makes no assumption about the two rows (the reference's own
 *            value test feeds unordered rows).
 * The summaries are read once per token for all `rep` query heads of a KV head.
 */
DA_API int da_score_pages(const void *q, const void *summaries, float *scores,
                   int n_tokens, int n_kv_heads, int rep, int n_pages, int head_dim,
                   int dtype, int summaries_ordered, da_stream_t stream);

/*
 * Per-query-head top-k page selection, written directly as the per-KV-head page
 * list.  Replaces torch.argsort(ip, descending=True)[..., :k]
 * (dram_attention/topk_selector.py:61) and the list concatenation of
 * LRUCache.get_kv_cache_ (dram_attention/lru_cache.py:260-264).
 *
 * For every row (s, hq) the k pages with the largest score, in descending
 * score order, equal scores (including -0.0 and +0.0) in ascending page id.
 *
 * scores     (n_tokens, n_kv_heads * rep, n_pages) float32
 * page_list  (n_kv_heads, n_tokens * rep * k) int32, written:
 *            page_list[hk][(s * rep + r) * k + j] = j-th page of query head hk*rep+r
 * Requires 1 <= k <= n_pages and k <= 4096.
 */
DA_API int da_topk_pages(const float *scores, int32_t *page_list,
                  int n_tokens, int n_kv_heads, int rep, int n_pages, int k,
                  da_stream_t stream);

/*
 * The same selection with a hint on how many SMs it may count on.  Rows of more than 16 384 pages
 * (up to 65 536) are split over a thread-block cluster of four CTAs (partial histograms summed
 * through distributed shared memory, candidates collected in one CTA) when all clusters of the
 * launch find an SM per CTA at once: n_tokens * n_kv_heads * rep * 4 <= sm_budget.  A caller
 * that runs another launch beside the selection (the first attention launch of the two-launch
 * step keeps all but 32 SMs) passes what is left; 0 means the whole GPU, which is what
 * da_topk_pages passes.  The result does not depend on sm_budget.
 */
DA_API int da_topk_pages_wide(const float *scores, int32_t *page_list,
                       int n_tokens, int n_kv_heads, int rep, int n_pages, int k,
                       int sm_budget, da_stream_t stream);

/*
 * LRU slot-table update, one call for all KV heads.  Replaces load_lru_cache_()
 * without its payload copy: _update_page_access_time_
 * (dram_attention/lru_triton_kernel.py:110-137), the stable argsort of the
 * timestamps (:170) and the table part of _load_lru_cache_inline_kernel
 * (:30-78, :99-107), plus the step increment of LRUCache.load_
 * (dram_attention/lru_cache.py:224).
 *
 * Per head: step += 1; every listed page that is resident gets time = step; the
 * listed pages that are not resident, in order of first appearance, take the
 * slots with the smallest (time, slot); the evicted pages are unmapped.  The
 * result equals the reference's sequential walk whenever the distinct listed
 * pages fit in the slot table; otherwise DA_STATUS_LRU_OVERFLOW is set and the
 * tables of that head are left as after the hit marking.
 *
 * page_list   (n_kv_heads, list_len) int32
 * dram_to_slot(n_kv_heads, n_dram_pages) int32, -1 = not resident   (in/out)
 * slot_to_dram(n_kv_heads, n_slots) int32, -1 = empty slot           (in/out)
 * access_time (n_kv_heads, n_slots) int32, non-negative             (in/out)
 * step        (n_kv_heads) int32, one counter per head               (in/out)
 * miss_pages, miss_slots (n_kv_heads, list_len) int32, written: the (page, slot)
 *             pairs whose payload has to be copied, in list order
 * n_miss      (n_kv_heads) int32, written
 * slot_source optional (n_kv_heads, n_slots) int32 for da_decode_attention_fetch, rewritten by
 *             every call: slot_source[h][s] = the DRAM page that slot s was just given and
 *             whose payload is not in the slot yet, -1 for every other slot.  NULL when
 *             da_fetch_pages does the copy.
 * evict_queue, front_count, split_flip, split_redo  optional, all or none: the eviction queue that
 *             makes the update cheap and that da_decode_attention_phased works from.
 *             evict_queue is [2][n_kv_heads][n_slots] int32, front_count [2][n_kv_heads],
 *             split_flip [n_kv_heads], split_redo [3][n_kv_heads] (row 0 the flag described
 *             below; rows 1 and 2 running totals the call adds to: pages missed, calls that
 *             set the flag).  Copy split_flip[h] of evict_queue[.][h] is
 *             the CURRENT queue of head h: all its slots in eviction order, i.e. sorted by
 *             (access_time, slot) ascending; the first front_count entries are the FRONT, the
 *             slots an attention launch that runs beside this update has left out because they
 *             may be evicted.  The call
 *               - takes its victims from the head of the current queue (the first slots no listed
 *                 page hit), without reading access_time;
 *               - sets split_redo[h] = 1 if a victim lay beyond the current front (the attention
 *                 then has to redo the head), else 0;
 *               - writes the other copy: the untouched slots in their old order, then the slots
 *                 this call touched in slot order, with front_count = split_cap (n_slots when
 *                 split_cap <= 0);
 *               - with bit 0 of split_advance set makes that copy current itself (callers that run
 *                 no phased attention after the update); otherwise phase 2 of the attention does.
 *             Bit 1 of split_advance is a promise about the launch before this one in the stream: it
 *             is da_topk_pages (or anything else that writes none of this call's tables and has
 *             itself waited for its predecessors).  The kernel is launched as a programmatic
 *             dependent; with the promise it reads its tables and both queue copies while that
 *             launch still runs and waits only for the page list, without it it waits first.
 *             Before the first call: both copies = the slots sorted by (access_time, slot) (the
 *             identity when every time is zero), split_flip = 0, front_count at most n_slots.
 *             Without a queue the victims are found by a radix select on access_time.
 * dram_pages, slots, page_bytes, inline_fetch_max  optional (queue only): when a head misses at
 *             most inline_fetch_max pages, the call copies them from dram_pages (n_kv_heads,
 *             n_dram_pages, page_bytes; pinned, device-mapped host memory) into slots
 *             (n_kv_heads, n_slots, page_bytes) itself -- one bulk copy (TMA) per page into
 *             shared memory as soon as the missed pages are known, moved on to the slots at the
 *             end, so that the host-link latency overlaps the rest of the update; the wait is
 *             bounded (DA_STATUS_WAIT_TIMEOUT) -- and leaves their slot_source entries at -1.
 *             inline_fetch_max is lowered to what fits into shared memory beside the tables.
 *             page_bytes a multiple of 16, both bases 16-byte aligned.  NULL / 0: the pages are
 *             left to da_fetch_pages or to the attention kernel.
 * status      (1) int32, bits or-ed in
 * Requires n_slots <= 8192, list_len <= 8192 and the shared-memory plan to fit 222 KiB: with a
 * queue 2*T + 2*list_len ints + n_slots bytes, without 2*T + 2*n_slots + 3*list_len ints
 * (T = power of two >= 2*list_len); e.g. 8192 slots with lists up to 4096.
 * The kernel is launched so that it may move onto the SMs while the kernel before it in `stream`
 * is still running (it waits for that kernel's results before it reads anything).
 */
DA_API int da_lru_update(const int32_t *page_list, int list_len,
                  int32_t *dram_to_slot, int n_dram_pages,
                  int32_t *slot_to_dram, int32_t *access_time, int n_slots,
                  int32_t *step, int n_kv_heads,
                  int32_t *miss_pages, int32_t *miss_slots, int32_t *n_miss,
                  int32_t *slot_source, int32_t *evict_queue, int32_t *front_count,
                  int32_t *split_flip, int32_t *split_redo, int split_cap, int split_advance,
                  const void *dram_pages, void *slots, size_t page_bytes, int inline_fetch_max,
                  int32_t *status, da_stream_t stream);

/*
 * Miss-page fetch: gather-copy of the pages named by da_lru_update from DRAM into
 * their slots.  Replaces the payload loop of _load_lru_cache_inline_kernel
 * (dram_attention/lru_triton_kernel.py:81-98).
 *
 * dram_pages  (n_kv_heads, n_dram_pages, page_bytes): pinned, device-mapped HOST
 *             memory (or device memory); read with 128-bit loads by many CTAs
 * slots       (n_kv_heads, n_slots, page_bytes) device memory, written
 * miss_pages, miss_slots, n_miss: as written by da_lru_update (device memory; the
 *             host never reads them)
 * page_bytes  multiple of 16 with both bases 16-byte aligned for the fast path;
 *             any other size is copied bytewise.
 */
DA_API int da_fetch_pages(const void *dram_pages, void *slots,
                   const int32_t *miss_pages, const int32_t *miss_slots,
                   const int32_t *n_miss, int list_len,
                   int n_kv_heads, int n_dram_pages, int n_slots, size_t page_bytes,
                   da_stream_t stream);

/* Bytes of workspace da_decode_attention needs for this shape. */
DA_API size_t da_decode_attention_workspace_bytes(int n_kv_heads, int rep, int head_dim);

/*
 * Decode attention of one query token over the whole slot table and the local
 * window, with the append of the new key/value and the merge of the parts.
 * Replaces _compute_prefix_attention, _compute_suffix_attention and
 * _combine_attention (dram_attention/dram_attention.py:191-238), i.e. the two
 * flash_attn_with_kvcache calls and the log-sum-exp merge.
 *
 *   T = start_pos - dram_tokens; local_k[T] = new_k, local_v[T] = new_v;
 *   out[hq] = softmax over {all prefix tokens} U {local tokens 0..T} of
 *             (q[hq] . k / sqrt(head_dim)), applied to v; float32 softmax and
 *             accumulation; one split-K pass with a single final merge.
 *
 * q            (n_kv_heads * rep, head_dim) `dtype`
 * prefix_kv    (n_kv_heads, n_prefix_tokens, 2, head_dim) `dtype`: the slot table
 *              seen as tokens, key then value per token (page payload layout of
 *              dram_attention/lru_cache.py:121-142); head stride in elements
 * local_k/v    local window, token t of head h at t * local_token_stride +
 *              h * local_head_stride (elements); capacity local_capacity tokens
 * new_k/new_v  (n_kv_heads, head_dim) `dtype`
 * start_pos_dev  device int32[1], or NULL to use start_pos_host
 * out          (n_kv_heads * rep, head_dim) `dtype`, written
 * lse_out      optional (n_kv_heads * rep) float32: log-sum-exp of all logits
 * workspace    da_decode_attention_workspace_bytes() bytes, 256-byte aligned; the
 *              first 1024 bytes hold counters that must be ZERO before the first
 *              call; each call leaves them zero again
 * status       (1) int32, bits or-ed in
 * Requires head_dim in {64, 128}, rep <= 16 (8 for float32); all bases and strides
 * multiples of 16 bytes.
 */
DA_API int da_decode_attention(const void *q,
                        const void *prefix_kv, long long prefix_head_stride,
                        int n_prefix_tokens,
                        void *local_k, void *local_v,
                        long long local_token_stride, long long local_head_stride,
                        int local_capacity,
                        const void *new_k, const void *new_v,
                        const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                        void *out, float *lse_out,
                        void *workspace, size_t workspace_bytes, int32_t *status,
                        int n_kv_heads, int rep, int head_dim, int dtype,
                        da_stream_t stream);

/*
 * da_decode_attention for several query tokens in one call: the generate stage with
 * seq_len > 1 (dram_attention/dram_attention.py:144-177 with a (1, s, Hq, D) query; the
 * evaluation harness feeds the unaligned tail of a prompt this way).
 *
 *   T = start_pos - dram_tokens; local[T + i] = new_k/new_v[i] for the s tokens;
 *   query token i attends over the prefix tokens [0, n_prefix_tokens - (s - 1 - i)) and the
 *   local tokens [0, T + i]: both parts carry the bottom-right aligned causal mask that
 *   flash_attn_with_kvcache(causal=True) applies (dram_attention.py:195-205, :211-223) --
 *   on the prefix it hides the LAST s - 1 - i tokens of the slot table from token i, as the
 *   reference does.
 *
 * q, out       (n_q_tokens, n_kv_heads * rep, head_dim); new_k, new_v (n_q_tokens, n_kv_heads,
 *              head_dim); lse_out optional (n_q_tokens, n_kv_heads * rep)
 * workspace    da_decode_attention_tokens_workspace_bytes() bytes
 * One launch covers 16 / rep tokens for 16-bit types (8 / rep for float32); longer calls are
 * several launches on `stream`.  Requires rep <= 16 (8 for float32), n_q_tokens <= local_capacity.
 */
DA_API size_t da_decode_attention_tokens_workspace_bytes(int n_kv_heads, int rep, int head_dim,
                        int n_q_tokens);
DA_API int da_decode_attention_tokens(const void *q, int n_q_tokens,
                        const void *prefix_kv, long long prefix_head_stride,
                        int n_prefix_tokens,
                        void *local_k, void *local_v,
                        long long local_token_stride, long long local_head_stride,
                        int local_capacity,
                        const void *new_k, const void *new_v,
                        const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                        void *out, float *lse_out,
                        void *workspace, size_t workspace_bytes, int32_t *status,
                        int n_kv_heads, int rep, int head_dim, int dtype,
                        da_stream_t stream);

/*
 * da_decode_attention with the miss fetch folded in: replaces, in one launch, the payload
 * loop of _load_lru_cache_inline_kernel (dram_attention/lru_triton_kernel.py:81-98) and
 * the attention calls of dram_attention/dram_attention.py:191-238.
 *
 * The warp that attends over a 16-token unit of a slot marked in `slot_source` (written by
 * da_lru_update) reads that unit from the DRAM page instead (bulk copies from pinned host
 * memory, issued stages ahead so the host-link latency overlaps the other units), uses it,
 * and writes it through to the slot.  Every marked page is read from DRAM exactly once and
 * no separate da_fetch_pages launch is needed.
 *
 * slots        (n_kv_heads, n_slots, page_size, 2, head_dim) `dtype`, read AND written
 * dram_pages   (n_kv_heads, n_dram_pages, page_size, 2, head_dim): pinned, device-mapped
 *              host memory (or device memory), 16-byte aligned
 * slot_source  (n_kv_heads, n_slots) int32 as left by da_lru_update
 * Other arguments as da_decode_attention.  Requires page_size to be a multiple of 16;
 * otherwise DA_ERR_UNSUPPORTED (use da_fetch_pages + da_decode_attention).
 */
DA_API int da_decode_attention_fetch(const void *q,
                        void *slots, long long slots_head_stride, int n_slots, int page_size,
                        const void *dram_pages, int n_dram_pages, const int32_t *slot_source,
                        void *local_k, void *local_v,
                        long long local_token_stride, long long local_head_stride,
                        int local_capacity,
                        const void *new_k, const void *new_v,
                        const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                        void *out, float *lse_out,
                        void *workspace, size_t workspace_bytes, int32_t *status,
                        int n_kv_heads, int rep, int head_dim, int dtype,
                        da_stream_t stream);

/*
 * da_decode_attention_fetch as two launches, so that nearly all of the attention runs BESIDE
 * the scoring, the selection and the LRU update instead of after them (same reference lines
 * as da_decode_attention_fetch; the result is the same).
 *
 *   phase 1  (may run concurrently with da_score_pages / da_topk_pages / da_lru_update of the
 *            same step): appends the new key/value, attends over the local window and over
 *            every slot outside the current eviction front, writes partials.  By default at
 *            most 116 CTAs that each fill an SM, so 32 SMs stay free for the other kernels.
 *   phase 2  (directly after da_lru_update in the same stream; need NOT wait for phase 1; q,
 *            new_k, new_v and start_pos_dev must have been complete before that update was
 *            enqueued -- the launch overlaps it and reads them early): attends over the slots of the
 *            front, reading freshly assigned ones from DRAM as da_decode_attention_fetch
 *            does, and writes partials.  If the update set split_redo[h] (it had to evict a
 *            slot outside the front, e.g. after a query that shares nothing with the last
 *            one), phase 2 covers the whole head -- every slot and the local window -- and the
 *            rows phase 1 wrote for that head are ignored.
 *   The CTA of a head that finishes LAST, whichever launch it belongs to, merges the
 *   partials, writes the output, and flips split_flip[h], which makes the front the update
 *   wrote current.  Both launches of a step must have been enqueued before the next step's
 *   first one; a step is complete when both have finished.
 *
 * split_order, split_count, split_flip, split_redo   the evict_queue, front_count, split_flip and
 *            split_redo of da_lru_update (called with split_advance = 0 between the two launches).
 * phase1_ctas, phase2_ctas  CTAs per KV head of the two launches, the same values in both
 *            calls of a step; 0 = defaults (116 / n_kv_heads and 64 / n_kv_heads), at most 148.
 * workspace  da_decode_attention_phased_workspace_bytes() bytes, shared by both phases.
 */
DA_API size_t da_decode_attention_phased_workspace_bytes(int n_kv_heads, int rep, int head_dim);
/* 1 if da_decode_attention_phased accepts this shape (page_size a multiple of 16, the phase-1
 * CTA fits an SM's shared memory), else 0. */
DA_API int da_decode_attention_phased_supported(int n_kv_heads, int rep, int head_dim, int dtype,
                        int n_slots, int page_size, int local_capacity);
DA_API int da_decode_attention_phased(int phase, const int32_t *split_order, const int32_t *split_count,
                        int32_t *split_flip, const int32_t *split_redo,
                        int phase1_ctas, int phase2_ctas,
                        const void *q,
                        void *slots, long long slots_head_stride, int n_slots, int page_size,
                        const void *dram_pages, int n_dram_pages, const int32_t *slot_source,
                        void *local_k, void *local_v,
                        long long local_token_stride, long long local_head_stride,
                        int local_capacity,
                        const void *new_k, const void *new_v,
                        const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                        void *out, float *lse_out,
                        void *workspace, size_t workspace_bytes, int32_t *status,
                        int n_kv_heads, int rep, int head_dim, int dtype,
                        da_stream_t stream);

/*
 * da_decode_attention for callers that cannot hand over a workspace.  (No counterpart
 * in the reference; it does not change what is computed.)
 *
 * Some hosts of this library may not allocate device memory once they are running:
 * a serving process whose memory plan is frozen after start-up, a plugin loaded into
 * a runtime that owns the allocator, code that is entered while the application holds
 * a capture or a lock under which cudaMalloc is off limits.  For them this variant
 * keeps the kernel's scratch (ticket counters and split partials) in a buffer that is
 * part of the library image: da_decode_attention_static_capacity() bytes (2 MiB),
 * resident on every GPU that loads the library until the process exits.  The call
 * allocates nothing and calls no allocating routine.
 *
 * Arguments and result are those of da_decode_attention without workspace and
 * workspace_bytes.  Differences to know about:
 *   - shapes whose workspace (da_decode_attention_workspace_bytes) exceeds the
 *     capacity are rejected with DA_ERR_STATIC_SCRATCH;
 *   - the first call on a device looks up the buffer's device address (a host-side
 *     runtime query); make that first call outside any stream capture;
 *   - every call clears the counters it needs on `stream` before the kernel, so a
 *     previous call's leftovers cannot leak in;
 *   - there is ONE buffer per GPU: two calls that may run at the same time on one GPU
 *     (different streams, different threads, different operator instances) race on
 *     it.  Serialise them, or use da_decode_attention with a workspace per caller.
 */
DA_API size_t da_decode_attention_static_capacity(void);
DA_API int da_decode_attention_static(const void *q,
                        const void *prefix_kv, long long prefix_head_stride,
                        int n_prefix_tokens,
                        void *local_k, void *local_v,
                        long long local_token_stride, long long local_head_stride,
                        int local_capacity,
                        const void *new_k, const void *new_v,
                        const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                        void *out, float *lse_out, int32_t *status,
                        int n_kv_heads, int rep, int head_dim, int dtype,
                        da_stream_t stream);

/*
 * Cache construction on the device: splits a prefill K/V into DRAM pages, page
 * summaries and warm-started slots in one pass.  Replaces the torch code of
 * IPUpperboundTopKSelector.__init__ (dram_attention/topk_selector.py:24-35) and
 * of LRUCache.__init__ (dram_attention/lru_cache.py:121-153, :192-209).
 *
 * k, v        token t of head h at t * kv_token_stride + h * kv_head_stride
 *             (elements), n_pages * page_size tokens are read
 * dram_pages  optional (n_kv_heads, n_pages, page_size, 2, head_dim): pinned,
 *             device-mapped HOST memory (or device memory), written
 * summaries   optional (n_kv_heads, n_pages, 2, head_dim), written
 * slots       optional (n_kv_heads, n_slots, page_size, 2, head_dim), written with
 *             the last n_slots pages (slot s <- page n_pages - n_slots + s)
 */
DA_API int da_build_pages(const void *k, const void *v,
                   long long kv_token_stride, long long kv_head_stride,
                   void *dram_pages, void *summaries, void *slots,
                   int n_kv_heads, int n_pages, int n_slots, int page_size, int head_dim,
                   int dtype, da_stream_t stream);

/*
 * Rotary position embedding of the new queries and keys: the caller-side step in front of the
 * operator call, apply_rotary_emb (evaluation/dram-attention/model.py:125-135, called at :201;
 * freqs_cis as precompute_freqs_cis :105-114 makes it and Transformer.forward slices it to the
 * call's positions).  Adjacent channels (2i, 2i+1) of every head are one complex number that
 * is multiplied by freqs_cis[token][i]; fp32 arithmetic with each product and the sum rounded
 * once, as a complex64 multiply, then rounding to the tensors' type.  One launch for q and k
 * of all tokens of the call, chained to the launch after it (the page scorer) by a programmatic
 * dependent launch.
 *
 * q, q_out     (n_tokens, n_q_heads, head_dim) contiguous
 * k, k_out     (n_tokens, n_kv_heads, head_dim) contiguous (q_out may be q, k_out may be k)
 * freqs_cis    (n_tokens, head_dim / 2) pairs of float32 (cos, sin) = complex64
 * All pointers 8-byte aligned, head_dim even.
 */
DA_API int da_rope_qk(const void *q, const void *k, const void *freqs_cis, void *q_out, void *k_out,
                      int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int dtype,
                      da_stream_t stream);

/*
 * Dense causal attention of the prompt: replaces the flash_attn_func call of the prefill
 * stage (dram_attention/dram_attention.py:136) for 16-bit element types and head_dim 128.
 * tcgen05 tensor-core kernel (operands by TMA into shared memory, accumulators in tensor
 * memory), one CTA per 128 query rows and query head; softmax scale 1/sqrt(head_dim), GQA
 * by contiguous groups, float32 softmax and accumulation.
 *
 * q            (seq_len, n_q_heads, head_dim), unit channel stride, heads packed, rows
 *              q_row_stride elements apart
 * k, v         (seq_len, n_kv_heads, head_dim), rows kv_row_stride elements apart
 * out          (seq_len, n_q_heads, head_dim) contiguous, same dtype
 * All base pointers 16-byte aligned, row strides multiples of 8 elements.
 * da_prefill_attention_supported: 1 for head_dim 128 with DA_BF16 / DA_F16; for anything
 * else da_prefill_attention returns DA_ERR_UNSUPPORTED and the caller keeps its library call.
 */
DA_API int da_prefill_attention_supported(int head_dim, int dtype);
DA_API int da_prefill_attention(const void *q, const void *k, const void *v, void *out,
                         int seq_len, int n_q_heads, int n_kv_heads, int head_dim,
                         long long q_row_stride, long long kv_row_stride, int dtype,
                         int32_t *status, da_stream_t stream);

/*
 * All-gather of the per-rank attention outputs over NVLink peer memory, for KV-head
 * sharding on the GPUs of one node (no counterpart in the reference, which runs on one
 * GPU; it replaces the library all-gather that would otherwise follow the attention
 * launch).  One launch of one CTA: the rank's rows are stored into every rank's gather
 * buffer as 8-byte words {4 bytes of payload, tag = *seq + 1} (one aligned store each, so a
 * word that carries the tag carries its payload; no fence or flag round follows), the CTA
 * waits until every word of its own buffer carries this step's tag, copies the payload to
 * `out` and advances *seq.  The kernel is launched as a programmatic dependent of the kernel
 * before it in the stream and waits for it on the device before it reads `local`.
 * The wait is bounded by the GPU's timer: after timeout_us microseconds (0 = the default,
 * 200 000) the kernel sets DA_STATUS_WAIT_TIMEOUT in *status, writes 0xFF bytes (NaN in every
 * floating-point format) for what did not come and returns: nothing hangs, and a gather that
 * timed out cannot be mistaken for a result.  The caller has to look at *status (between
 * steps; it is sticky).
 *
 * local         bytes_per_rank bytes, device memory, 16-byte aligned (this rank's rows); NULL when the
 *               attention launch before it has sent them itself (da_decode_attention_push_next): the
 *               kernel then only waits and copies
 * peer_buffers  DEVICE array of `world` pointers; entry g = rank g's gather buffer of
 *               da_gather_heads_buffer_bytes(bytes_per_rank, world) bytes, mapped into
 *               this process (symmetric / IPC memory), zero before the first call
 * seq           (1) int32 device memory, zero before the first call, same value on all
 *               ranks (every rank makes the same sequence of calls)
 * out           world * bytes_per_rank bytes: rank-major concatenation
 * Every rank of the group must make the call for a step; ranks run on different GPUs.
 */
/*
 * Makes the NEXT attention call of this host thread (da_decode_attention, _tokens with one token, _fetch,
 * _phased: both launches of a step need it) send its output rows to the gather buffers of all ranks
 * straight from the CTA that merges a head, in the word format above, with tag *seq + 1 into slot *seq & 1:
 * the rows are on their way while the other heads are still being merged, and da_gather_heads(local =
 * NULL) after the launch only waits and copies.  The setting is consumed by that one call.
 * peer_buffers is a HOST array of `world` device pointers (the same buffers da_gather_heads is given as a
 * device array; they are copied into the launch's parameters), seq device memory.  bytes_per_rank must equal
 * n_kv_heads * rep * head_dim * element size of the call.
 */
DA_API int da_decode_attention_push_next(void *const *peer_buffers, const int32_t *seq, int rank, int world,
                                  int bytes_per_rank);

DA_API size_t da_gather_heads_buffer_bytes(int bytes_per_rank, int world);
DA_API int da_gather_heads(const void *local, int bytes_per_rank, void *const *peer_buffers,
                    int32_t *seq, int rank, int world, void *out, int timeout_us, int32_t *status,
                    da_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* DRAM_ATTENTION_B200_H */

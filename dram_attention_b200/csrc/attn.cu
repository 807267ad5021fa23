// Decode attention of one query token over the whole slot table plus the local
// window: split-K flash-decode with the append of the new key/value and the final
// merge in the same launch.
//
// Work unit = 16 consecutive tokens (8 KiB for head_dim 128 in 16-bit types).  A
// unit of the slot table is one contiguous block (token-major, key then value), so
// one untiled bulk copy (TMA) brings it into shared memory; a unit of the local
// window is gathered row by row with small bulk copies into the same layout.  Every
// warp owns a private ring of stages with one mbarrier each, so there is no
// CTA-wide synchronisation in the main loop.
//
// Arithmetic mapping: 8 lanes share a token (each owns D/8 channels, as two
// chunks that make conflict-free 128-bit shared-memory reads), 4 tokens per warp
// pass, all `rep` query heads of the KV head at once.  The dot products finish
// with a 3-step shuffle tree; softmax is online in the log2 domain with float32
// state; partial (m, l, acc) of the 4 token groups and the 4 warps are merged
// through shuffles and shared memory, written to the workspace, and the last CTA
// of a head (atomic ticket) merges the splits and writes the output.

#include "attn_body.cuh"

namespace da {

// Arithmetic of a 16-token unit on CUDA cores.  8 lanes share a token (each owns D/8 channels,
// as two chunks that make conflict-free 128-bit shared-memory reads), 4 tokens per warp pass,
// all query rows of the KV head at once.  The dot products finish with a 3-step shuffle tree;
// softmax is online in the log2 domain with float32 state.
template <typename T, int D_, int ROWS>
struct SimtMath {
    using Elem = T;
    static constexpr int kD = D_;
    static constexpr int E = (int)sizeof(T);
    static constexpr int ROWB = kD * E;
    static constexpr int kPitch = 2 * ROWB;                       // tokens packed as in HBM
    static constexpr int UNITB = kUnitTokens * kPitch;
    static constexpr int kStages = UNITB >= 16384 ? 2 : (UNITB >= 8192 ? 3 : 4);
    static constexpr bool kPerTokenCopy = false;                  // one copy per slot-table unit
    static constexpr int NPL = kD / 8;                            // channels per lane
    static constexpr int CH = NPL / 2;                            // channels per chunk
    static constexpr int CHB = CH * E;

    struct State {
        float qr[ROWS][NPL];    // query rows, pre-scaled by log2(e) / sqrt(D)
        float m[ROWS], l[ROWS], acc[ROWS][NPL];
        int back[ROWS];         // tokens at the end of a unit's range that the row must not see
    };

    __device__ __forceinline__ static void init(State &st, const AttnParams &p, int h, int lane, int rows) {
        const int j = lane & 7;
        const int hq = p.n_kv_heads * p.rep;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int tok = p.q_tok0 + r / p.rep;
            const bool live = r < rows;
            const unsigned char *qrow = p.q + ((size_t)(live ? tok : p.q_tok0) * hq + (size_t)h * p.rep +
                                               (live ? r % p.rep : 0)) * ROWB;
            load_elems<T, CH>(qrow + j * CHB, &st.qr[r][0]);
            load_elems<T, CH>(qrow + ROWB / 2 + j * CHB, &st.qr[r][CH]);
#pragma unroll
            for (int i = 0; i < NPL; ++i) st.qr[r][i] = live ? st.qr[r][i] * p.scale_log2 : 0.f;
            st.back[r] = live ? p.s_total - 1 - tok : 0;
            st.m[r] = -INFINITY;
            st.l[r] = 0.f;
#pragma unroll
            for (int i = 0; i < NPL; ++i) st.acc[r][i] = 0.f;
        }
    }

    // `avail` = tokens that exist from the unit's first token on; row r sees the first avail - back[r]
    __device__ __forceinline__ static void consume(State &st, const unsigned char *sb, int avail, int lane, float) {
        constexpr float NEG_INF = -INFINITY;
        const int g = lane >> 3;  // token group inside the warp
        const int j = lane & 7;   // channel block inside the token
        const int ntok = min(kUnitTokens, avail);
        // logits (log2 domain) of 4 tokens x ROWS rows
        float sc[4][ROWS];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            const unsigned char *kp = sb + (g + 4 * tt) * kPitch;
            float kf[NPL];
            load_elems<T, CH>(kp + j * CHB, &kf[0]);
            load_elems<T, CH>(kp + ROWB / 2 + j * CHB, &kf[CH]);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < NPL; ++i) a = fmaf(st.qr[r][i], kf[i], a);
                sc[tt][r] = a;
            }
        }
#pragma unroll
        for (int off = 1; off <= 4; off <<= 1)
#pragma unroll
            for (int tt = 0; tt < 4; ++tt)
#pragma unroll
                for (int r = 0; r < ROWS; ++r) sc[tt][r] += __shfl_xor_sync(DA_FULL_MASK, sc[tt][r], off);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (g + 4 * tt >= avail - st.back[r]) sc[tt][r] = NEG_INF;

        // online softmax update
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float mx = fmaxf(fmaxf(sc[0][r], sc[1][r]), fmaxf(sc[2][r], sc[3][r]));
            const float mnew = fmaxf(st.m[r], mx);
            const float msafe = (mnew == NEG_INF) ? 0.f : mnew;
            const float alpha = fast_exp2(st.m[r] - msafe);
            float psum = 0.f;
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
                sc[tt][r] = fast_exp2(sc[tt][r] - msafe);
                psum += sc[tt][r];
            }
            st.l[r] = st.l[r] * alpha + psum;
            st.m[r] = mnew;
#pragma unroll
            for (int i = 0; i < NPL; ++i) st.acc[r][i] *= alpha;
        }

        // values
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            if (g + 4 * tt < ntok) {
                const unsigned char *vp = sb + (g + 4 * tt) * kPitch + ROWB;
                float vf[NPL];
                load_elems<T, CH>(vp + j * CHB, &vf[0]);
                load_elems<T, CH>(vp + ROWB / 2 + j * CHB, &vf[CH]);
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
#pragma unroll
                    for (int i = 0; i < NPL; ++i) st.acc[r][i] = fmaf(sc[tt][r], vf[i], st.acc[r][i]);
            }
        }
    }

    // merge the 4 token groups of the warp, then lanes 0..7 write the rows
    __device__ __forceinline__ static void publish(State &st, float *red, int lane, int rows) {
        constexpr float NEG_INF = -INFINITY;
        constexpr int PW = PartialRow<kD>::kWidth;
        const int g = lane >> 3;
        const int j = lane & 7;
#pragma unroll
        for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const float mo = __shfl_xor_sync(DA_FULL_MASK, st.m[r], off);
                const float lo = __shfl_xor_sync(DA_FULL_MASK, st.l[r], off);
                const float mn = fmaxf(st.m[r], mo);
                const float ms = (mn == NEG_INF) ? 0.f : mn;
                const float a = fast_exp2(st.m[r] - ms);
                const float b = fast_exp2(mo - ms);
                st.l[r] = st.l[r] * a + lo * b;
                st.m[r] = mn;
#pragma unroll
                for (int i = 0; i < NPL; ++i) {
                    const float ao = __shfl_xor_sync(DA_FULL_MASK, st.acc[r][i], off);
                    st.acc[r][i] = st.acc[r][i] * a + ao * b;
                }
            }
        }
        if (g == 0) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r < rows) {
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        red[r * PW + j * CH + i] = st.acc[r][i];
                        red[r * PW + kD / 2 + j * CH + i] = st.acc[r][CH + i];
                    }
                    if (j == 0) {
                        red[r * PW + kD] = st.m[r];
                        red[r * PW + kD + 1] = st.l[r];
                    }
                }
            }
        }
    }
};

template <typename T, int D, int ROWS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 4 ? 2 : 1) decode_attention_kernel(const AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    decode_attention_body<SimtMath<T, D, ROWS>, WARPS, SimtMath<T, D, ROWS>::kStages>(p, smem);
}

constexpr int kSimtPhase1Warps = 8;   // float32 stages are twice as large: 8 warps fill an SM

template <typename T, int D, int ROWS, int WARPS>
static cudaError_t launch_attn_w(const AttnParams &p, int n_kv_heads, int splits, cudaStream_t stream) {
    using M = SimtMath<T, D, ROWS>;
    constexpr int SMEM = WARPS * M::kStages * M::UNITB;
    auto kern = decode_attention_kernel<T, D, ROWS, WARPS>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    dim3 grid(splits, n_kv_heads);
    // phase 1 runs on a stream of its own beside the kernels of the step; the other launches follow
    // the LRU update in their stream and may move onto the SMs while it is still running
    if (p.phase != 1) return launch_dependent(kern, grid, dim3(WARPS * 32), (size_t)SMEM, stream, p);
    kern<<<grid, WARPS * 32, SMEM, stream>>>(p);
    return cudaGetLastError();
}

template <typename T, int D, int ROWS>
static cudaError_t launch_attn(const AttnParams &p, int n_kv_heads, int splits, cudaStream_t stream) {
    if (p.phase == 1) return launch_attn_w<T, D, ROWS, kSimtPhase1Warps>(p, n_kv_heads, splits, stream);
    return launch_attn_w<T, D, ROWS, kAttnWarps>(p, n_kv_heads, splits, stream);
}

// float32: up to 8 query rows per launch (register budget)
constexpr int kSimtMaxRows = 8;

template <typename T>
static cudaError_t dispatch_attn(const AttnParams &p, int n_kv_heads, int head_dim, int splits, cudaStream_t s) {
    const int rows = p.n_q * p.rep;
#define DA_ATTN_CASE(DD, RR) \
    if (head_dim == DD && rows <= RR) return launch_attn<T, DD, RR>(p, n_kv_heads, splits, s);
    DA_ATTN_CASE(128, 1) DA_ATTN_CASE(128, 2) DA_ATTN_CASE(128, 4) DA_ATTN_CASE(128, 8)
    DA_ATTN_CASE(64, 1) DA_ATTN_CASE(64, 2) DA_ATTN_CASE(64, 4) DA_ATTN_CASE(64, 8)
#undef DA_ATTN_CASE
    return cudaErrorInvalidValue;
}

}  // namespace da

// ---- host side ---------------------------------------------------------------------------

namespace da {

// Everything one attention call needs; the entry points below fill it in.
struct AttnCall {
    const void *q = nullptr;
    int n_q_tokens = 1;
    const void *prefix_kv = nullptr;
    long long prefix_head_stride = 0;
    int n_prefix_tokens = 0;
    void *local_k = nullptr, *local_v = nullptr;
    long long local_token_stride = 0, local_head_stride = 0;
    int local_capacity = 0;
    const void *new_k = nullptr, *new_v = nullptr;
    const int32_t *start_pos_dev = nullptr;
    int start_pos_host = 0, dram_tokens = 0;
    void *out = nullptr;
    float *lse_out = nullptr;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    int32_t *status = nullptr;
    int n_kv_heads = 0, rep = 0, head_dim = 0, dtype = 0;
    // miss fetch inside the kernel
    const void *dram_pages = nullptr;
    int n_dram_pages = 0;
    const int32_t *slot_source = nullptr;
    int n_slots = 0, page_size = 0;
    // two launches
    int phase = 0;
    const int32_t *order = nullptr, *n_evictable = nullptr, *redo = nullptr;
    int32_t *flip = nullptr;
    int splits1 = 0, splits2 = 0;
    da_stream_t stream = nullptr;
};

// What da_decode_attention_push_next() left for the next attention call of this host thread.
struct PeerPush {
    void *bufs[kAttnMaxPeers] = {};
    const int32_t *seq = nullptr;
    int rank = 0, world = 0, bytes_per_rank = 0;   // world == 0: nothing set
};
static thread_local PeerPush g_next_push;

static int max_rows_of(int dtype) { return dtype == DA_F32 ? kSimtMaxRows : kAttnMaxRows; }

static size_t partial_bytes(int n_kv_heads, int part_rows, int rows, int head_dim) {
    return (size_t)n_kv_heads * part_rows * rows * (head_dim + 4) * sizeof(float);
}

static int run_attention(const AttnCall &c) {
    const PeerPush push = g_next_push;   // consumed by this call, whatever becomes of it
    g_next_push = PeerPush();
    if (!c.q || !c.prefix_kv || !c.local_k || !c.local_v || !c.new_k || !c.new_v || !c.out || !c.workspace ||
        !c.status)
        return DA_ERR_NULL;
    if (c.n_kv_heads < 1 || c.n_prefix_tokens < 1 || c.local_capacity < 1 || c.dram_tokens < 0 || c.rep < 1 ||
        c.n_q_tokens < 1 || c.n_q_tokens > c.local_capacity)
        return DA_ERR_SHAPE;
    if (c.head_dim != 64 && c.head_dim != 128) return DA_ERR_UNSUPPORTED;
    if (c.dtype != DA_F32 && c.dtype != DA_F16 && c.dtype != DA_BF16) return DA_ERR_DTYPE;
    if (c.rep > max_rows_of(c.dtype)) return DA_ERR_UNSUPPORTED;
    if (c.n_kv_heads * 4 > kCounterBytes || c.n_kv_heads > 65535) return DA_ERR_UNSUPPORTED;
    const size_t esz = c.dtype == DA_F32 ? 4 : 2;
    const uintptr_t ptrs = (uintptr_t)c.q | (uintptr_t)c.prefix_kv | (uintptr_t)c.local_k | (uintptr_t)c.local_v |
                           (uintptr_t)c.new_k | (uintptr_t)c.new_v | (uintptr_t)c.out;
    if ((ptrs & 15) || ((uintptr_t)c.workspace & 255)) return DA_ERR_ALIGN;
    if (((size_t)c.prefix_head_stride * esz) % 16 || ((size_t)c.local_token_stride * esz) % 16 ||
        ((size_t)c.local_head_stride * esz) % 16)
        return DA_ERR_ALIGN;
    if (c.phase < 0 || c.phase > 2) return DA_ERR_SHAPE;
    if (c.phase != 0 && c.n_q_tokens != 1) return DA_ERR_UNSUPPORTED;
    if (push.world > 0 &&
        (c.n_q_tokens != 1 || (size_t)push.bytes_per_rank != (size_t)c.n_kv_heads * c.rep * c.head_dim * esz))
        return DA_ERR_SHAPE;

    const int tokens_per_launch = max_rows_of(c.dtype) / c.rep;
    const int rows_max = (c.n_q_tokens < tokens_per_launch ? c.n_q_tokens : tokens_per_launch) * c.rep;
    const int splits0 = attn_splits(c.n_kv_heads);
    const int part_rows = c.phase == 0 ? splits0 : c.splits1 + c.splits2;
    if (c.workspace_bytes < (size_t)kCounterBytes + partial_bytes(c.n_kv_heads, part_rows, rows_max, c.head_dim))
        return DA_ERR_WORKSPACE;

    AttnParams p{};
    for (int g = 0; g < kAttnMaxPeers; ++g) p.peer_buf[g] = static_cast<uint2 *>(push.bufs[g]);
    p.peer_seq = push.seq;
    p.peer_rank = push.rank;
    p.peer_world = push.world;
    p.peer_words = push.bytes_per_rank / 4;
    p.q = static_cast<const unsigned char *>(c.q);
    p.prefix = static_cast<const unsigned char *>(c.prefix_kv);
    p.prefix_head_stride = c.prefix_head_stride;
    p.n_prefix_tokens = c.n_prefix_tokens;
    p.local_k = static_cast<unsigned char *>(c.local_k);
    p.local_v = static_cast<unsigned char *>(c.local_v);
    p.local_tok_stride = c.local_token_stride;
    p.local_head_stride = c.local_head_stride;
    p.local_capacity = c.local_capacity;
    p.new_k = static_cast<const unsigned char *>(c.new_k);
    p.new_v = static_cast<const unsigned char *>(c.new_v);
    p.start_pos_dev = c.start_pos_dev;
    p.start_pos_host = c.start_pos_host;
    p.dram_tokens = c.dram_tokens;
    p.out = static_cast<unsigned char *>(c.out);
    p.lse_out = c.lse_out;
    p.counters = static_cast<unsigned int *>(c.workspace);
    p.partials = reinterpret_cast<float *>(static_cast<unsigned char *>(c.workspace) + kCounterBytes);
    p.status = c.status;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)c.head_dim);
    if (c.slot_source) {
        // units (16 tokens) must not straddle pages and the slot table must be exactly the prefix
        if (!c.dram_pages) return DA_ERR_NULL;
        if (c.page_size < 1 || c.n_slots < 1 || c.n_dram_pages < 1) return DA_ERR_SHAPE;
        if (c.page_size % kUnitTokens != 0 || (long long)c.n_slots * c.page_size != c.n_prefix_tokens)
            return DA_ERR_UNSUPPORTED;
        if ((uintptr_t)c.dram_pages & 15) return DA_ERR_ALIGN;
        p.dram = static_cast<const unsigned char *>(c.dram_pages);
        p.dram_head_stride = (long long)c.n_dram_pages * c.page_size * 2 * c.head_dim;
        p.slot_source = c.slot_source;
        p.n_slots = c.n_slots;
        p.page_tokens = c.page_size;
    }
    p.phase = c.phase;
    p.n_kv_heads = c.n_kv_heads;
    p.rep = c.rep;
    p.head_dim = c.head_dim;
    p.s_total = c.n_q_tokens;
    p.part_rows = part_rows;
    p.part_offset = 0;
    p.ticket_target = part_rows;
    p.splits1 = 0;
    int splits = splits0;
    if (c.phase != 0) {
        if (!c.slot_source || !c.order || !c.n_evictable || !c.flip || !c.redo) return DA_ERR_NULL;
        if (c.splits1 < 1 || c.splits2 < 1 || c.splits1 > kAttnMaxSplits || c.splits2 > kAttnMaxSplits)
            return DA_ERR_SHAPE;
        p.order = c.order;
        p.n_evictable = c.n_evictable;
        p.flip = c.flip;
        p.redo = c.redo;
        p.splits1 = c.splits1;                       // phase-1 rows, then phase-2 rows
        p.part_offset = c.phase == 2 ? c.splits1 : 0;
        splits = c.phase == 1 ? c.splits1 : c.splits2;
    }

    cudaStream_t s = static_cast<cudaStream_t>(c.stream);
    for (int tok0 = 0; tok0 < c.n_q_tokens; tok0 += tokens_per_launch) {
        p.q_tok0 = tok0;
        p.n_q = c.n_q_tokens - tok0 < tokens_per_launch ? c.n_q_tokens - tok0 : tokens_per_launch;
        cudaError_t e;
        if (c.dtype == DA_F32) e = dispatch_attn<float>(p, c.n_kv_heads, c.head_dim, splits, s);
        else e = launch_attention_mma(p, c.n_kv_heads, c.head_dim, c.dtype, splits, s);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

}  // namespace da

extern "C" size_t da_decode_attention_tokens_workspace_bytes(int n_kv_heads, int rep, int head_dim,
                                                             int n_q_tokens) {
    if (n_kv_heads < 1 || rep < 1 || head_dim < 1 || n_q_tokens < 1) return 0;
    long long rows = (long long)rep * n_q_tokens;
    if (rows > da::kAttnMaxRows) rows = da::kAttnMaxRows > rep ? da::kAttnMaxRows / rep * rep : rep;
    return (size_t)da::kCounterBytes +
           da::partial_bytes(n_kv_heads, da::attn_splits(n_kv_heads), (int)rows, head_dim);
}

extern "C" size_t da_decode_attention_workspace_bytes(int n_kv_heads, int rep, int head_dim) {
    return da_decode_attention_tokens_workspace_bytes(n_kv_heads, rep, head_dim, 1);
}

extern "C" int da_decode_attention_tokens(const void *q, int n_q_tokens, const void *prefix_kv,
                                          long long prefix_head_stride, int n_prefix_tokens, void *local_k,
                                          void *local_v, long long local_token_stride,
                                          long long local_head_stride, int local_capacity, const void *new_k,
                                          const void *new_v, const int32_t *start_pos_dev, int start_pos_host,
                                          int dram_tokens, void *out, float *lse_out, void *workspace,
                                          size_t workspace_bytes, int32_t *status, int n_kv_heads, int rep,
                                          int head_dim, int dtype, da_stream_t stream) {
    da::AttnCall c;
    c.q = q; c.n_q_tokens = n_q_tokens;
    c.prefix_kv = prefix_kv; c.prefix_head_stride = prefix_head_stride; c.n_prefix_tokens = n_prefix_tokens;
    c.local_k = local_k; c.local_v = local_v;
    c.local_token_stride = local_token_stride; c.local_head_stride = local_head_stride;
    c.local_capacity = local_capacity;
    c.new_k = new_k; c.new_v = new_v;
    c.start_pos_dev = start_pos_dev; c.start_pos_host = start_pos_host; c.dram_tokens = dram_tokens;
    c.out = out; c.lse_out = lse_out;
    c.workspace = workspace; c.workspace_bytes = workspace_bytes; c.status = status;
    c.n_kv_heads = n_kv_heads; c.rep = rep; c.head_dim = head_dim; c.dtype = dtype;
    c.stream = stream;
    return da::run_attention(c);
}

extern "C" int da_decode_attention(const void *q, const void *prefix_kv, long long prefix_head_stride,
                                   int n_prefix_tokens, void *local_k, void *local_v,
                                   long long local_token_stride, long long local_head_stride,
                                   int local_capacity, const void *new_k, const void *new_v,
                                   const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                   void *out, float *lse_out, void *workspace, size_t workspace_bytes,
                                   int32_t *status, int n_kv_heads, int rep, int head_dim, int dtype,
                                   da_stream_t stream) {
    return da_decode_attention_tokens(q, 1, prefix_kv, prefix_head_stride, n_prefix_tokens, local_k, local_v,
                                      local_token_stride, local_head_stride, local_capacity, new_k, new_v,
                                      start_pos_dev, start_pos_host, dram_tokens, out, lse_out, workspace,
                                      workspace_bytes, status, n_kv_heads, rep, head_dim, dtype, stream);
}

static int fill_fetch_call(da::AttnCall &c, const void *q, void *slots, long long slots_head_stride, int n_slots,
                           int page_size, const void *dram_pages, int n_dram_pages, const int32_t *slot_source,
                           void *local_k, void *local_v, long long local_token_stride,
                           long long local_head_stride, int local_capacity, const void *new_k, const void *new_v,
                           const int32_t *start_pos_dev, int start_pos_host, int dram_tokens, void *out,
                           float *lse_out, void *workspace, size_t workspace_bytes, int32_t *status,
                           int n_kv_heads, int rep, int head_dim, int dtype, da_stream_t stream) {
    if (!slot_source) return DA_ERR_NULL;
    if (n_slots < 1 || page_size < 1 || (long long)n_slots * page_size > 0x7fffffffLL) return DA_ERR_SHAPE;
    c.q = q;
    c.prefix_kv = slots; c.prefix_head_stride = slots_head_stride; c.n_prefix_tokens = n_slots * page_size;
    c.local_k = local_k; c.local_v = local_v;
    c.local_token_stride = local_token_stride; c.local_head_stride = local_head_stride;
    c.local_capacity = local_capacity;
    c.new_k = new_k; c.new_v = new_v;
    c.start_pos_dev = start_pos_dev; c.start_pos_host = start_pos_host; c.dram_tokens = dram_tokens;
    c.out = out; c.lse_out = lse_out;
    c.workspace = workspace; c.workspace_bytes = workspace_bytes; c.status = status;
    c.n_kv_heads = n_kv_heads; c.rep = rep; c.head_dim = head_dim; c.dtype = dtype;
    c.dram_pages = dram_pages; c.n_dram_pages = n_dram_pages; c.slot_source = slot_source;
    c.n_slots = n_slots; c.page_size = page_size;
    c.stream = stream;
    return 0;
}

extern "C" int da_decode_attention_fetch(const void *q, void *slots, long long slots_head_stride, int n_slots,
                                         int page_size, const void *dram_pages, int n_dram_pages,
                                         const int32_t *slot_source, void *local_k, void *local_v,
                                         long long local_token_stride, long long local_head_stride,
                                         int local_capacity, const void *new_k, const void *new_v,
                                         const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                         void *out, float *lse_out, void *workspace, size_t workspace_bytes,
                                         int32_t *status, int n_kv_heads, int rep, int head_dim, int dtype,
                                         da_stream_t stream) {
    da::AttnCall c;
    const int rc = fill_fetch_call(c, q, slots, slots_head_stride, n_slots, page_size, dram_pages, n_dram_pages,
                                   slot_source, local_k, local_v, local_token_stride, local_head_stride,
                                   local_capacity, new_k, new_v, start_pos_dev, start_pos_host, dram_tokens, out,
                                   lse_out, workspace, workspace_bytes, status, n_kv_heads, rep, head_dim, dtype,
                                   stream);
    if (rc != 0) return rc;
    return da::run_attention(c);
}

// CTAs per head of the two launches: the caller's choice, or the defaults
static int phase_splits(int n_kv_heads, int requested, int phase) {
    if (requested > 0) return requested;
    return phase == 1 ? da::attn_splits_phase1(n_kv_heads) : da::attn_splits_phase2(n_kv_heads);
}

extern "C" int da_decode_attention_phased_supported(int n_kv_heads, int rep, int head_dim, int dtype, int n_slots,
                                                    int page_size, int local_capacity) {
    if (n_kv_heads < 1 || n_slots < 1 || page_size < 1 || local_capacity < 1 || rep < 1) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    if (dtype != DA_F32 && dtype != DA_F16 && dtype != DA_BF16) return 0;
    if (rep > da::max_rows_of(dtype)) return 0;
    if (n_kv_heads * 4 > da::kCounterBytes) return 0;
    if (page_size % da::kUnitTokens != 0 || (long long)n_slots * page_size > 0x7fffffffLL) return 0;
    // shared memory of a phase-1 CTA: warps x stages x stage bytes, plus the plan tables
    const size_t esz = dtype == DA_F32 ? 4 : 2;
    size_t stage = (size_t)da::kUnitTokens * (2 * head_dim * esz + (esz == 2 ? 16 : 0));
    const int stages = esz == 2 ? 2 : (stage >= 16384 ? 2 : (stage >= 8192 ? 3 : 4));
    const int warps = esz == 2 ? da::kAttnPhase1Warps : da::kSimtPhase1Warps;
    const size_t smem = (size_t)warps * stages * stage + (size_t)warps * da::kRoundUnits * 16 + 2048;
    return smem <= 227 * 1024 ? 1 : 0;
}

extern "C" size_t da_decode_attention_phased_workspace_bytes(int n_kv_heads, int rep, int head_dim) {
    if (n_kv_heads < 1 || rep < 1 || head_dim < 1) return 0;
    // room for any choice of CTAs per head in the two launches
    return (size_t)da::kCounterBytes + da::partial_bytes(n_kv_heads, 2 * da::kAttnMaxSplits, rep, head_dim);
}

extern "C" int da_decode_attention_phased(int phase, const int32_t *order, const int32_t *n_evictable,
                                          int32_t *split_flip, const int32_t *split_redo, int phase1_ctas,
                                          int phase2_ctas, const void *q, void *slots,
                                          long long slots_head_stride, int n_slots, int page_size,
                                          const void *dram_pages, int n_dram_pages, const int32_t *slot_source,
                                          void *local_k, void *local_v, long long local_token_stride,
                                          long long local_head_stride, int local_capacity, const void *new_k,
                                          const void *new_v, const int32_t *start_pos_dev, int start_pos_host,
                                          int dram_tokens, void *out, float *lse_out, void *workspace,
                                          size_t workspace_bytes, int32_t *status, int n_kv_heads, int rep,
                                          int head_dim, int dtype, da_stream_t stream) {
    if (phase != 1 && phase != 2) return DA_ERR_SHAPE;
    if (!slot_source || !order || !n_evictable || !split_flip || !split_redo) return DA_ERR_NULL;
    if (phase1_ctas < 0 || phase2_ctas < 0 || phase1_ctas > da::kAttnMaxSplits || phase2_ctas > da::kAttnMaxSplits)
        return DA_ERR_SHAPE;
    if (!da_decode_attention_phased_supported(n_kv_heads, rep, head_dim, dtype, n_slots, page_size, local_capacity))
        return DA_ERR_UNSUPPORTED;
    da::AttnCall c;
    const int rc = fill_fetch_call(c, q, slots, slots_head_stride, n_slots, page_size, dram_pages, n_dram_pages,
                                   slot_source, local_k, local_v, local_token_stride, local_head_stride,
                                   local_capacity, new_k, new_v, start_pos_dev, start_pos_host, dram_tokens, out,
                                   lse_out, workspace, workspace_bytes, status, n_kv_heads, rep, head_dim, dtype,
                                   stream);
    if (rc != 0) return rc;
    c.phase = phase;
    c.order = order;
    c.n_evictable = n_evictable;
    c.flip = split_flip;
    c.redo = split_redo;
    c.splits1 = phase_splits(n_kv_heads, phase1_ctas, 1);
    c.splits2 = phase_splits(n_kv_heads, phase2_ctas, 2);
    return da::run_attention(c);
}

extern "C" int da_decode_attention_push_next(void *const *peer_buffers, const int32_t *seq, int rank, int world,
                                             int bytes_per_rank) {
    if (!peer_buffers || !seq) return DA_ERR_NULL;
    if (world < 1 || world > da::kAttnMaxPeers || rank < 0 || rank >= world || bytes_per_rank < 16 ||
        bytes_per_rank % 16 != 0)
        return DA_ERR_SHAPE;
    for (int g = 0; g < world; ++g) {
        if (!peer_buffers[g]) return DA_ERR_NULL;
        da::g_next_push.bufs[g] = peer_buffers[g];
    }
    da::g_next_push.seq = seq;
    da::g_next_push.rank = rank;
    da::g_next_push.world = world;
    da::g_next_push.bytes_per_rank = bytes_per_rank;
    return 0;
}

DA_DEFINE_TRACE_SETTER(trace_set_attn)

// ---- entry point with built-in scratch ------------------------------------------------

namespace da {
// Scratch for da_decode_attention_static: the same layout da_decode_attention expects in
// its workspace (ticket counters, then the per-CTA partials).  2 MiB covers every shape
// the kernels accept with head_dim <= 128 and rep <= 8 (the largest needs about 1.2 MiB).
// The array is part of the loaded module: every GPU that loads this library keeps it
// until the process exits, and it starts out zero-filled.
constexpr size_t kStaticScratchBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
}  // namespace da

extern "C" size_t da_decode_attention_static_capacity(void) { return da::kStaticScratchBytes; }

extern "C" int da_decode_attention_static(const void *q, const void *prefix_kv, long long prefix_head_stride,
                                          int n_prefix_tokens, void *local_k, void *local_v,
                                          long long local_token_stride, long long local_head_stride,
                                          int local_capacity, const void *new_k, const void *new_v,
                                          const int32_t *start_pos_dev, int start_pos_host, int dram_tokens,
                                          void *out, float *lse_out, int32_t *status, int n_kv_heads, int rep,
                                          int head_dim, int dtype, da_stream_t stream) {
    if (n_kv_heads < 1 || rep < 1 || head_dim < 1) return DA_ERR_SHAPE;
    const size_t need = da_decode_attention_workspace_bytes(n_kv_heads, rep, head_dim);
    if (need > da::kStaticScratchBytes) return DA_ERR_STATIC_SCRATCH;

    // In host code the array's name is only a handle for the runtime, not a device
    // address: ask the runtime for the address once per device, with that device
    // current (it is: the caller's stream belongs to it), and hand that to the kernel.
    static void *scratch_of_device[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DA_ERR_UNSUPPORTED;
    if (scratch_of_device[dev] == nullptr) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, da::g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        scratch_of_device[dev] = ptr;
    }
    void *scratch = scratch_of_device[dev];

    // All calls share the array and it keeps what the last call left.  The kernel only
    // needs the ticket counters to be zero on entry; clear them on the caller's stream
    // (a call that was cut short could have left them half counted).
    e = cudaMemsetAsync(scratch, 0, da::kCounterBytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return (int)e;
    return da_decode_attention(q, prefix_kv, prefix_head_stride, n_prefix_tokens, local_k, local_v,
                               local_token_stride, local_head_stride, local_capacity, new_k, new_v,
                               start_pos_dev, start_pos_host, dram_tokens, out, lse_out, scratch,
                               da::kStaticScratchBytes, status, n_kv_heads, rep, head_dim, dtype, stream);
}

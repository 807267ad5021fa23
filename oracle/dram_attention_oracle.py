"""CPU oracle for the generate-stage hot path of DRAM Attention.

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, the algorithm of
the reference implementation (project `long-context/dram-attention`, package
`dram_attention/`).  It exists to check the CUDA kernels and to be timed as the
CPU baseline; the product package never imports it.

Pinning: every function below is checked (tests/test_oracle_*.py) against
  * the reference's own known-answer cases for the LRU kernel
    (dram_attention/lru_triton_kernel_test.py:17-204),
  * the reference's scorer value test (max_ip_triton_kernel_test.py:29-38),
  * golden trajectories under tests/golden/ that were produced by importing and
    running the reference's own classes on the CPU (tests/golden/make_golden.py).
The attention arithmetic of the reference lives in the third-party package
flash-attn (>=2.6.3, not vendored); the reference's tests check only shapes at
that boundary, so attention VALUES are pinned by the published softmax
attention definition, not by a reference vector.

Arithmetic: page scores are float32 on float32-upcast inputs (the quantity the
selection is defined on); attention and the merge are float64 on upcast
inputs; integer work (selection, LRU tables) is exact.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------
# Page summaries and the Quest upper-bound page score
# --------------------------------------------------------------------------

def rope_qk(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The caller's rotary embedding in front of the operator call
    (evaluation/dram-attention/model.py:125-135): channels (2i, 2i+1) of every head as a
    complex number times freqs_cis[token, i], in float32, rounded to the input type.
    xq (1, s, Hq, D), xk (1, s, Hk, D), freqs_cis (s, D/2) complex64.  Written out on the real
    and imaginary parts with numpy float32 arrays, so every product and the sum round once."""
    f = torch.view_as_real(freqs_cis).numpy().astype(np.float32)      # (s, D/2, 2)
    c, sn = f[None, :, None, :, 0], f[None, :, None, :, 1]

    def rot(x: torch.Tensor) -> torch.Tensor:
        a = x.float().numpy().reshape(*x.shape[:-1], -1, 2)
        x0, x1 = a[..., 0], a[..., 1]
        re = (x0 * c).astype(np.float32) - (x1 * sn).astype(np.float32)
        im = (x0 * sn).astype(np.float32) + (x1 * c).astype(np.float32)
        out = np.stack([re, im], axis=-1).reshape(x.shape).astype(np.float32)
        return torch.from_numpy(out).to(x.dtype)

    return rot(xq), rot(xk)


def page_minmax(k_cache: torch.Tensor, num_pages: int) -> torch.Tensor:
    """Per-page, per-channel min and max of the keys.

    Follows dram_attention/topk_selector.py:24-35: `k_cache` is
    (num_kv_heads, length, head_dim); the result is
    (num_kv_heads, num_pages, 2, head_dim) with [..., 0, :] = min and
    [..., 1, :] = max, in the dtype of the keys.
    """
    h, length, d = k_cache.shape
    assert length % num_pages == 0, "Cache size must be divisible by num_pages."
    page = length // num_pages
    chunked = k_cache.reshape(h, num_pages, page, d)
    mn, mx = torch.aminmax(chunked, dim=2)
    return torch.stack((mn, mx), dim=-2)


def score_pages(q: torch.Tensor, min_max: torch.Tensor) -> torch.Tensor:
    """score[n, h, l] = sum_d max(q[n,h,d]*min[h,l,d], q[n,h,d]*max[h,l,d]).

    Follows `max_ip_ref`, dram_attention/max_ip_triton_kernel.py:127-133, on
    float32-upcast inputs.  q is (N, H, D); min_max is (H, L, 2, D); the
    result is float32 (N, H, L).
    """
    n, h, d = q.shape
    h1, l, r, d1 = min_max.shape
    assert h1 == h and d1 == d and r == 2
    qf = q.to(torch.float32)
    mm = min_max.to(torch.float32)
    out = torch.empty(n, h, l, dtype=torch.float32)
    # chunk over pages to bound the (N, H, chunk, 2, D) temporary
    step = max(1, (1 << 24) // max(1, n * h * 2 * d))
    for s in range(0, l, step):
        e = min(l, s + step)
        prod = qf[:, :, None, None, :] * mm[None, :, s:e]
        out[:, :, s:e] = torch.amax(prod, dim=-2).sum(-1)
    return out


def gqa_fold_query(q: torch.Tensor, num_kv_heads: int) -> torch.Tensor:
    """(1, S, Hq, D) -> (S*rep, Hk, D) with query head hq = hk*rep + r.

    Follows dram_attention/topk_selector.py:48-55.
    """
    bsz, s, hq, d = q.shape
    assert bsz == 1
    assert hq % num_kv_heads == 0
    rep = hq // num_kv_heads
    return q.reshape(s, num_kv_heads, rep, d).swapaxes(1, 2).reshape(s * rep, num_kv_heads, d)


def scores_by_query_head(q: torch.Tensor, min_max: torch.Tensor) -> torch.Tensor:
    """(1, S, Hq, D) queries -> float32 scores (S, Hk, rep, L).

    Follows dram_attention/topk_selector.py:52-59.
    """
    hk = min_max.shape[0]
    bsz, s, hq, d = q.shape
    rep = hq // hk
    ip = score_pages(gqa_fold_query(q, hk), min_max)
    return ip.reshape(s, rep, hk, -1).swapaxes(1, 2).contiguous()


def select_pages(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Top-k page ids per query head: descending score, ties by ascending id.

    Follows dram_attention/topk_selector.py:61 (`argsort(descending)[..., :k]`)
    with the tie-break made deterministic by a stable sort.  Equal scores
    include -0.0 == +0.0.  int64, same leading shape as `scores`, last dim
    min(k, L).
    """
    return torch.argsort(scores, dim=-1, descending=True, stable=True)[..., :k]


def build_page_list(top_k_indices: torch.Tensor) -> torch.Tensor:
    """(S, Hk, rep, k) -> (Hk, S*rep*k): the per-KV-head list given to the LRU.

    Follows dram_attention/lru_cache.py:260-264: the lists of the `rep` query
    heads are concatenated, duplicates kept.
    """
    s, hk, rep, k = top_k_indices.shape
    return top_k_indices.swapaxes(0, 1).contiguous().reshape(hk, -1)


# --------------------------------------------------------------------------
# LRU slot table
# --------------------------------------------------------------------------

def lru_walk(page_list: np.ndarray, d2h: np.ndarray, h2d: np.ndarray,
             times: np.ndarray, step: int,
             dram: Optional[np.ndarray] = None, hbm: Optional[np.ndarray] = None
             ) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Sequential LRU update for all heads, in place.  `step` is the value
    AFTER the increment of dram_attention/lru_cache.py:224.

    Follows dram_attention/lru_triton_kernel.py:
      * :110-137  every listed page that is resident gets time = step;
      * :170      eviction order = stable ascending argsort of the times;
      * :30-107   walk the list in order; a page that is not resident takes the
                  next slot of the eviction order, the slot's old page is
                  unmapped, the payload is copied DRAM -> HBM.
    The reference stores d2h[-1] = -1 when the victim slot is empty
    (:56-66, old page == -1); that write lands on the last DRAM page's entry
    through negative indexing only by accident of pointer arithmetic, so here
    it is skipped (old >= 0 guard).

    Returns (miss_pages, miss_slots, n_miss) per head in list order, the pairs
    the payload copy has to move.
    """
    hk, kk = page_list.shape
    nh = h2d.shape[1]
    miss_pages = np.full((hk, kk), -1, dtype=np.int64)
    miss_slots = np.full((hk, kk), -1, dtype=np.int64)
    n_miss = np.zeros(hk, dtype=np.int64)
    for h in range(hk):
        lst = page_list[h]
        slots = d2h[h, lst]
        hit = slots >= 0
        times[h, slots[hit]] = step
        order = np.argsort(times[h], kind="stable")
        ptr = 0
        for i in range(kk):
            p = int(lst[i])
            s = int(d2h[h, p])
            if s < 0:
                v = int(order[ptr])
                times[h, v] = step
                old = int(h2d[h, v])
                if old >= 0:
                    d2h[h, old] = -1
                h2d[h, v] = p
                d2h[h, p] = v
                if dram is not None:
                    hbm[h, v] = dram[h, p]
                j = n_miss[h]
                miss_pages[h, j] = p
                miss_slots[h, j] = v
                n_miss[h] += 1
                ptr = (ptr + 1) % nh
            else:
                times[h, s] = step
    return miss_pages, miss_slots, n_miss


def lru_vectorised(page_list: np.ndarray, d2h: np.ndarray, h2d: np.ndarray,
                   times: np.ndarray, step: int,
                   dram: Optional[np.ndarray] = None, hbm: Optional[np.ndarray] = None
                   ) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Same result as `lru_walk`, written as array operations (used for timing
    the CPU baseline and for large cases).  Valid while the number of distinct
    listed pages does not exceed the number of slots; raises otherwise, since
    beyond that the sequential walk wraps its eviction pointer and evicts
    pages loaded earlier in the same call.
    """
    hk, kk = page_list.shape
    nh = h2d.shape[1]
    miss_pages = np.full((hk, kk), -1, dtype=np.int64)
    miss_slots = np.full((hk, kk), -1, dtype=np.int64)
    n_miss = np.zeros(hk, dtype=np.int64)
    for h in range(hk):
        lst = page_list[h]
        slots = d2h[h, lst]
        hit = slots >= 0
        times[h, slots[hit]] = step
        # first occurrences, in list order, of pages that are not resident
        cand = lst[~hit]
        _, first = np.unique(cand, return_index=True)
        misses = cand[np.sort(first)]
        m = misses.shape[0]
        if m == 0:
            continue
        order = np.argsort(times[h], kind="stable")
        victims = order[:m]
        if m > nh or times[h, victims[-1]] == step:
            raise ValueError("more distinct pages requested than slots available")
        old = h2d[h, victims]
        d2h[h, old[old >= 0]] = -1
        h2d[h, victims] = misses
        d2h[h, misses] = victims
        times[h, victims] = step
        if dram is not None:
            hbm[h, victims] = dram[h, misses]
        miss_pages[h, :m] = misses
        miss_slots[h, :m] = victims
        n_miss[h] = m
    return miss_pages, miss_slots, n_miss


# --------------------------------------------------------------------------
# Attention over the slot table and the local window, and the LSE merge
# --------------------------------------------------------------------------

def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
           dtype: torch.dtype = torch.float64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact softmax attention of one query token, GQA by contiguous groups.

    q (Hq, D); k, v (T, Hk, D); scale D**-0.5.  Returns out (Hq, D) and
    lse (Hq,) = log sum exp of the scaled logits, both computed and returned
    in float64 so that the checker's own rounding stays far below the 1e-4
    float32 tolerance (with x8 / x10 outlier channels the logits reach ~50
    and a float32 dot product alone is uncertain by ~1e-5 relative).  This is what the
    reference obtains from flash_attn_with_kvcache(..., return_softmax_lse=True)
    at dram_attention/dram_attention.py:195-205 and :211-223 (for a single
    query row the causal flag changes nothing).  `dtype` = float32 gives the
    arithmetic a pure-PyTorch float32 path would use; only the timed CPU
    baseline asks for it, every check uses float64.
    """
    hq, d = q.shape
    t, hk, _ = k.shape
    rep = hq // hk
    qf = q.to(dtype).reshape(hk, rep, d)
    kf = k.to(dtype).permute(1, 0, 2)  # (Hk, T, D)
    vf = v.to(dtype).permute(1, 0, 2)
    logits = torch.bmm(qf, kf.transpose(1, 2)) * (d ** -0.5)  # (Hk, rep, T)
    lse = torch.logsumexp(logits, dim=-1)
    p = torch.exp(logits - lse[..., None])
    out = torch.bmm(p, vf)
    return out.reshape(hq, d), lse.reshape(hq)


def attend_tokens(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax attention of S query tokens with the causal mask aligned to the bottom-right
    corner: query i sees keys j <= T - S + i.

    q (S, Hq, D); k, v (T, Hk, D).  Returns out (S, Hq, D) and lse (S, Hq), float64.  This is
    what both flash_attn_with_kvcache(causal=True) calls of the reference compute when the
    generate stage gets several tokens (dram_attention/dram_attention.py:195-205 with
    cache_seqlens = all slot tokens, :211-223 with the S new rows appended first); the mask
    alignment is the documented behaviour of flash-attn >= 2.1.  On the prefix part it hides the
    last S-1-i tokens of the slot table from query i.
    """
    s_q, hq, d = q.shape
    t = k.shape[0]
    outs, lses = [], []
    for i in range(s_q):
        o, l = attend(q[i], k[:t - s_q + i + 1], v[:t - s_q + i + 1])
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def combine(prefix_out: torch.Tensor, suffix_out: torch.Tensor,
            prefix_lse: torch.Tensor, suffix_lse: torch.Tensor) -> torch.Tensor:
    """LSE-weighted merge, dram_attention/dram_attention.py:225-238."""
    lse = torch.logaddexp(prefix_lse, suffix_lse)
    wp = torch.exp(prefix_lse - lse)[:, None]
    ws = torch.exp(suffix_lse - lse)[:, None]
    return prefix_out * wp + suffix_out * ws


# --------------------------------------------------------------------------
# Stateful objects mirroring LRUCache and DRAMAttention
# --------------------------------------------------------------------------

@dataclass
class StepTrace:
    """What one generate step produced (everything the parity tests compare)."""
    scores: Optional[torch.Tensor]      # (1, Hk, rep, L) float32, None without LRU
    page_list: Optional[np.ndarray]     # (Hk, rep*k) int64
    miss_pages: Optional[np.ndarray]
    miss_slots: Optional[np.ndarray]
    n_miss: Optional[np.ndarray]
    out: torch.Tensor                   # (Hq, D) float64


class OracleLRUCache:
    """State and behaviour of dram_attention/lru_cache.py:40-265 on the CPU."""

    def __init__(self, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                 top_k: int, lru_hbm_cache_size: Optional[int] = None,
                 hbm_kv_cache_fraction: float = 0.2):
        assert k_cache.shape == v_cache.shape, "Key and value cache shapes must match."
        hk, length, d = k_cache.shape
        assert length % page_size == 0, "KV cache size must be divisible by page size."
        self.page_size = page_size
        self.num_kv_heads = hk
        self.head_dim = d
        self.num_dram_pages = length // page_size
        self.num_hbm_pages = (int(self.num_dram_pages * hbm_kv_cache_fraction)
                              if lru_hbm_cache_size is None
                              else lru_hbm_cache_size // page_size)
        assert self.num_hbm_pages <= self.num_dram_pages, \
            "HBM cache size must be smaller than DRAM cache size."
        self.top_k = top_k
        self.chunk_min_max = page_minmax(k_cache, self.num_dram_pages)
        ld, nh, p = self.num_dram_pages, self.num_hbm_pages, page_size
        # lru_cache.py:121-142: page layout (P, 2, D), token-major, K then V
        dram = torch.empty(hk, ld, p, 2, d, dtype=k_cache.dtype)
        dram[..., 0, :] = k_cache.reshape(hk, ld, p, d)
        dram[..., 1, :] = v_cache.reshape(hk, ld, p, d)
        self.dram_kv_cache = dram.reshape(hk, ld, p * 2 * d)
        # lru_cache.py:192-209: warm start with the rightmost pages, times 0
        self.hbm_kv_cache = self.dram_kv_cache[:, ld - nh:].clone()
        self.page_access_time = np.zeros((hk, nh), dtype=np.int64)
        self.d2h = np.full((hk, ld), -1, dtype=np.int64)
        self.d2h[:, ld - nh:] = np.arange(nh)[None]
        self.h2d = np.tile(np.arange(ld - nh, ld)[None], (hk, 1)).astype(np.int64)
        self.current_step = 0
        self.sequential = False

    def load_(self, page_list: np.ndarray):
        """lru_cache.py:211-240."""
        self.current_step += 1
        fn = lru_walk if self.sequential else lru_vectorised
        dram = self.dram_kv_cache
        mp, ms, nm = fn(page_list, self.d2h, self.h2d, self.page_access_time,
                        self.current_step)
        for h in range(self.num_kv_heads):
            m = int(nm[h])
            if m:
                self.hbm_kv_cache[h, torch.from_numpy(ms[h, :m])] = \
                    dram[h, torch.from_numpy(mp[h, :m])]
        return mp, ms, nm

    def kv_views(self):
        c = self.hbm_kv_cache.view(self.num_kv_heads,
                                   self.num_hbm_pages * self.page_size, 2, self.head_dim)
        return c[:, :, 0], c[:, :, 1]

    def get_kv_cache_(self, q: torch.Tensor):
        """lru_cache.py:242-265.  q is (1, S, Hq, D)."""
        scores = scores_by_query_head(q, self.chunk_min_max)
        idx = select_pages(scores, self.top_k)
        page_list = build_page_list(idx).numpy()
        mp, ms, nm = self.load_(page_list)
        return scores, page_list, mp, ms, nm


class OracleDRAMAttention:
    """dram_attention/dram_attention.py:31-238 (generate stage) on the CPU."""

    def __init__(self, max_output_length: int, lru_hbm_cache_size: int,
                 local_cache_size: int, page_size: int, top_k: int,
                 n_kv_heads: int, head_dim: int, dtype: torch.dtype = torch.float32):
        self.max_output_length = max_output_length
        self.page_size = page_size
        self.dram_kv_cache_size = None
        self.lru_hbm_cache_size = lru_hbm_cache_size
        self.local_cache_size = local_cache_size
        self.top_k = top_k
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        shape = (local_cache_size + max_output_length, n_kv_heads, head_dim)
        self.cache_k = torch.zeros(shape, dtype=dtype)
        self.cache_v = torch.zeros(shape, dtype=dtype)
        self.lru_cache: Optional[OracleLRUCache] = None
        self.static_k = self.static_v = None
        self.attn_dtype = torch.float64   # float32 only for the timed CPU baseline

    def init_cache(self, k_cache: torch.Tensor, v_cache: torch.Tensor):
        """dram_attention.py:65-105.  k_cache, v_cache are (1, S, Hk, D)."""
        bsz, seqlen, h, d = k_cache.shape
        assert bsz == 1, "Only support batch size 1"
        dram = seqlen - self.local_cache_size + self.page_size
        self.dram_kv_cache_size = dram // self.page_size * self.page_size
        n_local = seqlen - self.dram_kv_cache_size
        self.cache_k[:n_local] = k_cache[0, self.dram_kv_cache_size:]
        self.cache_v[:n_local] = v_cache[0, self.dram_kv_cache_size:]
        dk = k_cache[0, :self.dram_kv_cache_size].transpose(0, 1)
        dv = v_cache[0, :self.dram_kv_cache_size].transpose(0, 1)
        if self.dram_kv_cache_size > self.lru_hbm_cache_size:
            self.lru_cache = OracleLRUCache(dk, dv, self.page_size,
                                            self.top_k // self.page_size,
                                            self.lru_hbm_cache_size)
        else:
            self.lru_cache = None
            self.static_k, self.static_v = dk.contiguous(), dv.contiguous()

    def generate(self, xq: torch.Tensor, xk: torch.Tensor, xv: torch.Tensor,
                 start_pos: int) -> StepTrace:
        """dram_attention.py:144-177.  xq (1,S,Hq,D); xk, xv (1,S,Hk,D).  `out` of the trace
        is (Hq, D) for one token and (S, Hq, D) for several."""
        assert xq.shape[0] == 1, "Only support batch size 1"
        s_q = xq.shape[1]
        if self.lru_cache is not None:
            scores, page_list, mp, ms, nm = self.lru_cache.get_kv_cache_(xq)
            pk, pv = self.lru_cache.kv_views()
        else:
            scores = page_list = mp = ms = nm = None
            pk, pv = self.static_k, self.static_v
        t = int(start_pos) - self.dram_kv_cache_size
        self.cache_k[t:t + s_q] = xk[0]
        self.cache_v[t:t + s_q] = xv[0]
        if s_q == 1:
            q = xq[0, 0]
            po, plse = attend(q, pk.transpose(0, 1), pv.transpose(0, 1), self.attn_dtype)
            so, slse = attend(q, self.cache_k[:t + 1], self.cache_v[:t + 1], self.attn_dtype)
            out = combine(po, so, plse, slse)
        else:
            po, plse = attend_tokens(xq[0], pk.transpose(0, 1), pv.transpose(0, 1))
            so, slse = attend_tokens(xq[0], self.cache_k[:t + s_q], self.cache_v[:t + s_q])
            out = torch.stack([combine(po[i], so[i], plse[i], slse[i]) for i in range(s_q)])
        return StepTrace(scores, page_list, mp, ms, nm, out)

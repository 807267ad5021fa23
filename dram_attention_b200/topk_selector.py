"""Quest top-k page selection on per-page key min/max summaries."""

from __future__ import annotations

import torch

from . import _native
from .max_ip import score_pages_


def build_pages_(k: torch.Tensor, v: torch.Tensor, page_size: int, dram_pages, summaries, slots,
                 n_slots: int) -> None:
    """Enqueue the cache-construction pass for k, v of shape (Hk, length, D) (any
    strides with a unit channel stride).  Any of the three outputs may be None."""
    hk, length, d = k.shape
    assert k.stride(2) == 1 and v.stride(2) == 1 and k.stride() == v.stride()
    n_pages = length // page_size
    ptr = lambda t: 0 if t is None else t.data_ptr()
    _native.check(_native.lib().da_build_pages(
        k.data_ptr(), v.data_ptr(), k.stride(1), k.stride(0), ptr(dram_pages), ptr(summaries), ptr(slots),
        hk, n_pages, n_slots, page_size, d, _native.dtype_code(k.dtype), _native.stream_ptr()),
        "da_build_pages")


class IPUpperboundTopKSelector:
    """Inner-product upper-bound top-k selector; mirrors the reference class
    (dram_attention/topk_selector.py:10-61).

    `chunk_min_max` is (num_heads, num_pages, 2, head_dim) in the dtype of the keys,
    [..., 0, :] = per-page channel minimum, [..., 1, :] = maximum."""

    def __init__(self, k_cache: torch.Tensor, num_pages: int, device="cuda", _summaries=None):
        num_heads, dram_kv_cache_size, head_dim = k_cache.shape
        self.num_kv_heads = num_heads
        assert dram_kv_cache_size % num_pages == 0, "Cache size must be divisible by num_pages."
        self.num_pages = num_pages
        self.device = torch.device(device)
        if _summaries is not None:
            self.chunk_min_max = _summaries
        else:
            page_size = dram_kv_cache_size // num_pages
            k_dev = k_cache.to(device=device)
            _native.require_cuda(k_dev, "k_cache")
            self.chunk_min_max = torch.empty(num_heads, num_pages, 2, head_dim, dtype=k_cache.dtype,
                                             device=device)
            with torch.cuda.device(k_dev.device):
                build_pages_(k_dev, k_dev, page_size, None, self.chunk_min_max, None, 0)
        self._buffers = {}

    def _workspace(self, seq_len: int, rep: int, k: int):
        key = (seq_len, rep, k)
        ws = self._buffers.get(key)
        if ws is None:
            dev = self.chunk_min_max.device
            scores = torch.empty(seq_len, self.num_kv_heads * rep, self.num_pages, dtype=torch.float32,
                                 device=dev)
            page_list = torch.empty(self.num_kv_heads, seq_len * rep * k, dtype=torch.int32, device=dev)
            ws = self._buffers[key] = (scores, page_list)
        return ws

    def score_(self, q: torch.Tensor, k: int):
        """Enqueue the page scorer for q (1, S, Hq, D); returns the float32 score
        buffer (S, Hq, L) (reused by the next call)."""
        bsz, seq_len, num_q_heads, head_dim = q.shape
        assert bsz == 1, f"Only batch size 1 is supported, but got batch size {bsz}"
        assert num_q_heads % self.num_kv_heads == 0
        _native.require_cuda(q, "q")
        assert q.dtype == self.chunk_min_max.dtype, "query dtype must match the key summaries"
        rep = num_q_heads // self.num_kv_heads
        scores, _ = self._workspace(seq_len, rep, min(k, self.num_pages))
        qc = q if q.is_contiguous() else q.contiguous()
        # chunk_min_max comes from aminmax over real keys, so min <= max holds
        score_pages_(qc, self.chunk_min_max, scores, seq_len, self.num_kv_heads, rep, ordered=True)
        return scores

    def select_(self, seq_len: int, rep: int, k: int, sm_budget: int = 0):
        """Enqueue the top-k selection on the scores of the last score_ call with the
        same (seq_len, rep, k); returns the int32 page list (Hk, S*rep*k).  `sm_budget`: SMs the
        selection may count on (0 = all), see da_topk_pages_wide."""
        k = min(k, self.num_pages)
        scores, page_list = self._workspace(seq_len, rep, k)
        _native.check(_native.lib().da_topk_pages_wide(
            scores.data_ptr(), page_list.data_ptr(), seq_len, self.num_kv_heads, rep, self.num_pages, k,
            int(sm_budget), _native.stream_ptr()), "da_topk_pages_wide")
        return page_list

    def page_list_(self, q: torch.Tensor, k: int):
        """Scores and selection for q (1, S, Hq, D).  Returns (scores, page_list):
        float32 (S, Hq, L) and int32 (Hk, S*rep*k) where row hk holds, for every token
        and every query head of the group in order, its k pages by descending score
        (ties by ascending page id).  Both tensors are reused by the next call."""
        scores = self.score_(q, k)
        seq_len, rep = q.shape[1], q.shape[2] // self.num_kv_heads
        return scores, self.select_(seq_len, rep, k)

    def top_k(self, q: torch.Tensor, k: int) -> torch.Tensor:
        """Top-k page ids for each token and query head: int64 (S, Hk, rep, k), as
        the reference's top_k (dram_attention/topk_selector.py:37-61)."""
        bsz, seq_len, num_q_heads, _ = q.shape
        with torch.cuda.device(q.device):
            _, page_list = self.page_list_(q, k)
        rep = num_q_heads // self.num_kv_heads
        kk = page_list.shape[1] // (seq_len * rep)
        return page_list.view(self.num_kv_heads, seq_len, rep, kk).swapaxes(0, 1).to(torch.int64)

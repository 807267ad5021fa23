"""HBM slot table in front of a KV cache that lives in pinned host DRAM.

Mirrors the reference's LRUCache / DummyCache / CacheOutput
(dram_attention/lru_cache.py) on top of the CUDA kernels: one kernel for the LRU
table update, one gather-copy kernel for the missed pages."""

from __future__ import annotations

from typing import NamedTuple, Optional

import torch

from . import _native
from .topk_selector import IPUpperboundTopKSelector, build_pages_


class CacheOutput(NamedTuple):
    k_cache: torch.Tensor
    v_cache: torch.Tensor


class DummyCache(torch.nn.Module):
    """The whole prefix resident in HBM (no scoring, no eviction); used when the
    DRAM prefix is not larger than the HBM cache (dram_attention/lru_cache.py:24-37).

    The prefix is stored in the slot payload layout (Hk, tokens, 2, D) so the same
    attention kernel reads it."""

    def __init__(self, k_cache: torch.Tensor, v_cache: torch.Tensor, device: str, page_size: int = 16,
                 *args, **kvargs):
        super().__init__()
        hk, length, d = k_cache.shape
        k_dev, v_dev = k_cache.to(device=device), v_cache.to(device=device)
        _native.require_cuda(k_dev, "k_cache")
        self.num_kv_heads, self.head_dim, self.num_tokens = hk, d, length
        self.register_buffer("hbm_kv_cache", torch.empty(hk, max(length, 1), 2 * d, dtype=k_cache.dtype,
                                                         device=device))
        if length:
            with torch.cuda.device(k_dev.device):
                # one "page" per token: the payload layout is token-major either way
                build_pages_(k_dev, v_dev, 1, None, None, self.hbm_kv_cache, length)

    def kv_views(self) -> CacheOutput:
        c = self.hbm_kv_cache.view(self.num_kv_heads, -1, 2, self.head_dim)[:, :self.num_tokens]
        return CacheOutput(k_cache=c[:, :, 0], v_cache=c[:, :, 1])

    def get_kv_cache_(self, q: torch.Tensor) -> CacheOutput:
        return self.kv_views()


class LRUCache(torch.nn.Module):
    """LRU-managed HBM page cache over a paged KV cache in pinned DRAM
    (dram_attention/lru_cache.py:40-265).

    Attributes (names as in the reference; the integer tables are int32 here):
        current_step: int32 (1,), a view of the per-head step counters.
        dram_kv_cache: pinned host (num_kv_heads, num_dram_pages, page_size*2*head_dim);
            inside a page the layout is (page_size, 2, head_dim): token-major, key then value.
        hbm_kv_cache: device (num_kv_heads, num_hbm_pages, page_size*2*head_dim), same row format.
        page_access_time: int32 (num_kv_heads, num_hbm_pages), step of last use.
        dram_page_to_hbm_page_mapping: int32 (num_kv_heads, num_dram_pages), -1 = not resident.
        hbm_page_to_dram_page_mapping: int32 (num_kv_heads, num_hbm_pages).
    """

    def __init__(self, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, top_k: int,
                 lru_hbm_cache_size: Optional[int] = None, hbm_kv_cache_fraction: float = 0.2,
                 device: str = "cuda", _share: Optional["LRUCache"] = None):
        super().__init__()
        if _share is not None:
            self._init_shared(_share, top_k)
            return
        assert k_cache.shape == v_cache.shape, "Key and value cache shapes must match."
        num_kv_heads, dram_kv_cache_size, head_dim = k_cache.shape
        dtype = k_cache.dtype
        assert dram_kv_cache_size % page_size == 0, "KV cache size must be divisible by page size."
        num_dram_pages = dram_kv_cache_size // page_size
        num_hbm_pages = (int(num_dram_pages * hbm_kv_cache_fraction) if lru_hbm_cache_size is None
                         else lru_hbm_cache_size // page_size)
        assert num_hbm_pages <= num_dram_pages, "HBM cache size must be smaller than DRAM cache size."

        self.page_size = page_size
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.num_dram_pages = num_dram_pages
        self.num_hbm_pages = num_hbm_pages
        self.top_k = top_k
        page_dim = page_size * 2 * head_dim

        k_dev, v_dev = k_cache.to(device=device), v_cache.to(device=device)
        _native.require_cuda(k_dev, "k_cache")
        dev = k_dev.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.register_buffer("step_counters", torch.zeros(num_kv_heads, **i32))
        self.register_buffer("dram_kv_cache", torch.empty(num_kv_heads, num_dram_pages, page_dim, dtype=dtype,
                                                          device="cpu", pin_memory=True), persistent=False)
        self.register_buffer("hbm_kv_cache", torch.empty(num_kv_heads, num_hbm_pages, page_dim, dtype=dtype,
                                                         device=dev))
        self.register_buffer("page_access_time", torch.zeros(num_kv_heads, num_hbm_pages, **i32))
        # -1: the DRAM page is not in HBM; otherwise the slot that holds it
        self.register_buffer("dram_page_to_hbm_page_mapping",
                             torch.full((num_kv_heads, num_dram_pages), -1, **i32))
        self.register_buffer("hbm_page_to_dram_page_mapping",
                             torch.arange(num_dram_pages - num_hbm_pages, num_dram_pages, **i32)
                             .repeat(num_kv_heads, 1))
        # warm start: the rightmost pages are resident, slot s <- page Ld - Nh + s, times 0
        self.dram_page_to_hbm_page_mapping[:, num_dram_pages - num_hbm_pages:] = \
            torch.arange(num_hbm_pages, **i32)[None]
        summaries = torch.empty(num_kv_heads, num_dram_pages, 2, head_dim, dtype=dtype, device=dev)
        with torch.cuda.device(dev):
            # one pass: pinned DRAM pages, page summaries and the resident slots
            build_pages_(k_dev, v_dev, page_size, self.dram_kv_cache, summaries, self.hbm_kv_cache,
                         num_hbm_pages)
            torch.cuda.current_stream().synchronize()  # k_dev/v_dev may be temporaries
        self.top_k_selector = IPUpperboundTopKSelector(k_cache, num_dram_pages, device=dev,
                                                       _summaries=summaries)
        self._init_tables(dev)

    @classmethod
    def sharing_dram_of(cls, other: "LRUCache", top_k: Optional[int] = None) -> "LRUCache":
        """A second cache over the SAME pinned DRAM pages and page summaries as `other` (neither is
        copied), with a slot table, LRU tables and queue of its own in the warm-start state.  For
        stacks of layers that are fed the same synthetic prefix: the host memory is paid once,
        everything a decode step reads or writes on the device is per layer."""
        return cls(None, None, other.page_size, other.top_k if top_k is None else top_k, _share=other)

    def _init_shared(self, other: "LRUCache", top_k: int) -> None:
        self.page_size, self.num_kv_heads, self.head_dim = other.page_size, other.num_kv_heads, other.head_dim
        self.num_dram_pages, self.num_hbm_pages, self.top_k = other.num_dram_pages, other.num_hbm_pages, top_k
        dev = other.hbm_kv_cache.device
        i32 = dict(dtype=torch.int32, device=dev)
        hk, ld, nh = self.num_kv_heads, self.num_dram_pages, self.num_hbm_pages
        self.register_buffer("step_counters", torch.zeros(hk, **i32))
        self.register_buffer("dram_kv_cache", other.dram_kv_cache, persistent=False)
        self.register_buffer("hbm_kv_cache", torch.empty_like(other.hbm_kv_cache))
        # warm start: the rightmost pages, read back from the shared DRAM pages
        self.hbm_kv_cache.copy_(other.dram_kv_cache[:, ld - nh:], non_blocking=True)
        self.register_buffer("page_access_time", torch.zeros(hk, nh, **i32))
        self.register_buffer("dram_page_to_hbm_page_mapping", torch.full((hk, ld), -1, **i32))
        self.register_buffer("hbm_page_to_dram_page_mapping", torch.arange(ld - nh, ld, **i32).repeat(hk, 1))
        self.dram_page_to_hbm_page_mapping[:, ld - nh:] = torch.arange(nh, **i32)[None]
        self.top_k_selector = IPUpperboundTopKSelector(
            torch.empty(hk, ld * self.page_size, self.head_dim, dtype=other.hbm_kv_cache.dtype, device="meta"),
            ld, device=dev, _summaries=other.top_k_selector.chunk_min_max)
        self._init_tables(dev)

    def _init_tables(self, dev) -> None:
        num_kv_heads, num_hbm_pages = self.num_kv_heads, self.num_hbm_pages
        i32 = dict(dtype=torch.int32, device=dev)
        self.register_buffer("status", torch.zeros(1, **i32), persistent=False)
        # slot -> DRAM page whose payload is still to be brought in (-1: slot is up to date);
        # maintained by the LRU kernel, consumed by the attention kernel that fetches on the fly
        self.register_buffer("slot_source", torch.full((num_kv_heads, num_hbm_pages), -1, **i32),
                             persistent=False)
        # Eviction queue: evict_order[h] (copy evict_flip[h]) lists the slots of head h in eviction
        # order ((time, slot) ascending; after the warm start every time is 0, so the identity).  The
        # LRU update takes its victims from the head of the queue and writes the other copy for the
        # following step.  The first n_evictable[h] entries are the FRONT: the slots the first
        # launch of the two-launch attention leaves out because the update running beside it may
        # evict them (`split_cap` of them); evict_redo[h] is set when a victim lay beyond the front
        # (the second launch then covers the whole head).  All of it lives on the device, so a
        # captured step stays consistent whatever ran between two replays.
        self.split_cap = min(self.default_split_cap, max(1, num_hbm_pages // 4))
        self.register_buffer("evict_order", torch.arange(num_hbm_pages, **i32).repeat(2, num_kv_heads, 1),
                             persistent=False)    # two copies; evict_flip[h] names the current one
        self.register_buffer("n_evictable", torch.full((2, num_kv_heads), self.split_cap, **i32),
                             persistent=False)
        self.register_buffer("evict_flip", torch.zeros(num_kv_heads, **i32), persistent=False)
        # row 0: redo flag of the last update; row 1: pages missed so far; row 2: updates that set the flag
        self.register_buffer("evict_redo", torch.zeros(3, num_kv_heads, **i32), persistent=False)
        self._miss = {}

    # slots per head in the eviction front (a steady decode step misses a handful of pages per head)
    default_split_cap = 64
    # a head that misses at most this many pages in a step has them copied by the LRU kernel itself
    inline_fetch_max = 16

    @property
    def current_step(self) -> torch.Tensor:
        return self.step_counters[:1]

    def _miss_buffers(self, list_len: int):
        bufs = self._miss.get(list_len)
        if bufs is None:
            dev = self.hbm_kv_cache.device
            mk = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
            bufs = self._miss[list_len] = (mk(self.num_kv_heads, list_len), mk(self.num_kv_heads, list_len),
                                           mk(self.num_kv_heads))
        return bufs

    def update_tables_(self, page_list: torch.Tensor, advance_split: bool = True,
                       inline_fetch: bool = False, after_selection: bool = False) -> None:
        """Enqueue the LRU table update for an int32 page list (Hk, list_len): step
        counters, hit stamps, victim choice, both maps, the device-side miss list, and the
        eviction front for the following step (written into the copy of evict_order /
        n_evictable that evict_flip does not name).  `advance_split=False` when the two-launch
        attention follows: its second launch makes the new front current when both are done;
        otherwise the update does it itself.  With `inline_fetch` the kernel also copies the
        pages of heads that miss only a few (at most `inline_fetch_max`) into their slots; the
        others are marked in slot_source for the attention kernel that fetches on the fly.
        `after_selection`: the launch before this one in the stream is the selection kernel that wrote
        `page_list` (the generate step's chain); the update then reads its tables while that launch still
        runs.  Leave it False after anything else (another update, an attention launch)."""
        list_len = page_list.shape[1]
        miss_pages, miss_slots, n_miss = self._miss_buffers(list_len)
        _native.check(_native.lib().da_lru_update(
            page_list.data_ptr(), list_len, self.dram_page_to_hbm_page_mapping.data_ptr(),
            self.num_dram_pages, self.hbm_page_to_dram_page_mapping.data_ptr(),
            self.page_access_time.data_ptr(), self.num_hbm_pages, self.step_counters.data_ptr(),
            self.num_kv_heads, miss_pages.data_ptr(), miss_slots.data_ptr(), n_miss.data_ptr(),
            self.slot_source.data_ptr(), self.evict_order.data_ptr(), self.n_evictable.data_ptr(),
            self.evict_flip.data_ptr(), self.evict_redo.data_ptr(), int(self.split_cap),
            (1 if advance_split else 0) | (2 if after_selection else 0),
            self.dram_kv_cache.data_ptr() if inline_fetch else 0,
            self.hbm_kv_cache.data_ptr() if inline_fetch else 0,
            self.dram_kv_cache.shape[2] * self.dram_kv_cache.element_size(),
            int(self.inline_fetch_max) if inline_fetch else 0,
            self.status.data_ptr(), _native.stream_ptr()), "da_lru_update")

    def fetch_(self, list_len: int) -> None:
        """Enqueue the gather-copy of the pages the last update_tables_ found missing."""
        miss_pages, miss_slots, n_miss = self._miss_buffers(list_len)
        page_bytes = self.dram_kv_cache.shape[2] * self.dram_kv_cache.element_size()
        _native.check(_native.lib().da_fetch_pages(
            self.dram_kv_cache.data_ptr(), self.hbm_kv_cache.data_ptr(), miss_pages.data_ptr(),
            miss_slots.data_ptr(), n_miss.data_ptr(), list_len, self.num_kv_heads, self.num_dram_pages,
            self.num_hbm_pages, page_bytes, _native.stream_ptr()), "da_fetch_pages")

    def _load_int32_(self, page_list: torch.Tensor) -> None:
        self.update_tables_(page_list)
        self.fetch_(page_list.shape[1])

    def last_miss_counts(self, list_len: int) -> torch.Tensor:
        """int32 (Hk,) device tensor: pages fetched per head by the last step."""
        return self._miss_buffers(list_len)[2]

    def kv_views(self) -> CacheOutput:
        c = self.hbm_kv_cache.view(self.num_kv_heads, self.num_hbm_pages * self.page_size, 2, self.head_dim)
        k_cache, v_cache = c.unbind(dim=2)
        return CacheOutput(k_cache=k_cache, v_cache=v_cache)

    def load_(self, top_k_dram_page_index: torch.Tensor) -> CacheOutput:
        """Make the listed DRAM pages resident (in place) and return the slot table
        as strided key and value views, each (num_kv_heads, num_hbm_pages*page_size, head_dim)
        (dram_attention/lru_cache.py:211-240)."""
        idx = top_k_dram_page_index
        _native.require_cuda(idx, "top_k_dram_page_index")
        assert idx.dim() == 2 and idx.shape[0] == self.num_kv_heads
        if idx.dtype != torch.int32 or not idx.is_contiguous():
            idx = idx.to(torch.int32).contiguous()
        with torch.cuda.device(idx.device):
            self._load_int32_(idx)
        return self.kv_views()

    def get_kv_cache_(self, q: torch.Tensor) -> CacheOutput:
        """Score the pages for q (1, S, Hq, D), select top_k pages per query head,
        make them resident, return the slot table (dram_attention/lru_cache.py:242-265)."""
        with torch.cuda.device(q.device):
            _, page_list = self.top_k_selector.page_list_(q, self.top_k)
            self._load_int32_(page_list)
        return self.kv_views()

    def check_status(self) -> None:
        """Synchronises; raises if a kernel flagged a problem since the last check."""
        bits = int(self.status.item())
        if bits:
            self.status.zero_()
            raise RuntimeError("dram_attention_b200 device status: " + _native.status_message(bits))

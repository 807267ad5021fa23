"""DRAM Attention operator: same constructor and call signature as the reference's
DRAMAttention (dram_attention/dram_attention.py:6-238); the generate stage runs on
hand-written sm_100a kernels."""

from __future__ import annotations

from typing import Optional

import torch

from . import _native
from .lru_cache import DummyCache, LRUCache


class DRAMAttention(torch.nn.Module):
    """Long-context decode attention with the prefix KV cache in host DRAM.

    `fused_fetch` (class attribute, default True): pages that miss the slot table are read
    from DRAM by the attention kernel itself and written through to their slots, instead of
    by a separate gather-copy launch before it.  Results are identical either way.

    Two caches: a local window of the most recent tokens in HBM, and the prefix in
    pinned DRAM behind an LRU-managed HBM slot table.  Every generate step scores
    all prefix pages against the query, makes the top pages resident and attends
    over the whole slot table plus the local window.

    Args:
        max_output_length: tokens that may be generated after the prefill.
        lru_hbm_cache_size: size of the HBM slot table, in tokens.
        local_cache_size: size of the local window, in tokens.
        page_size: tokens per page.
        top_k: tokens (not pages) selected per query head and step.
        n_kv_heads, head_dim: KV head count and channel count.
        device: CUDA device of all device-side state.
        dtype: element type of the caches (bfloat16, float16 or float32).
    """

    def __init__(self, max_output_length: int, lru_hbm_cache_size: int, local_cache_size: int,
                 page_size: int, top_k: int, n_kv_heads: int, head_dim: int, device: str = "cuda",
                 dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.max_output_length = max_output_length
        self.page_size = page_size
        self.dram_kv_cache_size = None  # set by init_cache
        self.lru_hbm_cache_size = lru_hbm_cache_size
        self.local_cache_size = local_cache_size
        self.top_k = top_k
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        self.num_page = self.lru_hbm_cache_size // self.page_size
        self.device = device
        _native.dtype_code(dtype)
        _native.lib()  # fail here, loudly, if the CUDA library has not been built

        cache_shape = (1, local_cache_size + max_output_length, n_kv_heads, head_dim)
        self.register_buffer("cache_k", torch.zeros(cache_shape, device=device, dtype=dtype))
        self.register_buffer("cache_v", torch.zeros(cache_shape, device=device, dtype=dtype))
        self.lru_cache = None
        self._ws = {}
        self._can_fuse = False
        self._can_overlap = False
        self._overlap_ok = {}
        self._side = None
        self._prefill_status = None

    # stage="prefill": this package's tcgen05 kernel where it applies (16-bit, head_dim 128)
    prefill_kernel = True
    fused_fetch = True
    # Two attention launches per step: the first (local window + every slot outside the eviction
    # front) runs on a side stream beside scoring, selection and LRU update; the second (the few
    # slots of the front, with the miss fetch) follows the update without waiting for the first.
    overlap = True
    # ... and, when the step is being captured into a CUDA graph, that first launch forks off before
    # the page scorer rather than after it
    fork_before_score = True
    # CTAs per KV head of the two launches (0: the library's defaults)
    phase1_ctas = 0
    phase2_ctas = 0
    # KV-head sharding (set by KVHeadShardedDRAMAttention): (peer buffer array, step counter, rank, world, bytes
    # per rank) of the peer gather; the attention launches of a one-token step then send the output rows
    peer_push = None
    selection_sm_budget = 0    # SMs the selection may count on beside the first attention launch of the
                               # two-launch step; 0 = 148 minus that launch's CTAs (one SM each)

    # ---- cache construction ---------------------------------------------------
    def init_cache(self, k_cache: torch.Tensor, v_cache: torch.Tensor):
        """Split a prefill KV cache (1, S, Hk, D) into the DRAM prefix and the local
        window (dram_attention/dram_attention.py:65-105)."""
        bsz, seqlen, H, D = k_cache.shape
        assert bsz == 1, "Only support batch size 1"
        dram_kv_cache_size = seqlen - self.local_cache_size + self.page_size
        self.dram_kv_cache_size = dram_kv_cache_size // self.page_size * self.page_size
        L = seqlen - self.dram_kv_cache_size
        self.cache_k[:, :L].copy_(k_cache[:, self.dram_kv_cache_size:], non_blocking=True)
        self.cache_v[:, :L].copy_(v_cache[:, self.dram_kv_cache_size:], non_blocking=True)

        dram_k_cache = k_cache[:, :self.dram_kv_cache_size]
        dram_v_cache = v_cache[:, :self.dram_kv_cache_size]
        if self.dram_kv_cache_size > self.lru_hbm_cache_size:
            self.lru_cache = LRUCache(
                k_cache=dram_k_cache[0].transpose(0, 1), v_cache=dram_v_cache[0].transpose(0, 1),
                page_size=self.page_size, top_k=self.top_k // self.page_size,
                lru_hbm_cache_size=self.lru_hbm_cache_size, device=self.device)
            # the kernel that fetches on the fly needs its 16-token units inside one page
            self._can_fuse = self.page_size % 16 == 0
            self._can_overlap = self._can_fuse   # refined per GQA group size at the first generate call
            self._overlap_ok = {}
        else:
            self._can_fuse = False
            self._can_overlap = False
            self.lru_cache = DummyCache(
                k_cache=dram_k_cache[0].transpose(0, 1), v_cache=dram_v_cache[0].transpose(0, 1),
                device=self.device, page_size=self.page_size)

    def init_cache_sharing(self, other: "DRAMAttention") -> None:
        """Initialise this operator as `init_cache` would with the prefill KV `other` was given,
        WITHOUT a second copy of the DRAM prefix: the pinned pages and their summaries are shared
        with `other`, while the slot table, the LRU state and the local window are this operator's
        own (in the state right after cache construction).  For synthetic stacks in which several
        layers are fed the same prefix."""
        assert isinstance(other.lru_cache, LRUCache), "the other operator has no DRAM-backed cache"
        assert (self.page_size, self.n_kv_heads, self.head_dim, self.lru_hbm_cache_size, self.local_cache_size) == \
            (other.page_size, other.n_kv_heads, other.head_dim, other.lru_hbm_cache_size, other.local_cache_size)
        self.dram_kv_cache_size = other.dram_kv_cache_size
        n = min(self.cache_k.shape[1], other.cache_k.shape[1], other.local_cache_size)
        self.cache_k[:, :n].copy_(other.cache_k[:, :n])
        self.cache_v[:, :n].copy_(other.cache_v[:, :n])
        self.lru_cache = LRUCache.sharing_dram_of(other.lru_cache, top_k=self.top_k // self.page_size)
        self._can_fuse = self.page_size % 16 == 0
        self._can_overlap = self._can_fuse
        self._overlap_ok = {}

    # ---- forward ------------------------------------------------------------------
    def forward(self, xq: torch.Tensor, xk: torch.Tensor, xv: torch.Tensor, *, start_pos, stage: str,
                freqs_cis: Optional[torch.Tensor] = None):
        """xq (1, s, Hq, D), xk/xv (1, s, Hk, D).  `stage` is "prefill" (dense causal
        attention, then init_cache) or "generate" (one new token; start_pos is its
        absolute position, a Python int or an int32 CUDA tensor of shape (1,)).  Generate also
        takes s > 1 tokens (appended at start_pos .. start_pos + s - 1), as the reference does for
        the unaligned tail of a prompt.

        `freqs_cis` (not in the reference's signature): when given, xq and xk are the caller's
        projections BEFORE the rotary embedding and the operator applies it itself, in one launch
        chained to the scorer (rotate_), instead of the caller's apply_rotary_emb
        (evaluation/dram-attention/model.py:201).  Shape (s, D / 2) complex64, or (s, D / 2, 2)
        float32 (cos, sin), on the device: the rows of the call's positions."""
        bsz, seqlen, H, D = xq.shape
        assert bsz == 1, "Only support batch size 1"
        if freqs_cis is not None:
            xq, xk = self.rotate_(xq, xk, freqs_cis)
        if stage == "prefill":
            output = self._prefill_attention(xq, xk, xv)
            self.init_cache(xk, xv)
            return output
        elif stage == "generate":
            return self._generate(xq, xk, xv, start_pos)
        else:
            raise RuntimeError(f"Unsupported stage: {stage}")

    def rotate_(self, xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor):
        """Enqueue the rotary embedding of xq (1, s, Hq, D) and xk (1, s, Hk, D) with freqs_cis
        (s, D / 2) and return the rotated pair (new tensors).  Same arithmetic as the reference
        caller's apply_rotary_emb (evaluation/dram-attention/model.py:125-135)."""
        _native.require_cuda(xq, "xq")
        bsz, seqlen, n_q_heads, D = xq.shape
        assert xk.shape[:2] == xq.shape[:2] and xk.shape[3] == D and xk.dtype == xq.dtype and D % 2 == 0
        f = torch.view_as_real(freqs_cis) if freqs_cis.is_complex() else freqs_cis
        assert f.dtype == torch.float32 and tuple(f.shape) == (seqlen, D // 2, 2), \
            f"freqs_cis must be ({seqlen}, {D // 2}) complex64, got {tuple(freqs_cis.shape)} {freqs_cis.dtype}"
        f = f if f.is_contiguous() else f.contiguous()
        xq = xq if xq.is_contiguous() else xq.contiguous()
        xk = xk if xk.is_contiguous() else xk.contiguous()
        with torch.cuda.device(xq.device):
            q_out, k_out = torch.empty_like(xq), torch.empty_like(xk)
            _native.check(_native.lib().da_rope_qk(
                xq.data_ptr(), xk.data_ptr(), f.data_ptr(), q_out.data_ptr(), k_out.data_ptr(), bsz * seqlen,
                n_q_heads, xk.shape[2], D, _native.dtype_code(xq.dtype), _native.stream_ptr()), "da_rope_qk")
        return q_out, k_out

    def _prefill_attention(self, xq, xk, xv):
        """Dense causal attention of the prompt (the reference calls a third-party library
        here, dram_attention/dram_attention.py:136).  16-bit tensors with head_dim 128 on a CUDA
        device go through this package's tensor-core kernel (da_prefill_attention); other
        shapes (the float32 test configuration) use torch's scaled_dot_product_attention."""
        bsz, seqlen, n_q_heads, head_dim = xq.shape
        lib = _native.lib()
        if (self.prefill_kernel and xq.is_cuda and xq.dtype in (torch.bfloat16, torch.float16)
                and xk.dtype == xq.dtype and xv.dtype == xq.dtype
                and lib.da_prefill_attention_supported(head_dim, _native.dtype_code(xq.dtype))):
            q, k, v = (t if t.is_contiguous() else t.contiguous() for t in (xq, xk, xv))
            out = torch.empty_like(q)
            if self._prefill_status is None:
                self._prefill_status = torch.zeros(1, dtype=torch.int32, device=q.device)
            with torch.cuda.device(q.device):
                _native.check(lib.da_prefill_attention(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), seqlen, n_q_heads, k.shape[2],
                    head_dim, n_q_heads * head_dim, k.shape[2] * head_dim, _native.dtype_code(q.dtype),
                    self._prefill_status.data_ptr(), _native.stream_ptr()), "da_prefill_attention")
            return out
        q, k, v = (t.transpose(1, 2) for t in (xq, xk, xv))
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return out.transpose(1, 2).contiguous()

    def _workspace(self, rep: int, dev, seqlen: int = 1):
        ws = self._ws.get((rep, seqlen))
        if ws is None:
            lib = _native.lib()
            nbytes = max(lib.da_decode_attention_tokens_workspace_bytes(self.n_kv_heads, rep, self.head_dim, seqlen),
                         lib.da_decode_attention_phased_workspace_bytes(self.n_kv_heads, rep, self.head_dim))
            buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)  # counters start at zero
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            ws = self._ws[(rep, seqlen)] = (buf, nbytes, status)
        return ws

    def _generate(self, xq: torch.Tensor, xk: torch.Tensor, xv: torch.Tensor, start_pos):
        bsz, seqlen, n_q_heads, D = xq.shape
        assert self.lru_cache is not None, "init_cache (or a prefill) must come first"
        assert xk.shape[1] == seqlen and xv.shape[1] == seqlen
        _native.require_cuda(xq, "xq")
        assert xq.dtype == self.cache_k.dtype and xk.dtype == xq.dtype and xv.dtype == xq.dtype
        assert n_q_heads % self.n_kv_heads == 0 and D == self.head_dim
        rep = n_q_heads // self.n_kv_heads
        xq = xq if xq.is_contiguous() else xq.contiguous()
        xk = xk if xk.is_contiguous() else xk.contiguous()
        xv = xv if xv.is_contiguous() else xv.contiguous()
        with torch.cuda.device(xq.device):
            out = torch.empty_like(xq)
            if seqlen > 1:
                # several tokens: one scoring / selection / LRU update over all of them (list of
                # seqlen * rep * k pages per KV head), the gather-copy of the misses, then the
                # attention of every token over the same slot table
                self.lru_cache.get_kv_cache_(xq)
                self.attend_(xq, xk, xv, start_pos, out)
            elif self._can_overlap and self.fused_fetch and self.overlap and self._overlap_supported(rep, xq.dtype):
                self._generate_overlapped(xq, xk, xv, start_pos, out)
            elif self._can_fuse and self.fused_fetch:
                # score -> select -> LRU update -> attention that also brings in the misses
                lc = self.lru_cache
                _, page_list = lc.top_k_selector.page_list_(xq, lc.top_k)
                lc.update_tables_(page_list, inline_fetch=True, after_selection=True)
                self.attend_(xq, xk, xv, start_pos, out, fetch=True)
            else:
                # score -> select -> LRU update -> fetch (no-ops for a fully resident prefix)
                self.lru_cache.get_kv_cache_(xq)
                self.attend_(xq, xk, xv, start_pos, out)
        return out

    def _overlap_supported(self, rep: int, dtype) -> bool:
        ok = self._overlap_ok.get(rep)
        if ok is None:
            ok = self._overlap_ok[rep] = bool(_native.lib().da_decode_attention_phased_supported(
                self.n_kv_heads, rep, self.head_dim, _native.dtype_code(dtype), self.lru_cache.num_hbm_pages,
                self.page_size, self.cache_k.shape[1]))
        return ok

    def _generate_overlapped(self, xq, xk, xv, start_pos, out) -> None:
        """{ score -> select -> LRU update -> attention phase 2 }  ||  attention phase 1."""
        lc = self.lru_cache
        sel = lc.top_k_selector
        rep = xq.shape[2] // self.n_kv_heads
        if self._side is None:
            self._side = torch.cuda.Stream(device=xq.device)
            self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
        main = torch.cuda.current_stream()
        # Phase 1 needs nothing this step computes (only the split the previous step left), so it
        # forks off before the scorer: its CTAs move onto the SMs as the scorer's short CTAs leave
        # them.  The scorer is launched first so that the chain score -> select -> update is not
        # the one that waits for SMs.
        # Only inside a graph capture: a graph dispatches the scorer's CTAs ahead of phase 1's (node
        # order), whereas two eager launches that become ready together (a backlogged GPU) may be
        # dispatched either way round, and phase 1 first would starve the scorer of SMs.
        budget = self.selection_sm_budget or max(
            1, 148 - self.n_kv_heads * (self.phase1_ctas or min(20, max(1, 116 // self.n_kv_heads))))
        early = self.fork_before_score and torch.cuda.is_current_stream_capturing()
        if early:
            self._fork.record(main)
        sel.score_(xq, lc.top_k)
        if not early:
            self._fork.record(main)
            page_list = sel.select_(1, rep, lc.top_k, sm_budget=budget)     # ahead of phase 1, so that its CTAs find SMs free
        self._side.wait_event(self._fork)
        with torch.cuda.stream(self._side):
            self.attend_(xq, xk, xv, start_pos, out, phase=1)
            self._join.record(self._side)
        if early:
            page_list = sel.select_(1, rep, lc.top_k, sm_budget=budget)
        lc.update_tables_(page_list, advance_split=False, inline_fetch=True, after_selection=True)
        # phase 2 needs the update, not phase 1: whichever of the two launches finishes last merges
        self.attend_(xq, xk, xv, start_pos, out, phase=2)
        main.wait_event(self._join)

    def attend_(self, xq, xk, xv, start_pos, out, lse=None, fetch=False, phase=0) -> None:
        """Enqueue the decode attention over the current slot table and the local
        window (appends xk/xv at start_pos - dram_kv_cache_size first).  With `fetch` the
        kernel also reads the pages the last LRU update marked from DRAM and writes them
        through to their slots (no fetch_ call needed)."""
        rep = xq.shape[2] // self.n_kv_heads
        seqlen = xq.shape[1]
        prefix = self.lru_cache.hbm_kv_cache
        n_prefix_tokens = (self.lru_cache.num_tokens if isinstance(self.lru_cache, DummyCache)
                           else self.lru_cache.num_hbm_pages * self.page_size)
        if n_prefix_tokens == 0:
            raise RuntimeError("empty DRAM prefix is not supported")
        buf, nbytes, status = self._workspace(rep, xq.device, seqlen)
        if isinstance(start_pos, torch.Tensor):
            assert start_pos.dtype == torch.int32 and start_pos.is_cuda and start_pos.numel() == 1
            pos_dev, pos_host = start_pos.data_ptr(), 0
        else:
            pos_dev, pos_host = 0, int(start_pos)
        lib = _native.lib()
        lse_ptr = 0 if lse is None else lse.data_ptr()
        if self.peer_push is not None and seqlen == 1:
            _native.check(lib.da_decode_attention_push_next(*self.peer_push), "da_decode_attention_push_next")
        if phase:
            lc = self.lru_cache
            _native.check(lib.da_decode_attention_phased(
                phase, lc.evict_order.data_ptr(), lc.n_evictable.data_ptr(), lc.evict_flip.data_ptr(),
                lc.evict_redo.data_ptr(), int(self.phase1_ctas), int(self.phase2_ctas),
                xq.data_ptr(), prefix.data_ptr(), prefix.stride(0), lc.num_hbm_pages, self.page_size,
                lc.dram_kv_cache.data_ptr(), lc.num_dram_pages, lc.slot_source.data_ptr(),
                self.cache_k.data_ptr(), self.cache_v.data_ptr(), self.cache_k.stride(1),
                self.cache_k.stride(2), self.cache_k.shape[1], xk.data_ptr(), xv.data_ptr(),
                pos_dev, pos_host, self.dram_kv_cache_size, out.data_ptr(), lse_ptr, buf.data_ptr(), nbytes,
                status.data_ptr(), self.n_kv_heads, rep, self.head_dim, _native.dtype_code(xq.dtype),
                _native.stream_ptr()), "da_decode_attention_phased")
            return
        if fetch:
            lc = self.lru_cache
            _native.check(lib.da_decode_attention_fetch(
                xq.data_ptr(), prefix.data_ptr(), prefix.stride(0), lc.num_hbm_pages, self.page_size,
                lc.dram_kv_cache.data_ptr(), lc.num_dram_pages, lc.slot_source.data_ptr(),
                self.cache_k.data_ptr(), self.cache_v.data_ptr(), self.cache_k.stride(1),
                self.cache_k.stride(2), self.cache_k.shape[1], xk.data_ptr(), xv.data_ptr(),
                pos_dev, pos_host, self.dram_kv_cache_size, out.data_ptr(), lse_ptr, buf.data_ptr(), nbytes,
                status.data_ptr(), self.n_kv_heads, rep, self.head_dim, _native.dtype_code(xq.dtype),
                _native.stream_ptr()), "da_decode_attention_fetch")
            return
        _native.check(lib.da_decode_attention_tokens(
            xq.data_ptr(), seqlen, prefix.data_ptr(), prefix.stride(0), n_prefix_tokens,
            self.cache_k.data_ptr(), self.cache_v.data_ptr(), self.cache_k.stride(1),
            self.cache_k.stride(2), self.cache_k.shape[1], xk.data_ptr(), xv.data_ptr(),
            pos_dev, pos_host, self.dram_kv_cache_size, out.data_ptr(), lse_ptr, buf.data_ptr(), nbytes,
            status.data_ptr(), self.n_kv_heads, rep, self.head_dim, _native.dtype_code(xq.dtype),
            _native.stream_ptr()), "da_decode_attention_tokens")

    def check_status(self) -> None:
        """Synchronises; raises if any kernel of this operator flagged a problem."""
        statuses = [status for _, _, status in self._ws.values()]
        if self._prefill_status is not None:
            statuses.append(self._prefill_status)
        for status in statuses:
            bits = int(status.item())
            if bits:
                status.zero_()
                raise RuntimeError("dram_attention_b200 device status: " + _native.status_message(bits))
        if isinstance(self.lru_cache, LRUCache):
            self.lru_cache.check_status()

"""KV-head sharding of the operator across the GPUs of one node.

The reference has no multi-GPU path.  Every piece of state of the generate stage
is indexed by KV head (DRAM pages, summaries, slot table, LRU tables, local
window), and a GQA group is a contiguous run of query heads, so rank g of G simply
owns KV heads [g*Hk/G, (g+1)*Hk/G) and the query heads of those groups.  The only
exchange is the all-gather of the per-head outputs: rank-major concatenation of
(Hq/G, D) blocks is exactly the (1, 1, Hq, D) output.

For one token per call (decode) the gather is a kernel of this package over NVLink peer
memory (csrc/gather.cu: every rank stores its rows into every rank's buffer and waits,
bounded, on its own flags); the buffers come from torch's symmetric-memory allocator.
`peer_gather=False`, several tokens per call, CPU tensors, or a platform where the
symmetric allocation fails fall back to `all_gather_into_tensor` of the process group.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def head_range(n_kv_heads: int, rank: int, world_size: int):
    """KV heads [lo, hi) owned by `rank`; requires world_size to divide n_kv_heads."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if n_kv_heads % world_size != 0:
        raise ValueError(f"world size {world_size} must divide n_kv_heads {n_kv_heads}")
    per = n_kv_heads // world_size
    return rank * per, (rank + 1) * per


class KVHeadShardedDRAMAttention(torch.nn.Module):
    """Same call signature as DRAMAttention, computing only this rank's KV heads and
    all-gathering the outputs.  Inputs are the full (1, s, Hq, D) / (1, s, Hk, D)
    tensors (replicated on every rank, as a tensor-parallel caller has them after
    its own projections) or, with `presliced=True`, only this rank's heads.

    `operator_factory(n_kv_heads=..., **ctor_kwargs)` builds the per-rank operator
    (DRAMAttention by default; tests inject a stand-in).

    The first decode call sets the peer-memory gather up (an allocation, a rendezvous and a
    barrier): make it eagerly, before any CUDA-graph capture.  The gather kernel never hangs: a
    rank that waits longer than `gather_timeout_us` for a peer gives up, marks the peer's rows
    of its output with NaN and sets a status bit.  `check_status()` reads that bit (it
    synchronises): call it between steps, or at the latest before the outputs are trusted."""

    gather_timeout_us = 0   # 0: the library's default (0.2 s)
    push_from_attention = True   # one-token steps: the CTA that merges a head sends its rows to the peers itself

    def __init__(self, *, n_kv_heads: int, rank: Optional[int] = None, world_size: Optional[int] = None,
                 process_group=None, operator_factory: Optional[Callable] = None, presliced: bool = False,
                 peer_gather: bool = True, **ctor_kwargs):
        super().__init__()
        self.group = process_group
        self.world_size = dist.get_world_size(process_group) if world_size is None else world_size
        self.rank = dist.get_rank(process_group) if rank is None else rank
        self.n_kv_heads = n_kv_heads
        self.lo, self.hi = head_range(n_kv_heads, self.rank, self.world_size)
        self.presliced = presliced
        if operator_factory is None:
            from .dram_attention import DRAMAttention as operator_factory
        self.inner = operator_factory(n_kv_heads=self.hi - self.lo, **ctor_kwargs)
        self.peer_gather = peer_gather
        self._peer = None          # (handle, buffer, seq, status, bytes_per_rank) once set up
        self._peer_failed = None   # why the peer path is not in use, if it is not

    # ---- gather over peer memory --------------------------------------------------
    def _peer_setup(self, local: torch.Tensor):
        """Collective (every rank calls it at its first decode step): allocates the symmetric
        gather buffer and exchanges the peer mappings."""
        import os
        from . import _native
        # plain peer stores only: the allocator need not bind the buffer to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        nbytes = local.numel() * local.element_size()
        total = _native.lib().da_gather_heads_buffer_bytes(nbytes, self.world_size)
        if total == 0 or nbytes % 16 != 0:
            raise RuntimeError(f"{nbytes} bytes per rank on {self.world_size} ranks: outside the gather kernel's range")
        buf = symm_mem.empty(total, dtype=torch.uint8, device=local.device)
        buf.zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        handle = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(local.device)
        dist.barrier(group=self.group)     # every buffer is zero before anybody's first push
        seq = torch.zeros(1, dtype=torch.int32, device=local.device)
        status = torch.zeros(1, dtype=torch.int32, device=local.device)
        return handle, buf, seq, status, nbytes

    def _peer_gather(self, local: torch.Tensor, pushed: bool = False) -> torch.Tensor:
        """`pushed`: the attention launches of this step have sent the rows already (the operator was given
        the gather's buffers, see DRAMAttention.peer_push); the kernel then only waits and copies."""
        from . import _native
        handle, buf, seq, status, nbytes = self._peer
        b, s, h, d = local.shape
        assert local.numel() * local.element_size() == nbytes, "the shard's output size changed between calls"
        out = torch.empty(b, 1, h * self.world_size, d, dtype=local.dtype, device=local.device)
        src = local if local.is_contiguous() else local.contiguous()
        with torch.cuda.device(local.device):
            _native.check(_native.lib().da_gather_heads(
                0 if pushed else src.data_ptr(), nbytes, handle.buffer_ptrs_dev, seq.data_ptr(), self.rank, self.world_size,
                out.data_ptr(), int(self.gather_timeout_us), status.data_ptr(), _native.stream_ptr()),
                "da_gather_heads")
        return out

    def check_status(self) -> None:
        """Synchronising check of the device-side status words (tests, debugging)."""
        if hasattr(self.inner, "check_status"):
            self.inner.check_status()
        if self._peer is not None:
            code = int(self._peer[3].item())
            if code:
                raise RuntimeError(f"peer gather reported status {code} (8 = a wait on another rank ran out)")

    def _kv(self, t: torch.Tensor) -> torch.Tensor:
        return t if self.presliced else t[:, :, self.lo:self.hi]

    def _q(self, t: torch.Tensor) -> torch.Tensor:
        if self.presliced:
            return t
        rep = t.shape[2] // self.n_kv_heads
        return t[:, :, self.lo * rep:self.hi * rep]

    def init_cache(self, k_cache: torch.Tensor, v_cache: torch.Tensor):
        self.inner.init_cache(self._kv(k_cache), self._kv(v_cache))

    def forward(self, xq, xk, xv, *, start_pos, stage: str, freqs_cis=None):
        extra = {} if freqs_cis is None else {"freqs_cis": freqs_cis}   # rotary embedding inside the call
        # once the peer gather is set up, a one-token generate step sends its rows from the attention launches
        pushed = (stage == "generate" and xq.shape[1] == 1 and self._peer is not None
                  and getattr(self.inner, "peer_push", None) is not None)
        local = self.inner(self._q(xq).contiguous(), self._kv(xk).contiguous(), self._kv(xv).contiguous(),
                           start_pos=start_pos, stage=stage, **extra)
        return self.all_gather_heads(local, pushed=pushed)

    def all_gather_heads(self, local: torch.Tensor, pushed: bool = False) -> torch.Tensor:
        """(1, s, Hq/G, D) on every rank -> (1, s, Hq, D) on every rank."""
        if self.world_size == 1:
            return local
        b, s, h, d = local.shape
        if s == 1 and self.peer_gather and local.is_cuda and self._peer_failed is None:
            if self._peer is None:
                try:
                    self._peer = self._peer_setup(local)
                except Exception as e:   # no symmetric memory on this platform: library gather
                    self._peer_failed = repr(e)
                # all ranks take the same path
                ok = torch.tensor([0 if self._peer is None else 1], dtype=torch.int32, device=local.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
                if int(ok.item()) == 0:
                    self._peer = None
                    self._peer_failed = self._peer_failed or "another rank could not set up its gather buffer"
            if self._peer is not None:
                if self.push_from_attention and hasattr(self.inner, "peer_push") and self.inner.peer_push is None:
                    import ctypes
                    handle, _buf, seq, _status, nbytes = self._peer
                    self._peer_host_ptrs = (ctypes.c_void_p * self.world_size)(*[int(x) for x in handle.buffer_ptrs])
                    self.inner.peer_push = (ctypes.cast(self._peer_host_ptrs, ctypes.c_void_p), seq.data_ptr(),
                                            self.rank, self.world_size, nbytes)
                return self._peer_gather(local, pushed)
        if s == 1:
            # rank-major concatenation is the head order; a tensor of its own per call, like the
            # single-GPU operator's result
            out = torch.empty(b, 1, h * self.world_size, d, dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(out.view(-1), local.contiguous().view(-1), group=self.group)
            return out
        # several tokens: gather (G, s, h, d) then put the rank axis next to the heads
        tmp = torch.empty(self.world_size, s, h, d, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(tmp.view(-1), local.contiguous().view(-1), group=self.group)
        return tmp.permute(1, 0, 2, 3).reshape(1, s, h * self.world_size, d)

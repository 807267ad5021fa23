"""Seeded synthetic decode workloads.

The reference project evaluates on long prompts and real model KV caches that
are not redistributable; these generators produce tensors with the same
shapes, dtypes and the value structure that matters to the path (a few
large-magnitude "outlier" channels, a handful of "needle" pages whose keys
align with the query, slowly drifting queries).  Nothing here is an item of a
public benchmark.

Every workload is generated on the CPU from `torch.Generator().manual_seed(seed)`
in a fixed order (keys, values, outlier channels, needles, first query,
per-step noise) so that a CPU checker and the GPU path see identical bits.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict

import torch


@dataclass
class DecodeWorkload:
    """One attention layer, batch 1: a prefill KV cache and `steps` decode inputs."""
    name: str
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    dtype: torch.dtype
    page_size: int
    lru_hbm_cache_size: int      # tokens
    local_cache_size: int        # tokens
    top_k: int                   # tokens
    max_output_length: int
    prefill_len: int             # S; DRAM prefix = floor((S - local + P) / P) * P tokens
    steps: int
    k: torch.Tensor = field(repr=False)    # (1, S, Hk, D)
    v: torch.Tensor = field(repr=False)
    xq: torch.Tensor = field(repr=False)   # (steps, 1, 1, Hq, D)
    xk: torch.Tensor = field(repr=False)   # (steps, 1, 1, Hk, D)
    xv: torch.Tensor = field(repr=False)

    @property
    def dram_tokens(self) -> int:
        p = self.page_size
        return (self.prefill_len - self.local_cache_size + p) // p * p

    def ctor_kwargs(self) -> Dict:
        """Keyword arguments of the `DRAMAttention` constructor for this workload."""
        return dict(max_output_length=self.max_output_length,
                    lru_hbm_cache_size=self.lru_hbm_cache_size,
                    local_cache_size=self.local_cache_size,
                    page_size=self.page_size, top_k=self.top_k,
                    n_kv_heads=self.n_kv_heads, head_dim=self.head_dim)


def _kv_with_outliers(g, s, hk, d, n_outliers, scale, chunk=16384):
    k = torch.empty(1, s, hk, d, dtype=torch.float32)
    v = torch.empty(1, s, hk, d, dtype=torch.float32)
    for t in (k, v):
        for a in range(0, s, chunk):
            b = min(s, a + chunk)
            t[0, a:b] = torch.randn(b - a, hk, d, generator=g)
    ch = torch.randperm(d, generator=g)[:n_outliers]
    k[..., ch] *= scale
    v[..., ch] *= scale
    return k, v, ch


def plumbing_workload(seed: int = 0, steps: int = 16) -> DecodeWorkload:
    """Small float32 case: 8 query / 2 KV heads, head_dim 64, 4096-token DRAM
    prefix in 256 pages of 16, 128 slots, local window 256, top_k 512 tokens.
    Keys/values N(0,1) with 4 outlier channels x8; the first query is the key
    of a random prefix token plus N(0, 0.5^2) noise and drifts by N(0, 0.1^2)."""
    hq, hk, d, p = 8, 2, 64, 16
    local, lru, top_k, max_out = 256, 2048, 512, 16
    s = 4096 + local - p          # DRAM prefix of exactly 4096 tokens
    g = torch.Generator().manual_seed(seed)
    k, v, ch = _kv_with_outliers(g, s, hk, d, 4, 8.0)
    rep = hq // hk
    tau = int(torch.randint(0, 4096, (1,), generator=g))
    q0 = k[0, tau].repeat_interleave(rep, dim=0) + 0.5 * torch.randn(hq, d, generator=g)
    xq = torch.empty(steps, 1, 1, hq, d)
    q = q0
    for i in range(steps):
        if i:
            q = q + 0.1 * torch.randn(hq, d, generator=g)
        xq[i, 0, 0] = q
    xk = torch.randn(steps, 1, 1, hk, d, generator=g)
    xv = torch.randn(steps, 1, 1, hk, d, generator=g)
    xk[..., ch] *= 8.0
    xv[..., ch] *= 8.0
    return DecodeWorkload("plumbing-fp32-4k", hq, hk, d, torch.float32, p, lru, local,
                          top_k, max_out, s, steps, k, v, xq, xk, xv)


def llama_layer_workload(seed: int = 0, steps: int = 64, dram_tokens: int = 131072,
                         n_kv_heads: int = 8, rep: int = 4, lru: int = 32768,
                         local: int = 4096, top_k: int = 4096, needles: int = 16,
                         redraw_every: int = 0, max_out: int | None = None,
                         dtype: torch.dtype = torch.bfloat16) -> DecodeWorkload:
    """Llama-3-8B-shaped decode layer: head_dim 128, page 16, bf16.  Keys and
    values N(0,1) with 8 outlier channels x10; `needles` pages at random
    positions have keys u + N(0, 0.3^2) for one shared direction u (|u| =
    sqrt(D)); queries are u + N(0,1) and drift by N(0, 0.05^2) per step.  With
    `redraw_every` > 0 the query is re-drawn from N(0,1) every that many steps
    (forces slot churn)."""
    hk, d, p = n_kv_heads, 128, 16
    hq = hk * rep
    max_out = steps if max_out is None else max_out
    s = dram_tokens + local - p
    g = torch.Generator().manual_seed(seed)
    k, v, ch = _kv_with_outliers(g, s, hk, d, 8, 10.0)
    u = torch.randn(d, generator=g)
    u = u / u.norm() * (d ** 0.5)
    if needles:
        pages = torch.randperm(dram_tokens // p, generator=g)[:needles]
        for pg in pages.tolist():
            k[0, pg * p:(pg + 1) * p] = u + 0.3 * torch.randn(p, hk, d, generator=g)
    xq = torch.empty(steps, 1, 1, hq, d)
    q = u[None] + torch.randn(hq, d, generator=g)
    for i in range(steps):
        if i:
            if redraw_every and i % redraw_every == 0:
                q = torch.randn(hq, d, generator=g)
            else:
                q = q + 0.05 * torch.randn(hq, d, generator=g)
        xq[i, 0, 0] = q
    xk = torch.randn(steps, 1, 1, hk, d, generator=g)
    xv = torch.randn(steps, 1, 1, hk, d, generator=g)
    xk[..., ch] *= 10.0
    xv[..., ch] *= 10.0
    name = f"llama3-8b-layer-{dram_tokens // 1024}k-{str(dtype).split('.')[-1]}"
    return DecodeWorkload(name, hq, hk, d, dtype, p, lru, local, top_k, max_out, s, steps,
                          k.to(dtype), v.to(dtype), xq.to(dtype), xk.to(dtype), xv.to(dtype))


def scorer_workload(seed: int = 0, pages: int = 65536, n_kv_heads: int = 8, rep: int = 4,
                    head_dim: int = 128, page_size: int = 16,
                    dtype: torch.dtype = torch.bfloat16):
    """Page-scorer micro-benchmark inputs: per-page min/max summaries of N(0,1)
    keys (Hk, pages, 2, D) in `dtype` and N(0,1) queries (1, 1, Hq, D)."""
    g = torch.Generator().manual_seed(seed)
    mm = torch.empty(n_kv_heads, pages, 2, head_dim, dtype=dtype)
    chunk = max(1, 4096)
    for h in range(n_kv_heads):
        for a in range(0, pages, chunk):
            b = min(pages, a + chunk)
            keys = torch.randn(b - a, page_size, head_dim, generator=g).to(dtype)
            mn, mx = torch.aminmax(keys, dim=1)
            mm[h, a:b, 0] = mn
            mm[h, a:b, 1] = mx
    q = torch.randn(1, 1, n_kv_heads * rep, head_dim, generator=g).to(dtype)
    return q, mm

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


def device_layer_inputs(device, seed: int, steps: int, dram_tokens: int, n_kv_heads: int = 8, rep: int = 4,
                        local: int = 4096, page_size: int = 16, needles: int = 16, redraw_every: int = 0,
                        dtype: torch.dtype = torch.bfloat16):
    """The same kind of layer as `llama_layer_workload` (head_dim 128; N(0,1) keys/values with 8
    outlier channels x10; `needles` pages along a shared direction u; queries u + N(0,1) drifting by
    N(0, 0.05^2), re-drawn from N(0,1) every `redraw_every` steps), generated ON THE DEVICE from a
    device generator seeded with `seed`: for the large benchmark workloads (a million-token prefix,
    many sequences) that take minutes to draw on the host.  Not bit-identical to the host version.

    Returns (k, v, xq, xk, xv, u, outlier_channels): k, v (1, S, Hk, D) with S = dram_tokens +
    local - page_size; xq (steps, 1, 1, Hq, D); xk, xv (steps, 1, 1, Hk, D); the needle direction
    and the outlier channels (for `device_decode_inputs` of further layers over the same prefix)."""
    d, hk, hq = 128, n_kv_heads, n_kv_heads * rep
    s = dram_tokens + local - page_size
    g = torch.Generator(device=device).manual_seed(seed)
    ch = torch.randperm(d, generator=g, device=device)[:8]
    k = torch.empty(1, s, hk, d, dtype=dtype, device=device)
    v = torch.empty(1, s, hk, d, dtype=dtype, device=device)
    chunk = 65536
    for t in (k, v):
        for a in range(0, s, chunk):
            b = min(s, a + chunk)
            x = torch.randn(b - a, hk, d, generator=g, device=device)
            x[..., ch] *= 10.0
            t[0, a:b] = x.to(dtype)
    u = torch.randn(d, generator=g, device=device)
    u = u / u.norm() * (d ** 0.5)
    if needles:
        pages = torch.randperm(dram_tokens // page_size, generator=g, device=device)[:needles]
        for pg in pages.tolist():
            k[0, pg * page_size:(pg + 1) * page_size] = \
                (u + 0.3 * torch.randn(page_size, hk, d, generator=g, device=device)).to(dtype)
    xq, xk, xv = device_decode_inputs(device, seed + 1, steps, u, ch, hk, rep, redraw_every, dtype)
    return k, v, xq, xk, xv, u, ch


def device_decode_inputs(device, seed: int, steps: int, u: torch.Tensor, outlier_channels: torch.Tensor,
                         n_kv_heads: int, rep: int, redraw_every: int = 0,
                         dtype: torch.dtype = torch.bfloat16):
    """Per-step decode inputs of one layer on the device: queries u + N(0,1) that drift by
    N(0, 0.05^2) per step (re-drawn from N(0,1) every `redraw_every` steps), new keys/values
    N(0,1) with the outlier channels x10."""
    d, hk, hq = u.shape[0], n_kv_heads, n_kv_heads * rep
    g = torch.Generator(device=device).manual_seed(seed)
    q = u[None] + torch.randn(hq, d, generator=g, device=device)
    noise = 0.05 * torch.randn(steps, hq, d, generator=g, device=device)
    xq = torch.empty(steps, 1, 1, hq, d, dtype=dtype, device=device)
    for i in range(steps):
        if i:
            if redraw_every and i % redraw_every == 0:
                q = torch.randn(hq, d, generator=g, device=device)
            else:
                q = q + noise[i]
        xq[i, 0, 0] = q.to(dtype)
    xk = torch.randn(steps, 1, 1, hk, d, generator=g, device=device)
    xv = torch.randn(steps, 1, 1, hk, d, generator=g, device=device)
    xk[..., outlier_channels] *= 10.0
    xv[..., outlier_channels] *= 10.0
    return xq, xk.to(dtype), xv.to(dtype)

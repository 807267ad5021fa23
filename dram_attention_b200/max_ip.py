"""Quest upper-bound page score: `max_inner_product` runs the CUDA page scorer,
`max_ip_ref` is the plain torch statement of the same formula (kept because the
reference package exports it; nothing in the operator calls it)."""

from __future__ import annotations

import torch

from . import _native


def score_pages_(q: torch.Tensor, min_max: torch.Tensor, scores: torch.Tensor,
                 n_tokens: int, n_kv_heads: int, rep: int, ordered: bool = False) -> None:
    """Enqueue the page scorer.  q (n_tokens, n_kv_heads*rep, D) contiguous;
    min_max (n_kv_heads, L, 2, D) contiguous; scores float32 (n_tokens, n_kv_heads*rep, L).
    `ordered` promises min_max[..., 0, :] <= min_max[..., 1, :] everywhere."""
    n_pages, d = min_max.shape[1], min_max.shape[3]
    _native.check(_native.lib().da_score_pages(
        q.data_ptr(), min_max.data_ptr(), scores.data_ptr(), n_tokens, n_kv_heads, rep, n_pages, d,
        _native.dtype_code(q.dtype), int(ordered), _native.stream_ptr()), "da_score_pages")


def max_inner_product(q: torch.Tensor, min_max: torch.Tensor) -> torch.Tensor:
    """out[n, h, l] = sum_d max(q[n,h,d] * min_max[h,l,0,d], q[n,h,d] * min_max[h,l,1,d]).

    Same signature and result dtype (q.dtype) as the reference's
    max_inner_product (dram_attention/max_ip_triton_kernel.py:95-124); products and
    the channel sum are float32 on the device before the final cast."""
    n, h, d = q.shape
    h1, l, r, d1 = min_max.shape
    assert h1 == h and d1 == d and r == 2
    _native.require_cuda(q, "q")
    _native.require_cuda(min_max, "min_max")
    assert q.dtype == min_max.dtype, "q and min_max must have the same dtype"
    scores = torch.empty(n, h, l, dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        score_pages_(q.contiguous(), min_max.contiguous(), scores, n, h, 1)
    return scores if q.dtype == torch.float32 else scores.to(q.dtype)


def max_ip_ref(q: torch.Tensor, min_max: torch.Tensor) -> torch.Tensor:
    """Plain torch statement of the score (dram_attention/max_ip_triton_kernel.py:127-133)."""
    n, h, d = q.shape
    h1, l, r, d1 = min_max.shape
    assert h1 == h and d1 == d
    return torch.amax(q[:, :, None, None, :] * min_max[None], dim=-2).sum(-1)

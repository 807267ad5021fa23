"""Run the reference's own Python classes on the CPU (test infrastructure only).

The reference package (`dram_attention/` of long-context/dram-attention) is
written for a CUDA device.  It can still be imported and stepped on CPU tensors
when four things are substituted at run time, none of which touches the
algorithm under test except where stated:

  1. `torch.empty(..., pin_memory=True)` -> pageable memory (no CUDA driver).
  2. the Triton page scorer -> the reference's own torch statement of it,
     `max_ip_ref` (dram_attention/max_ip_triton_kernel.py:127-133).
  3. `flash_attn_with_kvcache` / `flash_attn_func` (third-party, GPU only) ->
     explicit-softmax restatements written from the documented behaviour of
     those calls (in-place append at cache_seqlens, attention over
     [:cache_seqlens + s], scale D**-0.5, GQA by contiguous groups, float32
     lse of shape (b, Hq, s)); internally float64.
  4. `torch.argsort(..., descending=True)` -> the same call with stable=True,
     so ties resolve to the lowest page id.
The reference's own LRU Triton kernels run unchanged through Triton's
interpreter (TRITON_INTERPRET=1, set before triton is imported).

Only the golden-vector generator and tests that are skipped when the
reference tree is absent may import this module.
"""

from __future__ import annotations

import contextlib
import os
import sys

# where the reference project is checked out: the environment decides (nothing is assumed)
REFERENCE_ROOT = os.environ.get("DRAM_ATTENTION_REFERENCE", "")


def reference_available() -> bool:
    return bool(REFERENCE_ROOT) and os.path.isdir(os.path.join(REFERENCE_ROOT, "dram_attention"))


def _flash_attn_with_kvcache_cpu(q, k_cache, v_cache, k=None, v=None, rotary_cos=None,
                                 rotary_sin=None, causal=False, cache_seqlens=None,
                                 rotary_interleaved=True, return_softmax_lse=False, **_):
    """Documented behaviour of flash_attn_with_kvcache (flash_attn_interface.py docstring of
    flash-attn 2.8.3): k/v are written into the cache at cache_seqlens; attention runs over the
    first cache_seqlens + s tokens; with causal=True the mask is aligned to the bottom-right
    corner, i.e. query i of s sees keys j <= seqlen_k - s + i."""
    import torch
    b, s, hq, d = q.shape
    assert b == 1
    seqlen = int(cache_seqlens)
    if k is not None:
        k_cache[:, seqlen:seqlen + s] = k
        v_cache[:, seqlen:seqlen + s] = v
        seqlen = seqlen + s
    hk = k_cache.shape[2]
    rep = hq // hk
    qf = q[0].double().reshape(s, hk, rep, d).permute(1, 2, 0, 3)        # (Hk, rep, s, D)
    kf = k_cache[0, :seqlen].double().permute(1, 0, 2)[:, None]          # (Hk, 1, T, D)
    vf = v_cache[0, :seqlen].double().permute(1, 0, 2)[:, None]
    logits = torch.matmul(qf, kf.transpose(-1, -2)) * (d ** -0.5)        # (Hk, rep, s, T)
    if causal and s > 1:
        j = torch.arange(seqlen)[None, :]
        i = torch.arange(s)[:, None]
        logits = logits.masked_fill(j > seqlen - s + i, float("-inf"))
    lse = torch.logsumexp(logits, dim=-1)                                # (Hk, rep, s)
    out = torch.matmul(torch.exp(logits - lse[..., None]), vf)           # (Hk, rep, s, D)
    # flash-attn returns the output in q's dtype and the lse in float32; the
    # arithmetic in between is float64 here so the fixture is accurate to float32
    out = out.permute(2, 0, 1, 3).reshape(1, s, hq, d).to(q.dtype)
    lse = lse.permute(0, 1, 2).reshape(1, hq, s).float()
    return (out, lse) if return_softmax_lse else out


def _flash_attn_func_cpu(q, k, v, causal=False, **_):
    import torch
    b, s, hq, d = q.shape
    hk = k.shape[2]
    rep = hq // hk
    qf = q[0].float().reshape(s, hk, rep, d).permute(1, 2, 0, 3)        # (Hk, rep, S, D)
    kf = k[0].float().permute(1, 0, 2)[:, None]                        # (Hk, 1, S, D)
    vf = v[0].float().permute(1, 0, 2)[:, None]
    logits = torch.matmul(qf, kf.transpose(-1, -2)) * (d ** -0.5)       # (Hk, rep, S, S)
    if causal:
        mask = torch.ones(s, s, dtype=torch.bool).tril()
        logits = logits.masked_fill(~mask, float("-inf"))
    out = torch.matmul(torch.softmax(logits, dim=-1), vf)               # (Hk, rep, S, D)
    return out.permute(2, 0, 1, 3).reshape(1, s, hq, d).to(q.dtype)


@contextlib.contextmanager
def reference_on_cpu():
    """Context manager yielding the reference `dram_attention` package, patched
    as described in the module docstring.  Patches are undone on exit."""
    os.environ.setdefault("TRITON_INTERPRET", "1")
    import torch
    if not reference_available():
        raise RuntimeError("set DRAM_ATTENTION_REFERENCE to the checkout of long-context/dram-attention")
    if REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, REFERENCE_ROOT)
    orig_empty = torch.empty
    orig_argsort = torch.argsort

    def empty_no_pin(*a, **kw):
        kw.pop("pin_memory", None)
        return orig_empty(*a, **kw)

    def argsort_stable(x, *a, **kw):
        kw["stable"] = True
        return orig_argsort(x, *a, **kw)

    torch.empty = empty_no_pin
    torch.argsort = argsort_stable
    try:
        import dram_attention as ref
        import dram_attention.dram_attention as ref_da
        import dram_attention.topk_selector as ref_sel
        from dram_attention.max_ip_triton_kernel import max_ip_ref
        saved = (ref_sel.max_inner_product, ref_da.flash_attn_with_kvcache,
                 ref_da.flash_attn_func)
        ref_sel.max_inner_product = max_ip_ref
        ref_da.flash_attn_with_kvcache = _flash_attn_with_kvcache_cpu
        ref_da.flash_attn_func = _flash_attn_func_cpu
        try:
            yield ref
        finally:
            (ref_sel.max_inner_product, ref_da.flash_attn_with_kvcache,
             ref_da.flash_attn_func) = saved
    finally:
        torch.empty = orig_empty
        torch.argsort = orig_argsort

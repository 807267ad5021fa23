"""The attention arithmetic of the reference lives in the third-party package flash-attn
(`flash_attn_with_kvcache`, called at dram_attention/dram_attention.py:195-205 and :211-223).
Where that package imports and its kernels run on this GPU, compare its result -- prefix part,
suffix part with the in-place append, and the reference's own LSE merge (:225-238) -- with
da_decode_attention on the same tensors.  Skipped, with the library's own message, where the
installed wheel has no kernel for this GPU."""

import pytest
import torch

from tests.conftest import assert_out_close

pytestmark = pytest.mark.gpu

DEV = "cuda"


def test_decode_attention_matches_flash_attn_where_it_runs():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dram_attention_b200 import _native
    lib = _native.lib()
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as e:      # not installed, or built against another torch
        pytest.skip(f"flash-attn does not import here: {e!r}")
    hk, rep, d, n_slot_tokens, cap, t = 2, 4, 128, 4096, 256, 200
    g = torch.Generator().manual_seed(5)
    dtype = torch.bfloat16
    slots = torch.randn(hk, n_slot_tokens, 2, d, generator=g).to(dtype).to(DEV)     # slot payload layout
    local_k = torch.randn(1, cap, hk, d, generator=g).to(dtype).to(DEV)
    local_v = torch.randn(1, cap, hk, d, generator=g).to(dtype).to(DEV)
    q = (torch.randn(1, 1, hk * rep, d, generator=g) * 1.5).to(dtype).to(DEV)
    nk = torch.randn(1, 1, hk, d, generator=g).to(dtype).to(DEV)
    nv = torch.randn(1, 1, hk, d, generator=g).to(dtype).to(DEV)

    # ---- the reference's way: two library calls and the merge --------------------------------
    ref_lk, ref_lv = local_k.clone(), local_v.clone()
    kc = slots[:, :, 0].transpose(0, 1)[None]      # (1, T, Hk, D) strided views, as the reference builds them
    vc = slots[:, :, 1].transpose(0, 1)[None]
    try:
        po, plse = flash_attn_with_kvcache(q, kc, vc, None, None, causal=True, cache_seqlens=n_slot_tokens,
                                           rotary_interleaved=True, return_softmax_lse=True)
        so, slse = flash_attn_with_kvcache(q, ref_lk, ref_lv, nk, nv, rotary_cos=None, rotary_sin=None, causal=True,
                                           cache_seqlens=t, rotary_interleaved=True, return_softmax_lse=True)
        torch.cuda.synchronize()
    except Exception as e:      # e.g. no kernel image for this architecture in the installed wheel
        pytest.skip(f"flash-attn does not run on this GPU: {e!r}")
    lse = torch.logaddexp(plse, slse)
    want = po * (plse - lse).exp().transpose(1, 2)[..., None] + so * (slse - lse).exp().transpose(1, 2)[..., None]

    # ---- this package: one launch ----------------------------------------------------------------
    ws_bytes = lib.da_decode_attention_workspace_bytes(hk, rep, d)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(hk * rep, d, dtype=dtype, device=DEV)
    lse_out = torch.empty(hk * rep, dtype=torch.float32, device=DEV)
    dram_tokens = 1 << 20
    _native.check(lib.da_decode_attention(
        q.data_ptr(), slots.data_ptr(), slots.stride(0), n_slot_tokens, local_k.data_ptr(), local_v.data_ptr(),
        local_k.stride(1), local_k.stride(2), cap, nk.data_ptr(), nv.data_ptr(), 0, dram_tokens + t, dram_tokens,
        out.data_ptr(), lse_out.data_ptr(), ws.data_ptr(), ws_bytes, status.data_ptr(), hk, rep, d,
        _native.dtype_code(dtype), _native.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status) == 0
    # 2e-2 absolute (plus half a bfloat16 ulp of the value): both sides round to bfloat16, the library twice
    assert_out_close(out.float().cpu(), want[0, 0].float().cpu(), dtype)
    assert torch.allclose(lse_out.cpu(), lse[0, :, 0].float().cpu(), rtol=1e-3, atol=1e-3)
    assert torch.equal(local_k, ref_lk) and torch.equal(local_v, ref_lv)      # the same append

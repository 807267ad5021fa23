"""Prefill stage: the tcgen05 causal attention kernel (da_prefill_attention, through the C ABI)
against an explicit float64 softmax on the same inputs, and through DRAMAttention's
stage="prefill" (dram_attention/dram_attention.py:136 is a library call in the reference, so
its own tests pin shapes only: dram_attention_test.py:60)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def da():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dram_attention_b200 as pkg
    pkg._native.lib()
    return pkg


def _reference(q, k, v):
    """(S, Hq, D), (S, Hk, D) x2 -> causal softmax(q k^T / sqrt(D)) v in float64, GQA by contiguous groups."""
    s, hq, d = q.shape
    rep = hq // k.shape[1]
    qf = q.double().transpose(0, 1)
    kf = k.double().repeat_interleave(rep, 1).transpose(0, 1)
    vf = v.double().repeat_interleave(rep, 1).transpose(0, 1)
    sc = qf @ kf.transpose(1, 2) / d ** 0.5
    sc = sc.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return (torch.softmax(sc, -1) @ vf).transpose(0, 1)


def _close(out, ref, dtype):
    # 2e-2 absolute for 16-bit outputs, plus half a unit in the last place of the stored value
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    bad = (out.double() - ref).abs() > 2e-2 + ref.abs() * ulp
    assert not bool(bad.any()), float((out.double() - ref).abs().max())


@pytest.mark.parametrize("s,hq,hk,dtype,scale", [
    (1, 1, 1, torch.bfloat16, 1.0), (127, 2, 1, torch.bfloat16, 1.0), (128, 1, 1, torch.float16, 1.0),
    (129, 4, 4, torch.bfloat16, 1.0), (300, 8, 2, torch.bfloat16, 1.0), (1000, 8, 2, torch.float16, 1.0),
    (2048, 32, 8, torch.bfloat16, 1.0), (777, 4, 1, torch.bfloat16, 4.0),
])
def test_prefill_kernel_matches_float64_softmax(da, s, hq, hk, dtype, scale):
    from dram_attention_b200 import _native
    g = torch.Generator().manual_seed(s)
    q = (scale * torch.randn(s, hq, 128, generator=g)).to(dtype).to(DEV)
    k = (scale * torch.randn(s, hk, 128, generator=g)).to(dtype).to(DEV)
    v = torch.randn(s, hk, 128, generator=g).to(dtype).to(DEV)
    out = torch.full_like(q, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _native.check(_native.lib().da_prefill_attention(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), s, hq, hk, 128, hq * 128, hk * 128,
        _native.dtype_code(dtype), status.data_ptr(), _native.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status) == 0
    assert bool(torch.isfinite(out.float()).all())
    _close(out, _reference(q, k, v), dtype)


def test_prefill_argument_checks(da):
    from dram_attention_b200 import _native
    lib = _native.lib()
    assert lib.da_prefill_attention_supported(128, _native.dtype_code(torch.bfloat16)) == 1
    assert lib.da_prefill_attention_supported(64, _native.dtype_code(torch.bfloat16)) == 0
    assert lib.da_prefill_attention_supported(128, _native.dtype_code(torch.float32)) == 0
    t = torch.zeros(16, 2, 128, dtype=torch.bfloat16, device=DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    args = lambda **kw: [kw.get("q", t.data_ptr()), t.data_ptr(), t.data_ptr(), t.data_ptr(), kw.get("s", 16),
                         kw.get("hq", 2), kw.get("hk", 2), kw.get("d", 128), 256, 256,
                         _native.dtype_code(torch.bfloat16), st.data_ptr(), _native.stream_ptr()]
    assert lib.da_prefill_attention(*args(q=0)) == -1          # DA_ERR_NULL
    assert lib.da_prefill_attention(*args(s=0)) == -2          # DA_ERR_SHAPE
    assert lib.da_prefill_attention(*args(hq=3)) == -2         # heads not a multiple of KV heads
    assert lib.da_prefill_attention(*args(d=64)) == -5         # DA_ERR_UNSUPPORTED
    assert lib.da_prefill_attention(*args(q=t.data_ptr() + 2)) == -4   # DA_ERR_ALIGN


def test_operator_prefill_then_generate(da):
    """stage="prefill" through the operator: output of the kernel, then the cache it leaves
    serves a generate step (same flow as dram_attention_test.py:21-60, with values checked)."""
    kw = dict(max_output_length=4, lru_hbm_cache_size=2048, local_cache_size=512, page_size=16, top_k=512,
              n_kv_heads=2, head_dim=128)
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(5)
    s = 8192 + 512 - 16
    xq = torch.randn(1, s, 8, 128, generator=g).to(dtype).to(DEV)
    k = torch.randn(1, s, 2, 128, generator=g).to(dtype).to(DEV)
    v = torch.randn(1, s, 2, 128, generator=g).to(dtype).to(DEV)
    m = da.DRAMAttention(device=DEV, dtype=dtype, **kw)
    out = m(xq, k, v, start_pos=0, stage="prefill")
    assert out.shape == xq.shape and out.dtype == xq.dtype
    ref = _reference(xq[0], k[0], v[0])
    _close(out[0], ref, dtype)
    lib_call = da.DRAMAttention(device=DEV, dtype=dtype, **kw)
    lib_call.prefill_kernel = False
    _close(lib_call(xq, k, v, start_pos=0, stage="prefill")[0], ref, dtype)
    q1 = torch.randn(1, 1, 8, 128, generator=g).to(dtype).to(DEV)
    k1 = torch.randn(1, 1, 2, 128, generator=g).to(dtype).to(DEV)
    v1 = torch.randn(1, 1, 2, 128, generator=g).to(dtype).to(DEV)
    step = m(q1, k1, v1, start_pos=s, stage="generate")
    step2 = lib_call(q1, k1, v1, start_pos=s, stage="generate")
    assert torch.equal(step, step2)      # both built the same cache from the same keys and values
    m.check_status()

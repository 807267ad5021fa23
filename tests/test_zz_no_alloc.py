"""da_decode_attention_static: the attention entry point for hosts that may not
allocate device memory while running (a frozen memory plan, a plugin without access
to the allocator).  It keeps the kernel's scratch in a buffer built into the library.
Checked here through the C ABI against da_decode_attention (caller-provided
workspace) and against the CPU oracle on two consecutive calls, which also exercises the
reuse of the shared buffer.  The file name makes pytest collect it last."""

import pytest
import torch

from oracle import dram_attention_oracle as orc
from tests.conftest import assert_out_close

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def native():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dram_attention_b200 import _native
    _native.lib()
    return _native


def _inputs(dtype, hk, rep, d, n_prefix, cap, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g).to(dtype).to(DEV)
    return dict(prefix=r(hk, n_prefix, 2, d), lk=r(cap, hk, d), lv=r(cap, hk, d),
                q=[r(hk * rep, d) for _ in range(2)], nk=[r(hk, d) for _ in range(2)],
                nv=[r(hk, d) for _ in range(2)])


@pytest.mark.parametrize("dtype,hk,rep,d,n_prefix,cap,t0", [
    (torch.bfloat16, 8, 4, 128, 4096, 300, 257),
    (torch.float32, 2, 4, 64, 1000, 64, 30),
])
def test_static_scratch_matches_workspace_entry_point(native, dtype, hk, rep, d, n_prefix, cap, t0):
    lib = native.lib()
    x = _inputs(dtype, hk, rep, d, n_prefix, cap, seed=n_prefix)
    ws_bytes = lib.da_decode_attention_workspace_bytes(hk, rep, d)
    assert ws_bytes <= lib.da_decode_attention_static_capacity()
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    code, dram_tokens, s = native.dtype_code(dtype), 512, native.stream_ptr()
    # each entry point appends to its own copy of the local window
    lk_a, lv_a, lk_b, lv_b = x["lk"].clone(), x["lv"].clone(), x["lk"].clone(), x["lv"].clone()
    for call in range(2):
        q, nk, nv, pos = x["q"][call], x["nk"][call], x["nv"][call], dram_tokens + t0 + call
        out_a, out_b = torch.empty_like(q), torch.empty_like(q)
        lse_a = torch.empty(hk * rep, dtype=torch.float32, device=DEV)
        lse_b = torch.empty_like(lse_a)
        native.check(lib.da_decode_attention(
            q.data_ptr(), x["prefix"].data_ptr(), x["prefix"].stride(0), n_prefix, lk_a.data_ptr(),
            lv_a.data_ptr(), lk_a.stride(0), lk_a.stride(1), cap, nk.data_ptr(), nv.data_ptr(), 0, pos,
            dram_tokens, out_a.data_ptr(), lse_a.data_ptr(), ws.data_ptr(), ws_bytes, status.data_ptr(),
            hk, rep, d, code, s))
        native.check(lib.da_decode_attention_static(
            q.data_ptr(), x["prefix"].data_ptr(), x["prefix"].stride(0), n_prefix, lk_b.data_ptr(),
            lv_b.data_ptr(), lk_b.stride(0), lk_b.stride(1), cap, nk.data_ptr(), nv.data_ptr(), 0, pos,
            dram_tokens, out_b.data_ptr(), lse_b.data_ptr(), status.data_ptr(), hk, rep, d, code, s))
        torch.cuda.synchronize()
        assert int(status) == 0
        # same kernel, same split geometry, same merge order: 1e-4 / 2e-2 are the suite's
        # tolerances, the results are in fact identical
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        assert (out_a.float() - out_b.float()).abs().max().item() <= tol
        assert torch.equal(out_a, out_b)
        assert torch.allclose(lse_a, lse_b, rtol=1e-4, atol=1e-4)
        assert torch.equal(lk_a, lk_b) and torch.equal(lv_a, lv_b)
        # and against the CPU oracle on its own: prefix part, local part (new row appended), merge
        t = t0 + call
        prefix = x["prefix"].cpu()
        po, pl = orc.attend(q.cpu(), prefix[:, :, 0].transpose(0, 1), prefix[:, :, 1].transpose(0, 1))
        so, sl = orc.attend(q.cpu(), lk_b[:t + 1].cpu(), lv_b[:t + 1].cpu())
        assert_out_close(out_b.float().cpu(), orc.combine(po, so, pl, sl), dtype, call)
        assert torch.equal(lk_b[t].cpu(), nk.cpu()) and torch.equal(lv_b[t].cpu(), nv.cpu())


def test_static_scratch_rejects_shapes_beyond_its_capacity(native):
    lib = native.lib()
    # head_dim far beyond what 2 MiB of partials can hold is refused before any CUDA work
    assert lib.da_decode_attention_workspace_bytes(1, 8, 4096) > lib.da_decode_attention_static_capacity()
    rc = lib.da_decode_attention_static(256, 256, 4096, 16, 256, 256, 1024, 128, 64, 256, 256, 0, 0, 0, 256, 0,
                                        256, 1, 8, 4096, 2, 0)
    assert rc == -7
    assert b"built-in buffer" in lib.da_error_string(rc)

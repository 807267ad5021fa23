"""No-GPU checks of the boundary: the shared library loads, exports every symbol
the header declares, and rejects bad arguments on the host before touching CUDA."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dram_attention_b200.h")


@pytest.fixture(scope="module")
def native():
    from dram_attention_b200 import _native, build
    build.build()
    return _native


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"DA_API\s+[\w\s\*]+?\b(da_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for n in ["da_version", "da_error_string", "da_score_pages", "da_topk_pages", "da_lru_update",
              "da_fetch_pages", "da_decode_attention", "da_decode_attention_fetch",
              "da_decode_attention_static", "da_decode_attention_workspace_bytes", "da_decode_attention_phased",
              "da_decode_attention_phased_supported", "da_decode_attention_tokens",
              "da_build_pages"]:
        assert n in names


def test_library_exports_every_declared_symbol(native):
    handle = ctypes.CDLL(native.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(handle, name), name
    # and the Python binding covers every one of them
    assert sorted(native._SIGNATURES) == declared_symbols()


def test_version_and_error_text(native):
    lib = native.lib()
    assert lib.da_version() >= 100
    assert lib.da_error_string(0) == b"ok"
    assert b"null" in lib.da_error_string(-1)
    assert b"unknown" in lib.da_error_string(-99)


def test_host_side_argument_checks(native):
    lib = native.lib()
    assert lib.da_score_pages(0, 0, 0, 1, 1, 1, 1, 1, 0, 0, 0) == -1           # null pointers
    assert lib.da_score_pages(16, 16, 16, 1, 1, 1, 0, 1, 0, 0, 0) == -2         # zero pages
    assert lib.da_score_pages(16, 16, 16, 1, 1, 1, 1, 1, 7, 0, 0) == -3         # bad dtype
    assert lib.da_topk_pages(16, 16, 1, 1, 1, 8, 9, 0) == -2                 # k > pages
    assert lib.da_topk_pages(16, 16, 1, 1, 1, 10000, 5000, 0) == -5          # k too large
    assert lib.da_lru_update(16, 4, 16, 8, 16, 16, 9000, 16, 1, 16, 16, 16, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 16, 0) == -5
    # the four arrays of the eviction queue come together or not at all
    assert lib.da_lru_update(16, 4, 16, 8, 16, 16, 64, 16, 1, 16, 16, 16, 0, 16, 16, 16, 0, 8, 0, 0, 0, 0, 0, 16, 0) == -1
    assert lib.da_fetch_pages(0, 16, 16, 16, 16, 1, 1, 1, 1, 16, 0) == -1
    assert lib.da_decode_attention_phased_supported(8, 4, 128, 2, 2048, 16, 4160) == 1
    assert lib.da_decode_attention_phased_supported(8, 4, 128, 2, 2048, 8, 4160) == 0     # page < 16 tokens
    assert lib.da_decode_attention_phased_supported(8, 4, 128, 0, 2048, 16, 4160) == 0     # fp32, D 128: CTA too big
    ws = lib.da_decode_attention_workspace_bytes(8, 4, 128)
    assert ws == 1024 + 8 * 55 * 4 * 132 * 4
    assert lib.da_decode_attention_tokens_workspace_bytes(8, 4, 128, 3) == 1024 + 8 * 55 * 12 * 132 * 4
    assert lib.da_decode_attention_tokens_workspace_bytes(8, 4, 128, 9) == 1024 + 8 * 55 * 16 * 132 * 4
    assert lib.da_decode_attention_phased_workspace_bytes(8, 4, 128) == 1024 + 8 * (148 + 148) * 4 * 132 * 4
    args = [256, 256, 4096, 16, 256, 256, 1024, 128, 64, 256, 256, 0, 0, 0, 256, 0, 256, ws, 256,
            8, 4, 128, 2, 0]
    bad = list(args); bad[21] = 96
    assert lib.da_decode_attention(*bad) == -5                                # head_dim
    bad = list(args); bad[0] = 8
    assert lib.da_decode_attention(*bad) == -4                                # alignment
    bad = list(args); bad[17] = 16
    assert lib.da_decode_attention(*bad) == -6                                # workspace
    bad = list(args); bad[22] = 9
    assert lib.da_decode_attention(*bad) == -3                                # dtype
    bad = list(args); bad[20] = 17
    assert lib.da_decode_attention(*bad) == -5                                # GQA group wider than a launch


def test_operator_refuses_cpu_tensors(native):
    import torch
    import dram_attention_b200 as da
    m = da.DRAMAttention(max_output_length=4, lru_hbm_cache_size=64, local_cache_size=32, page_size=16,
                         top_k=32, n_kv_heads=2, head_dim=64, device="cpu", dtype=torch.float32)
    with pytest.raises(RuntimeError, match="Unsupported stage"):
        m(torch.zeros(1, 1, 4, 64), torch.zeros(1, 1, 2, 64), torch.zeros(1, 1, 2, 64), start_pos=0,
          stage="invalid")
    with pytest.raises(AssertionError, match="Only support batch size 1"):
        m(torch.zeros(2, 1, 4, 64), torch.zeros(2, 1, 2, 64), torch.zeros(2, 1, 2, 64), start_pos=0,
          stage="prefill")
    with pytest.raises(RuntimeError, match="no CPU path"):
        da.max_inner_product(torch.zeros(1, 1, 4), torch.zeros(1, 2, 2, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        m.init_cache(torch.zeros(1, 128, 2, 64), torch.zeros(1, 128, 2, 64))


def test_synthetic_workloads_are_deterministic():
    import torch
    from dram_attention_b200.synthetic import llama_layer_workload, plumbing_workload, scorer_workload
    a, b = plumbing_workload(0, 4), plumbing_workload(0, 4)
    assert torch.equal(a.k, b.k) and torch.equal(a.xq, b.xq)
    assert a.dram_tokens == 4096 and a.prefill_len == 4336
    w = llama_layer_workload(steps=2, dram_tokens=2048, n_kv_heads=2, lru=512, local=256, top_k=256)
    assert w.k.shape == (1, 2048 + 256 - 16, 2, 128) and w.k.dtype == torch.bfloat16
    assert w.dram_tokens == 2048 and w.xq.shape == (2, 1, 1, 8, 128)
    q, mm = scorer_workload(pages=64, n_kv_heads=2)
    assert mm.shape == (2, 64, 2, 128) and bool((mm[:, :, 0] <= mm[:, :, 1]).all())

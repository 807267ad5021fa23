"""The CPU oracle against the reference: the reference's own known-answer
cases (restated from its test files) and golden vectors produced by running
the reference's code (tests/golden/make_golden.py)."""

import os

import numpy as np
import pytest
import torch

from oracle import dram_attention_oracle as orc
from dram_attention_b200.synthetic import plumbing_workload


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


# ---- scorer ---------------------------------------------------------------

def test_scorer_matches_reference_values(golden_dir):
    # shape and tolerance of dram_attention/max_ip_triton_kernel_test.py:29-38
    g = _load(golden_dir, "scorer_values.npz")
    out = orc.score_pages(torch.from_numpy(g["q"]), torch.from_numpy(g["min_max"]))
    assert out.shape == (2, 4, 16)
    assert torch.allclose(out, torch.from_numpy(g["out_ref"]), rtol=1e-3, atol=1e-3)
    assert torch.allclose(out, torch.from_numpy(g["out_triton"]), rtol=1e-3, atol=1e-3)


def test_scorer_degenerate_shape():
    # dram_attention/max_ip_triton_kernel_test.py:41-49
    q = torch.tensor([[[2.0]]])
    mm = torch.tensor([[[[-3.0], [0.5]]]])
    assert orc.score_pages(q, mm).shape == (1, 1, 1)
    assert float(orc.score_pages(q, mm)) == 1.0
    assert float(orc.score_pages(-q, mm)) == 6.0


def test_selection_is_stable_descending():
    s = torch.tensor([[1.0, 3.0, 3.0, -0.0, 0.0, 2.0]])
    assert orc.select_pages(s, 4).tolist() == [[1, 2, 5, 0]]
    assert orc.select_pages(torch.zeros(1, 5), 3).tolist() == [[0, 1, 2]]
    # -0.0 and +0.0 tie: lowest index first
    assert orc.select_pages(torch.tensor([[-1.0, -0.0, 0.0]]), 2).tolist() == [[1, 2]]


# ---- LRU: the three known-answer cases of the reference ---------------------

def _kat_tables(num_heads=2, ld=8, nh=4):
    times = np.tile(np.arange(nh), (num_heads, 1)).astype(np.int64)
    d2h = np.full((num_heads, ld), -1, dtype=np.int64)
    h2d = np.full((num_heads, nh), -1, dtype=np.int64)
    return times, d2h, h2d


@pytest.mark.parametrize("fn", [orc.lru_walk, orc.lru_vectorised])
def test_lru_known_answer_cold_load(fn):
    # dram_attention/lru_triton_kernel_test.py:17-76
    rng = np.random.default_rng(0)
    dram = rng.standard_normal((2, 8, 64)).astype(np.float32)
    hbm = np.zeros((2, 4, 64), np.float32)
    times, d2h, h2d = _kat_tables()
    lst = np.array([[0, 1], [1, 2]])
    fn(lst, d2h, h2d, times, 4, dram, hbm)
    assert np.array_equal(hbm[0, 0], dram[0, 0]) and np.array_equal(hbm[0, 1], dram[0, 1])
    assert np.array_equal(hbm[1, 0], dram[1, 1]) and np.array_equal(hbm[1, 1], dram[1, 2])
    assert times[:, :2].tolist() == [[4, 4], [4, 4]]
    assert (d2h[0, 0], d2h[0, 1], d2h[1, 1], d2h[1, 2]) == (0, 1, 0, 1)
    assert h2d[:, :2].tolist() == [[0, 1], [1, 2]]


@pytest.mark.parametrize("fn", [orc.lru_walk, orc.lru_vectorised])
def test_lru_known_answer_eviction(fn):
    # dram_attention/lru_triton_kernel_test.py:78-143
    rng = np.random.default_rng(1)
    dram = rng.standard_normal((2, 8, 64)).astype(np.float32)
    hbm = dram[:, :4].copy()
    times, d2h, h2d = _kat_tables()
    d2h[:, :4] = np.arange(4)
    h2d[:, :] = np.arange(4)
    lst = np.array([[4, 5], [5, 6]])
    fn(lst, d2h, h2d, times, 4, dram, hbm)
    assert np.array_equal(hbm[0, 0], dram[0, 4]) and np.array_equal(hbm[0, 1], dram[0, 5])
    assert np.array_equal(hbm[1, 0], dram[1, 5]) and np.array_equal(hbm[1, 1], dram[1, 6])
    assert (d2h[0, 4], d2h[0, 5], d2h[1, 5], d2h[1, 6]) == (0, 1, 0, 1)
    assert h2d[:, :2].tolist() == [[4, 5], [5, 6]]
    assert times[:, :2].tolist() == [[4, 4], [4, 4]]
    # evicted pages are unmapped
    assert d2h[0, 0] == -1 and d2h[0, 1] == -1 and d2h[1, 0] == -1 and d2h[1, 1] == -1


@pytest.mark.parametrize("fn", [orc.lru_walk, orc.lru_vectorised])
def test_lru_known_answer_per_head_lists(fn):
    # dram_attention/lru_triton_kernel_test.py:145-204
    rng = np.random.default_rng(2)
    dram = rng.standard_normal((2, 8, 64)).astype(np.float32)
    hbm = np.zeros((2, 4, 64), np.float32)
    times, d2h, h2d = _kat_tables()
    lst = np.array([[0, 2], [1, 3]])
    fn(lst, d2h, h2d, times, 4, dram, hbm)
    assert np.array_equal(hbm[0, 1], dram[0, 2]) and np.array_equal(hbm[1, 1], dram[1, 3])
    assert (d2h[0, 0], d2h[0, 2], d2h[1, 1], d2h[1, 3]) == (0, 1, 0, 1)
    assert h2d[:, :2].tolist() == [[0, 2], [1, 3]]
    assert times[:, :2].tolist() == [[4, 4], [4, 4]]


@pytest.mark.parametrize("fn", [orc.lru_walk, orc.lru_vectorised])
def test_lru_matches_reference_kernel_runs(golden_dir, fn):
    """Tables after every step equal those the reference's own kernels produced."""
    g = _load(golden_dir, "lru_kernel_cases.npz")
    for c in range(int(g["n_cases"][0])):
        dram = g[f"c{c}_dram"]
        lists = g[f"c{c}_lists"]
        hk, ld, _ = dram.shape
        nh = g[f"c{c}_h2d"].shape[2]
        hbm = dram[:, ld - nh:].copy()
        times = np.zeros((hk, nh), np.int64)
        d2h = np.full((hk, ld), -1, np.int64)
        d2h[:, ld - nh:] = np.arange(nh)
        h2d = np.tile(np.arange(ld - nh, ld), (hk, 1)).astype(np.int64)
        for s in range(lists.shape[0]):
            fn(lists[s].astype(np.int64), d2h, h2d, times, s + 1, dram, hbm)
            assert np.array_equal(d2h, g[f"c{c}_d2h"][s]), (c, s)
            assert np.array_equal(h2d, g[f"c{c}_h2d"][s]), (c, s)
            assert np.array_equal(times, g[f"c{c}_time"][s]), (c, s)
            assert np.array_equal(hbm, g[f"c{c}_hbm"][s]), (c, s)


def test_lru_rejects_more_distinct_pages_than_slots():
    times, d2h, h2d = _kat_tables(1, 8, 2)
    d2h[0, 6:] = [0, 1]
    h2d[0] = [6, 7]
    with pytest.raises(ValueError):
        orc.lru_vectorised(np.array([[0, 1, 2]]), d2h, h2d, times, 5)


# ---- whole generate step: trajectories of the reference's DRAMAttention -------

def _run_oracle(ctor, k, v, xq, xk, xv, sequential):
    m = orc.OracleDRAMAttention(dtype=torch.float32, **ctor)
    m.init_cache(k, v)
    m.lru_cache.sequential = sequential
    s = k.shape[1]
    traces = []
    for i in range(xq.shape[0]):
        t = m.generate(xq[i], xk[i], xv[i], s + i)
        t.h2d = m.lru_cache.h2d.copy()
        t.time = m.lru_cache.page_access_time.copy()
        traces.append(t)
    return m, traces


@pytest.mark.parametrize("sequential", [True, False])
def test_mini_trajectory_matches_reference(golden_dir, sequential):
    g = _load(golden_dir, "mini_traj.npz")
    max_out, lru, local, p, top_k, hk, d = [int(x) for x in g["ctor"]]
    ctor = dict(max_output_length=max_out, lru_hbm_cache_size=lru, local_cache_size=local,
                page_size=p, top_k=top_k, n_kv_heads=hk, head_dim=d)
    f = lambda a: torch.from_numpy(a).float() / 8.0
    m, traces = _run_oracle(ctor, f(g["k8"]), f(g["v8"]), f(g["q8"]), f(g["xk8"]),
                            f(g["xv8"]), sequential)
    assert m.dram_kv_cache_size == int(g["dram_tokens"][0])
    for i, t in enumerate(traces):
        assert np.array_equal(t.page_list, g["lists"][i]), i
        assert np.allclose(t.out.numpy(), g["out"][i], rtol=1e-4, atol=1e-4), i
    assert np.array_equal(m.lru_cache.h2d, g["h2d"][-1])
    assert np.array_equal(m.lru_cache.d2h, g["d2h_final"])
    assert np.array_equal(m.lru_cache.page_access_time, g["time"][-1].astype(np.int64))
    assert m.lru_cache.current_step == int(g["step"][0])


def test_plumbing_trajectory_matches_reference(golden_dir):
    from tests.golden.make_golden import checksum
    g = _load(golden_dir, "plumbing_traj.npz")
    w = plumbing_workload(seed=0, steps=16)
    assert checksum(w.k, w.v, w.xq, w.xk, w.xv)[0] == g["input_checksum"][0], \
        "synthetic generator no longer reproduces the inputs the fixture was made from"
    m, traces = _run_oracle(w.ctor_kwargs(), w.k, w.v, w.xq, w.xk, w.xv, False)
    assert m.dram_kv_cache_size == 4096
    for i, t in enumerate(traces):
        assert np.array_equal(t.page_list, g["lists"][i]), i
        assert np.array_equal(t.h2d, g["h2d"][i]), i
        assert np.array_equal(t.time, g["time"][i].astype(np.int64)), i
        assert np.allclose(t.out.numpy(), g["out"][i], rtol=1e-4, atol=1e-4), i
    assert np.array_equal(m.lru_cache.h2d, g["h2d"][-1])
    assert np.array_equal(m.lru_cache.d2h, g["d2h_final"])
    assert np.array_equal(m.lru_cache.page_access_time, g["time"][-1].astype(np.int64))


@pytest.mark.parametrize("heads", ["hq4_hk1", "hq2_hk2"])
def test_multi_token_generate_matches_reference(golden_dir, heads):
    """Generate calls with several tokens each, run by the reference's own classes (the two
    head layouts its selector accepts with more than one token): lists, tables, the appended
    local rows and every token's output."""
    g = _load(golden_dir, f"multi_traj_{heads}.npz")
    max_out, lru, local, p, top_k, hk, d = [int(x) for x in g["ctor"]]
    ctor = dict(max_output_length=max_out, lru_hbm_cache_size=lru, local_cache_size=local,
                page_size=p, top_k=top_k, n_kv_heads=hk, head_dim=d)
    f = lambda a: torch.from_numpy(a).float() / 8.0
    m = orc.OracleDRAMAttention(dtype=torch.float32, **ctor)
    m.init_cache(f(g["k8"]), f(g["v8"]))
    assert m.dram_kv_cache_size == int(g["dram_tokens"][0])
    q, xk, xv = f(g["q8"]), f(g["xk8"]), f(g["xv8"])
    pos, a = g["k8"].shape[1], 0
    for i, c in enumerate(g["counts"].tolist()):
        t = m.generate(q[:, a:a + c], xk[:, a:a + c], xv[:, a:a + c], pos)
        assert np.array_equal(t.page_list, g[f"list{i}"]), i
        assert np.array_equal(m.lru_cache.h2d, g["h2d"][i]), i
        assert np.array_equal(m.lru_cache.page_access_time, g["time"][i].astype(np.int64)), i
        out = t.out if c > 1 else t.out[None]
        assert np.allclose(out.numpy(), g["out"][a:a + c], rtol=1e-4, atol=1e-4), i
        pos += c
        a += c
    assert np.array_equal(m.lru_cache.d2h, g["d2h_final"])
    assert np.array_equal(m.cache_k.numpy(), g["cache_k"])


def _rope_case(g, name):
    """(xq, xk, freqs, want_q, want_k) of the rope fixture in its own dtype."""
    freqs = torch.view_as_complex(torch.from_numpy(g["freqs"]).contiguous())
    if name == "f32":
        conv = lambda a: torch.from_numpy(a)
    else:
        conv = lambda a: torch.from_numpy(a).view(torch.bfloat16)
    return (conv(g[f"xq_{name}"]), conv(g[f"xk_{name}"]), freqs, conv(g[f"oq_{name}"]), conv(g[f"ok_{name}"]))


@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_rope_matches_reference_caller(golden_dir, name):
    """The rotary embedding in front of the operator call, as the reference's model file applies
    it (precompute_freqs_cis rows at scattered positions up to 199 999): bit for bit."""
    xq, xk, freqs, want_q, want_k = _rope_case(_load(golden_dir, "rope_values.npz"), name)
    got_q, got_k = orc.rope_qk(xq, xk, freqs)
    assert got_q.dtype == xq.dtype
    assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)

"""GPU parity tests, stage by stage: every CUDA kernel is called through the
C ABI (via the ctypes binding) and compared with the CPU oracle on the same
inputs.  Integer results are bit-exact; float tolerances are written per test."""

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import dram_attention_oracle as orc  # noqa: E402
from tests.conftest import assert_out_close  # noqa: E402

DEV = "cuda"


@pytest.fixture(scope="module")
def da():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dram_attention_b200 as pkg
    pkg._native.lib()
    return pkg


def _g(seed):
    return torch.Generator().manual_seed(seed)


# ------------------------------------------------------------------ scorer ----

def test_scorer_reference_value_case(da, golden_dir):
    # shape and tolerance of dram_attention/max_ip_triton_kernel_test.py:29-38
    g = np.load(os.path.join(golden_dir, "scorer_values.npz"))
    q, mm = torch.from_numpy(g["q"]).to(DEV), torch.from_numpy(g["min_max"]).to(DEV)
    out = da.max_inner_product(q, mm)
    assert out.shape == (2, 4, 16) and out.dtype == torch.float32
    assert torch.allclose(out.cpu(), torch.from_numpy(g["out_ref"]), rtol=1e-3, atol=1e-3)
    assert torch.allclose(out, da.max_ip_ref(q, mm), rtol=1e-3, atol=1e-3)


def test_scorer_output_dtype_follows_query(da):
    # dram_attention/max_ip_triton_kernel_test.py:18-26
    q = torch.randn(2, 4, 64, dtype=torch.float16, device=DEV)
    mm = torch.randn(4, 16, 2, 64, dtype=torch.float16, device=DEV)
    assert da.max_inner_product(q, mm).dtype == torch.float16


def test_scorer_degenerate_and_large_shapes(da):
    # dram_attention/max_ip_triton_kernel_test.py:41-60
    q = torch.randn(1, 1, 1, device=DEV)
    mm = torch.randn(1, 1, 2, 1, device=DEV)
    out = da.max_inner_product(q, mm)
    assert out.shape == (1, 1, 1)
    assert torch.allclose(out, da.max_ip_ref(q, mm), rtol=1e-5, atol=1e-6)
    q = torch.randn(32, 32, 128, device=DEV)
    mm = torch.randn(32, 1024, 2, 128, device=DEV)
    out = da.max_inner_product(q, mm)
    assert out.shape == (32, 32, 1024)
    ref = orc.score_pages(q.cpu(), mm.cpu())
    assert torch.allclose(out.cpu(), ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype,d,rep,hk,pages", [
    (torch.bfloat16, 128, 4, 8, 8192), (torch.bfloat16, 128, 4, 2, 1), (torch.bfloat16, 128, 4, 2, 3),
    (torch.bfloat16, 128, 2, 3, 513), (torch.bfloat16, 128, 1, 2, 1000), (torch.float16, 128, 4, 2, 77),
    (torch.float32, 64, 4, 2, 256), (torch.float32, 128, 4, 2, 130), (torch.bfloat16, 64, 2, 2, 65),
    (torch.bfloat16, 128, 8, 2, 100), (torch.float32, 96, 3, 2, 50), (torch.bfloat16, 128, 4, 8, 65536),
])
@pytest.mark.parametrize("ordered", [False, True])
def test_scorer_folded_matches_oracle(da, dtype, d, rep, hk, pages, ordered):
    from dram_attention_b200.max_ip import score_pages_
    g = _g(pages + d + rep)
    keys = torch.randn(hk, pages, 4, d, generator=g).to(dtype)
    mm = orc.page_minmax(keys.reshape(hk, pages * 4, d), pages)
    q = torch.randn(1, 1, hk * rep, d, generator=g).to(dtype)
    scores = torch.empty(1, hk * rep, pages, dtype=torch.float32, device=DEV)
    score_pages_(q.to(DEV), mm.to(DEV).contiguous(), scores, 1, hk, rep, ordered=ordered)
    ref = orc.scores_by_query_head(q, mm).reshape(1, hk * rep, pages)
    # 1e-3 relative to the score scale (fp32 accumulation on both sides)
    scale = ref.abs().max().item()
    assert (scores.cpu() - ref).abs().max().item() <= 1e-3 * max(scale, 1.0)
    assert torch.allclose(scores.cpu(), ref, rtol=1e-3, atol=1e-3 * max(scale, 1.0))


def test_scorer_multi_token(da):
    from dram_attention_b200.max_ip import score_pages_
    g = _g(5)
    hk, rep, d, pages, s = 4, 2, 64, 200, 10
    mm = torch.sort(torch.randn(hk, pages, 2, d, generator=g), dim=2).values
    q = torch.randn(1, s, hk * rep, d, generator=g)
    scores = torch.empty(s, hk * rep, pages, dtype=torch.float32, device=DEV)
    score_pages_(q.to(DEV), mm.to(DEV), scores, s, hk, rep, ordered=True)
    ref = orc.scores_by_query_head(q, mm).reshape(s, hk * rep, pages)
    assert torch.allclose(scores.cpu(), ref, rtol=1e-3, atol=1e-3)


# ------------------------------------------------------------------- top-k ----

def _topk(da, scores, hk, rep, k):
    from dram_attention_b200 import _native
    s, hq, pages = scores.shape
    sc = scores.to(DEV).contiguous()
    out = torch.full((hk, s * rep * k), -7, dtype=torch.int32, device=DEV)
    _native.check(_native.lib().da_topk_pages(sc.data_ptr(), out.data_ptr(), s, hk, rep, pages, k,
                                              _native.stream_ptr()))
    return out.cpu()


def _topk_oracle(scores, hk, rep, k):
    s, hq, pages = scores.shape
    idx = orc.select_pages(scores.reshape(s, hk, rep, pages), k)
    return orc.build_page_list(idx).to(torch.int32)


@pytest.mark.parametrize("pages,k,hk,rep,s,kind", [
    (8192, 256, 8, 4, 1, "normal"), (256, 32, 2, 4, 1, "normal"), (1000, 100, 2, 2, 3, "normal"),
    (65536, 256, 2, 4, 1, "normal"), (65536, 512, 1, 4, 1, "normal"), (5000, 2048, 1, 2, 1, "normal"),
    (300, 300, 2, 1, 1, "normal"), (4096, 4096, 1, 1, 1, "normal"), (1, 1, 2, 2, 1, "normal"),
    (8192, 256, 2, 4, 1, "quantised"), (3000, 500, 2, 2, 1, "quantised"), (2048, 64, 2, 2, 1, "constant"),
    (4096, 100, 2, 2, 1, "zeros"), (1500, 200, 2, 2, 1, "bf16like"), (2000, 128, 2, 2, 1, "negative"),
    # rows of more than 16384 pages: a cluster of four CTAs per row (uneven parts, ties, the fall-back)
    (20000, 300, 1, 2, 1, "normal"), (16385, 64, 1, 1, 2, "bf16like"), (65536, 4096, 1, 1, 1, "normal"),
    (65536, 256, 1, 2, 1, "quantised"), (30000, 128, 1, 2, 1, "constant"), (40000, 200, 1, 2, 1, "zeros"),
    (50000, 100, 1, 2, 1, "negative"), (65536, 256, 1, 2, 1, "outlier"), (65534, 512, 2, 4, 1, "normal"),
])
def test_topk_bit_exact(da, pages, k, hk, rep, s, kind):
    g = _g(pages * 7 + k)
    sc = torch.randn(s, hk * rep, pages, generator=g) * 30
    if kind == "quantised":
        sc = torch.round(sc / 8)            # a few dozen distinct values: heavy ties
    elif kind == "constant":
        sc = torch.full_like(sc, 3.25)
    elif kind == "zeros":
        sc = torch.where(torch.rand(sc.shape, generator=g) < 0.5, torch.zeros_like(sc), -torch.zeros_like(sc))
        sc[..., ::7] = -1.0
    elif kind == "bf16like":
        sc = sc.to(torch.bfloat16).float()  # the reference's own score resolution
    elif kind == "negative":
        sc = -sc.abs() - 1
    elif kind == "outlier":
        sc[..., 5] = 1e30                   # the row's range is useless for equal-width buckets
        sc[..., 77] = -1e30
    got = _topk(da, sc, hk, rep, k)
    want = _topk_oracle(sc, hk, rep, k)
    assert torch.equal(got, want)


def test_topk_selector_api(da):
    # IPUpperboundTopKSelector.top_k returns (S, Hk, rep, k) int64 like the reference
    g = _g(3)
    hk, rep, d, pages, p = 2, 2, 64, 64, 16
    keys = torch.randn(hk, pages * p, d, generator=g)
    q = torch.randn(1, 3, hk * rep, d, generator=g)
    sel = da.topk_selector.IPUpperboundTopKSelector(keys.to(DEV), pages, device=DEV)
    assert torch.equal(sel.chunk_min_max.cpu(), orc.page_minmax(keys, pages))
    idx = sel.top_k(q.to(DEV), 8)
    assert idx.shape == (3, hk, rep, 8) and idx.dtype == torch.int64
    want = orc.select_pages(orc.scores_by_query_head(q, orc.page_minmax(keys, pages)), 8)
    # scores can differ in the last bits between CPU and GPU summation orders: compare as
    # sets per row unless the k-th gap is tiny (it is not for random normal data)
    assert torch.equal(idx.cpu(), want)


# --------------------------------------------------------------------- LRU ----

class Tables:
    def __init__(self, hk, ld, nh, page_dim=64, dtype=torch.float32, seed=0, warm=True, times=None):
        self.hk, self.ld, self.nh = hk, ld, nh
        self.dram = torch.randn(hk, ld, page_dim, generator=_g(seed)).to(dtype)
        self.d2h = np.full((hk, ld), -1, np.int64)
        self.h2d = np.full((hk, nh), -1, np.int64)
        self.time = np.zeros((hk, nh), np.int64) if times is None else times.astype(np.int64).copy()
        self.hbm = torch.zeros(hk, nh, page_dim, dtype=dtype)
        if warm:
            self.d2h[:, ld - nh:] = np.arange(nh)
            self.h2d[:] = np.arange(ld - nh, ld)
            self.hbm = self.dram[:, ld - nh:].clone()
        self.step = 0

    def to_device(self):
        i32 = lambda a: torch.from_numpy(a.astype(np.int32)).to(DEV)
        self.g_d2h, self.g_h2d, self.g_time = i32(self.d2h), i32(self.h2d), i32(self.time)
        self.g_step = torch.full((self.hk,), self.step, dtype=torch.int32, device=DEV)
        self.g_dram = self.dram.clone().pin_memory()
        self.g_hbm = self.hbm.to(DEV)
        self.g_status = torch.zeros(1, dtype=torch.int32, device=DEV)
        # eviction queue: the slots sorted by (time, slot); the update advances the flip itself.
        # use_queue = False exercises the kernel that selects its victims on the timestamps.
        order = np.stack([np.argsort(self.time[h], kind="stable") for h in range(self.hk)])
        self.g_order = torch.from_numpy(np.stack([order, order]).astype(np.int32)).to(DEV)
        self.split_cap = max(1, self.nh // 4)
        self.g_nev = torch.full((2, self.hk), self.split_cap, dtype=torch.int32, device=DEV)
        self.g_flip = torch.zeros(self.hk, dtype=torch.int32, device=DEV)
        self.g_redo = torch.zeros(3, self.hk, dtype=torch.int32, device=DEV)
        self.g_redo[0] = -5
        self.miss_total = np.zeros(self.hk, np.int64)
        self.g_src = torch.full((self.hk, self.nh), -1, dtype=torch.int32, device=DEV)
        self.g_prev = None
        return self

    def gpu_step(self, lst, use_queue=True, inline=0):
        """One da_lru_update (+ da_fetch_pages for what the update did not copy itself)."""
        from dram_attention_b200 import _native
        lib, s = _native.lib(), _native.stream_ptr()
        kk = lst.shape[1]
        gl = torch.from_numpy(lst.astype(np.int32)).to(DEV)
        if self.g_prev is None or self.g_prev[0].shape[1] != kk:
            self.g_prev = (torch.full((self.hk, kk), -9, dtype=torch.int32, device=DEV),
                           torch.full((self.hk, kk), -9, dtype=torch.int32, device=DEV),
                           torch.zeros(self.hk, dtype=torch.int32, device=DEV))
            self.g_src.fill_(-1)
        mp, ms, nm = self.g_prev
        page_bytes = self.dram.shape[2] * self.dram.element_size()
        if use_queue:
            flip = self.g_flip.cpu().numpy()
            cur_order = np.stack([self.g_order[flip[h], h].cpu().numpy() for h in range(self.hk)])
            cur_nev = np.array([int(self.g_nev[flip[h], h]) for h in range(self.hk)])
            before = self.g_order.clone()
        q = (self.g_order.data_ptr(), self.g_nev.data_ptr(), self.g_flip.data_ptr(), self.g_redo.data_ptr()) \
            if use_queue else (0, 0, 0, 0)
        _native.check(lib.da_lru_update(gl.data_ptr(), kk, self.g_d2h.data_ptr(), self.ld,
                                        self.g_h2d.data_ptr(), self.g_time.data_ptr(), self.nh,
                                        self.g_step.data_ptr(), self.hk, mp.data_ptr(), ms.data_ptr(),
                                        nm.data_ptr(), self.g_src.data_ptr(), *q, self.split_cap, 1,
                                        self.g_dram.data_ptr() if inline else 0,
                                        self.g_hbm.data_ptr() if inline else 0, page_bytes, inline,
                                        self.g_status.data_ptr(), s))
        torch.cuda.synchronize()
        mp_h, ms_h, nm_h = mp.cpu().numpy(), ms.cpu().numpy(), nm.cpu().numpy()
        src = self.g_src.cpu().numpy()
        copies_here = bool(inline) and use_queue and page_bytes % 16 == 0
        for h in range(self.hk):
            # slot_source marks exactly the pages the update left to somebody else
            want = np.full(self.nh, -1)
            if not (copies_here and nm_h[h] <= inline):
                want[ms_h[h, :nm_h[h]]] = mp_h[h, :nm_h[h]]
            assert np.array_equal(src[h], want), h
            if copies_here and nm_h[h] <= inline and nm_h[h] > 0:
                # ... and has already brought its own pages in
                got = self.g_hbm[h, torch.from_numpy(ms_h[h, :nm_h[h]]).long().to(DEV)].cpu()
                assert torch.equal(got, self.dram[h, torch.from_numpy(mp_h[h, :nm_h[h]]).long()]), h
        _native.check(lib.da_fetch_pages(self.g_dram.data_ptr(), self.g_hbm.data_ptr(), mp.data_ptr(),
                                         ms.data_ptr(), nm.data_ptr(), kk, self.hk, self.ld, self.nh,
                                         page_bytes, s))
        torch.cuda.synchronize()
        if use_queue and not (int(self.g_status) & 2):
            redo = self.g_redo[0].cpu().numpy()
            self.miss_total += nm_h
            assert np.array_equal(self.g_redo[1].cpu().numpy(), self.miss_total)
            new_flip = self.g_flip.cpu().numpy()
            times = self.g_time.cpu().numpy()
            for h in range(self.hk):
                # redo flag: exactly "a victim of this call lay beyond the front that was current"
                outside = not (set(ms_h[h, :nm_h[h]].tolist()) <= set(cur_order[h, :cur_nev[h]].tolist()))
                assert redo[h] == int(outside), (h, redo[h], outside)
                assert new_flip[h] == 1 - flip[h], h          # split_advance = 1
                # the copy that was current is untouched; the other one is the new eviction order
                assert torch.equal(self.g_order[flip[h], h], before[flip[h], h])
                order = self.g_order[new_flip[h], h].cpu().numpy()
                assert np.array_equal(order, np.argsort(times[h], kind="stable")), h
                assert int(self.g_nev[new_flip[h], h]) == min(self.split_cap, self.nh), h
        return mp_h, ms_h, nm_h

    def cpu_step(self, lst, fn=orc.lru_walk):
        self.step += 1
        mp, ms, nm = fn(lst.astype(np.int64), self.d2h, self.h2d, self.time, self.step)
        for h in range(self.hk):
            m = int(nm[h])
            if m:
                self.hbm[h, torch.from_numpy(ms[h, :m])] = self.dram[h, torch.from_numpy(mp[h, :m])]
        return mp, ms, nm

    def assert_equal(self, tag=""):
        assert np.array_equal(self.g_d2h.cpu().numpy(), self.d2h), tag
        assert np.array_equal(self.g_h2d.cpu().numpy(), self.h2d), tag
        assert np.array_equal(self.g_time.cpu().numpy(), self.time), tag
        assert torch.equal(self.g_hbm.cpu(), self.hbm), tag
        assert int(self.g_step[0]) == self.step and int(self.g_step[-1]) == self.step, tag


@pytest.mark.parametrize("lists,prefill", [
    ([[0, 1], [1, 2]], False),     # dram_attention/lru_triton_kernel_test.py:17-76 (cold load)
    ([[4, 5], [5, 6]], True),      # :78-143 (eviction of the oldest slots)
    ([[0, 2], [1, 3]], False),     # :145-204 (per-head lists)
])
def test_lru_reference_known_answers(da, lists, prefill):
    t = Tables(2, 8, 4, warm=False, times=np.tile(np.arange(4), (2, 1)))
    if prefill:
        t.d2h[:, :4] = np.arange(4)
        t.h2d[:] = np.arange(4)
        t.hbm = t.dram[:, :4].clone()
    t.step = 3  # the kernel increments: the reference test passes step 4
    t.to_device()
    lst = np.array(lists)
    mp, ms, nm = t.gpu_step(lst)
    hbm, dram = t.g_hbm.cpu(), t.dram
    for h in range(2):
        for j in range(2):
            assert torch.equal(hbm[h, j], dram[h, lst[h, j]])
            assert int(t.g_d2h[h, lst[h, j]]) == j
            assert int(t.g_h2d[h, j]) == lst[h, j]
            assert int(t.g_time[h, j]) == 4
    assert nm.tolist() == [2, 2] and ms[:, :2].tolist() == [[0, 1], [0, 1]]
    if prefill:
        assert t.g_d2h[:, :2].cpu().tolist() == [[-1, -1], [-1, -1]]
    assert int(t.g_status) == 0 and t.g_step.cpu().tolist() == [4, 4]


def test_lru_matches_reference_kernel_runs(da, golden_dir):
    g = np.load(os.path.join(golden_dir, "lru_kernel_cases.npz"))
    for c in range(int(g["n_cases"][0])):
        dram = g[f"c{c}_dram"]
        lists = g[f"c{c}_lists"]
        hk, ld, pd = dram.shape
        nh = g[f"c{c}_h2d"].shape[2]
        t = Tables(hk, ld, nh, page_dim=pd)
        t.dram = torch.from_numpy(dram)
        t.hbm = t.dram[:, ld - nh:].clone()
        t.to_device()
        for s in range(lists.shape[0]):
            t.gpu_step(lists[s])
            assert np.array_equal(t.g_d2h.cpu().numpy(), g[f"c{c}_d2h"][s]), (c, s)
            assert np.array_equal(t.g_h2d.cpu().numpy(), g[f"c{c}_h2d"][s]), (c, s)
            assert np.array_equal(t.g_time.cpu().numpy(), g[f"c{c}_time"][s]), (c, s)
            assert np.array_equal(t.g_hbm.cpu().numpy(), g[f"c{c}_hbm"][s]), (c, s)
        assert int(t.g_status) == 0


@pytest.mark.parametrize("hk,ld,nh,kk,steps,page_dim,dtype", [
    (2, 256, 128, 128, 12, 2048, torch.float32),      # plumbing geometry
    (8, 8192, 2048, 1024, 6, 4096, torch.bfloat16),   # Llama layer geometry
    (3, 100, 37, 20, 40, 24, torch.float32),          # odd sizes, page not a multiple of 16 bytes... (96 B ok)
    (2, 70, 33, 33, 30, 3, torch.float32),            # 12-byte pages: bytewise copy path
    (1, 9000, 8192, 4000, 4, 8, torch.float32),       # largest slot table
    (2, 5000, 4096, 2048, 5, 64, torch.bfloat16),     # 1M-context layer geometry (per-head)
    (2, 600, 300, 300, 300, 8, torch.float32),        # many steps: > 8 bits of time
])
@pytest.mark.parametrize("mode", ["queue", "queue+copy", "select"])
def test_lru_random_trajectories_bit_exact(da, hk, ld, nh, kk, steps, page_dim, dtype, mode):
    """queue: victims from the eviction queue; queue+copy: the update also copies the pages of
    heads that miss at most 6; select: no queue, victims by a select on the timestamps."""
    rng = np.random.default_rng(hk * 1000 + ld)
    t = Tables(hk, ld, nh, page_dim=page_dim, dtype=dtype, seed=ld).to_device()
    kw = dict(use_queue=mode != "select", inline=6 if mode == "queue+copy" else 0)
    for s in range(steps):
        # a hot set that drifts (hits), fresh pages (misses) and duplicates inside the list
        distinct = int(rng.integers(1, min(kk, nh) + 1))
        pool = rng.choice(ld, size=distinct, replace=False)
        lst = rng.choice(pool, size=(hk, kk))
        mp_c, ms_c, nm_c = t.cpu_step(lst)
        mp_g, ms_g, nm_g = t.gpu_step(lst, **kw)
        assert np.array_equal(nm_g, nm_c), s
        for h in range(hk):
            assert np.array_equal(mp_g[h, :nm_c[h]], mp_c[h, :nm_c[h]]), (s, h)
            assert np.array_equal(ms_g[h, :nm_c[h]], ms_c[h, :nm_c[h]]), (s, h)
        t.assert_equal(f"step {s}")
        # invariants: the two maps are inverse of each other; slots hold their page
        d2h, h2d = t.g_d2h.cpu().numpy(), t.g_h2d.cpu().numpy()
        for h in range(hk):
            assert np.array_equal(d2h[h, h2d[h]], np.arange(nh))
            assert (d2h[h] >= 0).sum() == nh
    assert int(t.g_status) == 0


def test_lru_overflow_and_bad_page_are_reported(da):
    t = Tables(1, 16, 4).to_device()
    lst = np.array([[0, 1, 2, 3, 4, 5]])  # 6 distinct non-resident pages, 4 slots
    before = (t.g_d2h.clone(), t.g_h2d.clone())
    t.gpu_step(lst)
    assert int(t.g_status) & 2
    assert torch.equal(t.g_d2h, before[0]) and torch.equal(t.g_h2d, before[1])
    t.g_status.zero_()
    mp, ms, nm = t.gpu_step(np.array([[99, -3, 1, 1, 15, 99]]))
    assert int(t.g_status) & 1
    assert nm.tolist() == [1] and mp[0, 0] == 1
    assert int(t.g_d2h[0, 1]) == int(ms[0, 0])


def test_lru_cache_class_mirrors_reference(da):
    # dram_attention/lru_cache_test.py:16-98
    k = torch.randn(4, 1024 * 8, 64, device=DEV)
    v = torch.randn(4, 1024 * 8, 64, device=DEV)
    c = da.LRUCache(k, v, page_size=16, top_k=10)
    assert (c.num_kv_heads, c.num_dram_pages, c.num_hbm_pages, c.head_dim, c.page_size, c.top_k) == \
        (4, 512, 102, 64, 16, 10)
    assert torch.all(c.dram_page_to_hbm_page_mapping[:, -102:] == torch.arange(102).cuda())
    assert torch.all(c.dram_page_to_hbm_page_mapping[:, :-102] == -1)
    kc, vc = c.load_(torch.randint(0, 512, (4, 10), device=DEV))
    assert kc.shape == (4, 102 * 16, 64) and vc.shape == (4, 102 * 16, 64)
    assert c.current_step == 1
    out = c.get_kv_cache_(torch.randn(1, 10, 4, 64, device=DEV))
    assert out.k_cache.shape == (4, 102 * 16, 64) and out.v_cache.shape == (4, 102 * 16, 64)
    assert c.current_step == 2
    c.get_kv_cache_(torch.randn(1, 10, 4, 64, device=DEV))
    assert c.current_step == 3
    assert out.k_cache.device.type == "cuda" and torch.any(out.k_cache != 0) and torch.any(out.v_cache != 0)
    c.check_status()
    # the slot table holds exactly the pages the map says, keys and values in place
    h2d = c.hbm_page_to_dram_page_mapping.cpu().long()
    kk = k.cpu().view(4, 512, 16, 64)
    vv = v.cpu().view(4, 512, 16, 64)
    for h in range(4):
        assert torch.equal(out.k_cache[h].cpu().view(102, 16, 64), kk[h, h2d[h]])
        assert torch.equal(out.v_cache[h].cpu().view(102, 16, 64), vv[h, h2d[h]])
    for page_size in (8, 16, 32):
        c2 = da.LRUCache(torch.randn(4, 1024 * 8, 64), torch.randn(4, 1024 * 8, 64), page_size=page_size,
                         top_k=10)
        assert c2.page_size == page_size and c2.num_dram_pages == 1024 * 8 // page_size and c2.top_k == 10
    with pytest.raises(AssertionError):
        da.LRUCache(torch.randn(4, 1007 * 8, 64), torch.randn(4, 1007 * 8, 64), page_size=16, top_k=10)
    c3 = da.LRUCache(torch.randn(4, 1024 * 8, 64), torch.randn(4, 1024 * 8, 64), page_size=16,
                     lru_hbm_cache_size=1024, top_k=10)
    assert c3.num_hbm_pages == 64 and c3.top_k == 10


# --------------------------------------------------------------- attention ----

def _attention_case(da, dtype, d, hk, rep, n_prefix, cap, t_new, seed, device_pos, calls=2):
    from dram_attention_b200 import _native
    lib = _native.lib()
    g = _g(seed)
    hq = hk * rep
    prefix = torch.randn(hk, n_prefix, 2, d, generator=g).to(dtype)
    local_k = torch.randn(cap, hk, d, generator=g).to(dtype)
    local_v = torch.randn(cap, hk, d, generator=g).to(dtype)
    dram_tokens = 4096
    ws_bytes = lib.da_decode_attention_workspace_bytes(hk, rep, d)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    g_prefix, g_lk, g_lv = prefix.to(DEV), local_k.to(DEV), local_v.to(DEV)
    for call in range(calls):
        q = (torch.randn(hq, d, generator=g) * 1.5).to(dtype)
        nk = torch.randn(hk, d, generator=g).to(dtype)
        nv = torch.randn(hk, d, generator=g).to(dtype)
        t = t_new + call
        if t >= cap:
            break
        g_q, g_nk, g_nv = q.to(DEV), nk.to(DEV), nv.to(DEV)
        out = torch.empty(hq, d, dtype=dtype, device=DEV)
        lse = torch.empty(hq, dtype=torch.float32, device=DEV)
        pos = torch.tensor([dram_tokens + t], dtype=torch.int32, device=DEV)
        _native.check(lib.da_decode_attention(
            g_q.data_ptr(), g_prefix.data_ptr(), g_prefix.stride(0), n_prefix, g_lk.data_ptr(),
            g_lv.data_ptr(), g_lk.stride(0), g_lk.stride(1), cap, g_nk.data_ptr(), g_nv.data_ptr(),
            pos.data_ptr() if device_pos else 0, 0 if device_pos else dram_tokens + t, dram_tokens,
            out.data_ptr(), lse.data_ptr(), ws.data_ptr(), ws_bytes, status.data_ptr(), hk, rep, d,
            _native.dtype_code(dtype), _native.stream_ptr()))
        torch.cuda.synchronize()
        assert int(status) == 0
        # oracle: append, then prefix part + local part + merge
        local_k[t], local_v[t] = nk, nv
        po, pl = orc.attend(q, prefix[:, :, 0].transpose(0, 1), prefix[:, :, 1].transpose(0, 1))
        so, sl = orc.attend(q, local_k[:t + 1], local_v[:t + 1])
        want = orc.combine(po, so, pl, sl)
        want_lse = torch.logaddexp(pl, sl)
        assert_out_close(out.float().cpu(), want, dtype, call)
        assert torch.allclose(lse.cpu().double(), want_lse, rtol=1e-4, atol=1e-4)
        assert torch.equal(g_lk.cpu(), local_k) and torch.equal(g_lv.cpu(), local_v)
        assert int(ws[:1024].view(torch.int32).abs().sum()) == 0  # tickets back at zero


@pytest.mark.parametrize("dtype,d,hk,rep,n_prefix,cap,t_new,device_pos", [
    (torch.float32, 64, 2, 4, 2048, 272, 240, False),     # plumbing geometry
    (torch.bfloat16, 128, 8, 4, 32768, 4160, 4080, True), # Llama layer geometry
    (torch.bfloat16, 128, 2, 4, 160, 64, 0, True),        # first local token only
    (torch.bfloat16, 128, 2, 4, 24, 64, 15, False),       # prefix not a multiple of 16 tokens
    (torch.bfloat16, 128, 1, 4, 8, 40, 16, True),         # tiny prefix, unit boundary in local
    (torch.float16, 128, 2, 2, 1000, 100, 17, False),
    (torch.float32, 128, 2, 1, 520, 90, 33, True),
    (torch.bfloat16, 64, 3, 8, 700, 50, 47, False),
    (torch.bfloat16, 128, 1, 8, 5000, 300, 255, True),
    (torch.float32, 64, 16, 2, 300, 33, 31, False),
    (torch.bfloat16, 128, 1, 1, 65536, 8224, 8176, True), # one head of the 1M-context layer
])
def test_decode_attention_matches_oracle(da, dtype, d, hk, rep, n_prefix, cap, t_new, device_pos):
    # tolerances (tests/conftest.py:out_tolerance): 1e-4 absolute in float32; 2e-2 absolute
    # plus half an ulp of the stored value in 16-bit types
    _attention_case(da, dtype, d, hk, rep, n_prefix, cap, t_new, n_prefix + t_new, device_pos)


@pytest.mark.parametrize("dtype,d,hk,rep,n_prefix,cap,t0,s_q", [
    (torch.bfloat16, 128, 2, 4, 512, 96, 40, 2),     # 8 rows: the half-tile kernel
    (torch.bfloat16, 128, 2, 4, 512, 96, 40, 4),     # 16 rows: the full tile
    (torch.bfloat16, 128, 1, 4, 1000, 64, 13, 7),    # two launches (4 + 3 tokens), ragged prefix
    (torch.float16, 64, 3, 2, 300, 40, 5, 8),        # 16 rows with rep 2
    (torch.bfloat16, 128, 2, 1, 200, 64, 0, 16),     # 16 tokens of one head each, empty local window before
    (torch.float32, 64, 2, 4, 2048, 272, 240, 2),    # float32: 8 rows per launch
    (torch.float32, 64, 2, 4, 520, 64, 30, 5),       # float32: three launches (2 + 2 + 1)
    (torch.float32, 128, 1, 3, 100, 32, 7, 3),       # a GQA group of three
])
def test_decode_attention_tokens_matches_oracle(da, dtype, d, hk, rep, n_prefix, cap, t0, s_q):
    """Several query tokens per call: each sees the slot table minus its last s-1-i tokens
    and the local window up to its own position (bottom-right causal mask on both parts)."""
    from dram_attention_b200 import _native
    lib = _native.lib()
    g = _g(n_prefix + s_q)
    hq = hk * rep
    prefix = torch.randn(hk, n_prefix, 2, d, generator=g).to(dtype)
    local_k = torch.randn(cap, hk, d, generator=g).to(dtype)
    local_v = torch.randn(cap, hk, d, generator=g).to(dtype)
    q = (torch.randn(s_q, hq, d, generator=g) * 1.5).to(dtype)
    nk = torch.randn(s_q, hk, d, generator=g).to(dtype)
    nv = torch.randn(s_q, hk, d, generator=g).to(dtype)
    dram_tokens = 4096
    ws_bytes = lib.da_decode_attention_tokens_workspace_bytes(hk, rep, d, s_q)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    g_prefix, g_lk, g_lv = prefix.to(DEV), local_k.to(DEV), local_v.to(DEV)
    g_q, g_nk, g_nv = q.to(DEV), nk.to(DEV), nv.to(DEV)
    out = torch.empty(s_q, hq, d, dtype=dtype, device=DEV)
    lse = torch.empty(s_q, hq, dtype=torch.float32, device=DEV)
    _native.check(lib.da_decode_attention_tokens(
        g_q.data_ptr(), s_q, g_prefix.data_ptr(), g_prefix.stride(0), n_prefix, g_lk.data_ptr(),
        g_lv.data_ptr(), g_lk.stride(0), g_lk.stride(1), cap, g_nk.data_ptr(), g_nv.data_ptr(),
        0, dram_tokens + t0, dram_tokens, out.data_ptr(), lse.data_ptr(), ws.data_ptr(), ws_bytes,
        status.data_ptr(), hk, rep, d, _native.dtype_code(dtype), _native.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status) == 0
    local_k[t0:t0 + s_q], local_v[t0:t0 + s_q] = nk, nv
    po, pl = orc.attend_tokens(q, prefix[:, :, 0].transpose(0, 1), prefix[:, :, 1].transpose(0, 1))
    so, sl = orc.attend_tokens(q, local_k[:t0 + s_q], local_v[:t0 + s_q])
    for i in range(s_q):
        assert_out_close(out[i].float().cpu(), orc.combine(po[i], so[i], pl[i], sl[i]), dtype, i)
        assert torch.allclose(lse[i].cpu().double(), torch.logaddexp(pl[i], sl[i]), rtol=1e-4, atol=1e-4)
    assert torch.equal(g_lk.cpu(), local_k) and torch.equal(g_lv.cpu(), local_v)
    assert int(ws[:1024].view(torch.int32).abs().sum()) == 0
    # more tokens than the local window can take, or a group wider than a launch: rejected on the host
    rc = lib.da_decode_attention_tokens(
        g_q.data_ptr(), cap + 1, g_prefix.data_ptr(), g_prefix.stride(0), n_prefix, g_lk.data_ptr(),
        g_lv.data_ptr(), g_lk.stride(0), g_lk.stride(1), cap, g_nk.data_ptr(), g_nv.data_ptr(),
        0, dram_tokens, dram_tokens, out.data_ptr(), 0, ws.data_ptr(), ws_bytes, status.data_ptr(), hk, rep, d,
        _native.dtype_code(dtype), _native.stream_ptr())
    assert rc == -2


def test_decode_attention_bad_position_is_reported(da):
    from dram_attention_b200 import _native
    lib = _native.lib()
    hk, rep, d, n_prefix, cap = 2, 4, 128, 64, 32
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=DEV)
    ws_bytes = lib.da_decode_attention_workspace_bytes(hk, rep, d)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    prefix, lk, lv, q, nk, nv, out = z(hk, n_prefix, 2, d), z(cap, hk, d), z(cap, hk, d), z(hk * rep, d), \
        z(hk, d) + 1, z(hk, d) + 1, z(hk * rep, d)
    _native.check(lib.da_decode_attention(
        q.data_ptr(), prefix.data_ptr(), prefix.stride(0), n_prefix, lk.data_ptr(), lv.data_ptr(),
        lk.stride(0), lk.stride(1), cap, nk.data_ptr(), nv.data_ptr(), 0, 1000 + cap, 1000, out.data_ptr(), 0,
        ws.data_ptr(), ws_bytes, status.data_ptr(), hk, rep, d, 2, _native.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status) & 4
    assert float(lk.abs().sum()) == 0  # nothing appended outside the window


@pytest.mark.parametrize("dtype,d,hk,rep", [(torch.bfloat16, 128, 2, 4), (torch.float32, 64, 3, 2)])
def test_attention_sends_its_rows_to_the_gather_buffers(da, dtype, d, hk, rep):
    """da_decode_attention_push_next: the CTA that merges a head stores the head's output rows as
    {payload, tag} words into every rank's gather buffer (two local buffers stand in for two ranks,
    this launch is rank 1), and da_gather_heads with local = NULL only waits and copies: rank 1's rows
    of its output are the attention's output, rank 0's are what was put into the buffer by hand.  The
    setting is used up by one call."""
    from dram_attention_b200 import _native
    lib = _native.lib()
    g = _g(hk * 10 + rep)
    hq, n_prefix, cap, t0, dram_tokens = hk * rep, 700, 64, 9, 4096
    prefix = torch.randn(hk, n_prefix, 2, d, generator=g).to(dtype).to(DEV)
    local_k = torch.randn(cap, hk, d, generator=g).to(dtype).to(DEV)
    local_v = torch.randn(cap, hk, d, generator=g).to(dtype).to(DEV)
    q = torch.randn(1, hq, d, generator=g).to(dtype).to(DEV)
    nk = torch.randn(1, hk, d, generator=g).to(dtype).to(DEV)
    nv = torch.randn(1, hk, d, generator=g).to(dtype).to(DEV)
    ws_bytes = lib.da_decode_attention_tokens_workspace_bytes(hk, rep, d, 1)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    world, rank = 2, 1
    nbytes = hq * d * q.element_size()
    words = nbytes // 4
    total = lib.da_gather_heads_buffer_bytes(nbytes, world)
    bufs = [torch.zeros(total, dtype=torch.uint8, device=DEV) for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)     # for the gather kernel
    import ctypes
    host_ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])                # for the attention launch
    host_ptrs_p = ctypes.cast(host_ptrs, ctypes.c_void_p)
    seq = torch.full((1,), 4, dtype=torch.int32, device=DEV)      # step 4: slot 0, tag 5

    def attend(out):
        _native.check(lib.da_decode_attention_tokens(
            q.data_ptr(), 1, prefix.data_ptr(), prefix.stride(0), n_prefix, local_k.data_ptr(), local_v.data_ptr(),
            local_k.stride(0), local_k.stride(1), cap, nk.data_ptr(), nv.data_ptr(), 0, dram_tokens + t0, dram_tokens,
            out.data_ptr(), 0, ws.data_ptr(), ws_bytes, status.data_ptr(), hk, rep, d, _native.dtype_code(dtype),
            _native.stream_ptr()))

    out = torch.empty(1, hq, d, dtype=dtype, device=DEV)
    _native.check(lib.da_decode_attention_push_next(host_ptrs_p, seq.data_ptr(), rank, world, nbytes))
    attend(out)
    torch.cuda.synchronize()
    assert int(status) == 0
    for b in bufs:      # both "ranks" got rank 1's rows: slot 0, place 1, every word tagged 5
        wv = b.view(torch.int32).view(2, world, words, 2)
        assert bool((wv[0, rank, :, 1] == 5).all()) and bool((wv[0, 1 - rank] == 0).all()) and bool((wv[1] == 0).all())
        assert torch.equal(wv[0, rank, :, 0].contiguous().view(dtype).view(1, hq, d), out)
    # rank 0's rows by hand, then the gather that only waits and copies
    other = torch.randn(1, hq, d, generator=g).to(dtype).to(DEV)
    mine = bufs[rank].view(torch.int32).view(2, world, words, 2)
    mine[0, 0, :, 0] = other.view(torch.int32).view(-1)
    mine[0, 0, :, 1] = 5
    gathered = torch.zeros(world, hq, d, dtype=dtype, device=DEV)
    _native.check(lib.da_gather_heads(0, nbytes, ptrs.data_ptr(), seq.data_ptr(), rank, world, gathered.data_ptr(), 2000,
                                      status.data_ptr(), _native.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status) == 0 and int(seq) == 5
    assert torch.equal(gathered[1:2], out) and torch.equal(gathered[0:1], other)
    # the setting was used up: a second launch sends nothing
    for b in bufs:
        b.zero_()
    out2 = torch.empty_like(out)
    attend(out2)
    torch.cuda.synchronize()
    assert torch.equal(out2, out) and all(int(b.count_nonzero()) == 0 for b in bufs)
    # a size that does not match the call is refused (and uses the setting up)
    _native.check(lib.da_decode_attention_push_next(host_ptrs_p, seq.data_ptr(), rank, world, nbytes + 16))
    rc = lib.da_decode_attention_tokens(
        q.data_ptr(), 1, prefix.data_ptr(), prefix.stride(0), n_prefix, local_k.data_ptr(), local_v.data_ptr(),
        local_k.stride(0), local_k.stride(1), cap, nk.data_ptr(), nv.data_ptr(), 0, dram_tokens + t0, dram_tokens,
        out2.data_ptr(), 0, ws.data_ptr(), ws_bytes, status.data_ptr(), hk, rep, d, _native.dtype_code(dtype),
        _native.stream_ptr())
    assert rc == -2
    assert lib.da_decode_attention_push_next(host_ptrs_p, seq.data_ptr(), 2, world, nbytes) == -2


# -------------------------------------------------------------------- rope ----

@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_rope_kernel_matches_reference_caller(da, golden_dir, name):
    """da_rope_qk against the outputs of the reference caller's apply_rotary_emb (fixture made by
    running it), bit for bit, out of place and in place."""
    from dram_attention_b200 import _native
    from tests.test_oracle_golden import _rope_case, _load
    xq, xk, freqs, want_q, want_k = _rope_case(_load(golden_dir, "rope_values.npz"), name)
    lib = _native.lib()
    q, k = xq.to(DEV).contiguous(), xk.to(DEV).contiguous()
    f = torch.view_as_real(freqs).contiguous().to(DEV)
    oq, ok = torch.zeros_like(q), torch.zeros_like(k)
    s, hq, hk, d = q.shape[1], q.shape[2], k.shape[2], q.shape[3]
    code = _native.dtype_code(q.dtype)
    _native.check(lib.da_rope_qk(q.data_ptr(), k.data_ptr(), f.data_ptr(), oq.data_ptr(), ok.data_ptr(), s, hq, hk, d,
                                 code, _native.stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(oq.cpu(), want_q) and torch.equal(ok.cpu(), want_k)
    _native.check(lib.da_rope_qk(q.data_ptr(), k.data_ptr(), f.data_ptr(), q.data_ptr(), k.data_ptr(), s, hq, hk, d,
                                 code, _native.stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(q.cpu(), want_q) and torch.equal(k.cpu(), want_k)
    # the oracle's statement at a shape of its own (odd head counts, 1 token, fp16)
    g = _g(5)
    xq2, xk2 = torch.randn(1, 1, 3, 64, generator=g).half(), torch.randn(1, 1, 1, 64, generator=g).half()
    ang = torch.rand(1, 32, generator=g) * 6.0
    fr = torch.polar(torch.ones_like(ang), ang)
    wq, wk = orc.rope_qk(xq2, xk2, fr)
    q2, k2 = xq2.to(DEV), xk2.to(DEV)
    f2 = torch.view_as_real(fr).contiguous().to(DEV)
    _native.check(lib.da_rope_qk(q2.data_ptr(), k2.data_ptr(), f2.data_ptr(), q2.data_ptr(), k2.data_ptr(), 1, 3, 1, 64,
                                 _native.dtype_code(torch.float16), _native.stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(q2.cpu(), wq) and torch.equal(k2.cpu(), wk)
    assert lib.da_rope_qk(q2.data_ptr(), k2.data_ptr(), f2.data_ptr(), q2.data_ptr(), k2.data_ptr(), 1, 3, 1, 63,
                          _native.dtype_code(torch.float16), _native.stream_ptr()) == -2


# ------------------------------------------------------------------ gather ----

def test_gather_wait_runs_out_and_is_reported(da):
    """The all-gather kernel of the KV-head sharding with a peer that never shows up (rank 0 of 2
    on one GPU, nothing writes rank 1's words): the kernel returns after its time budget, reports
    DA_STATUS_WAIT_TIMEOUT, marks the missing rank's rows with NaN, and the context stays usable;
    when the peer's words are there (written by hand, as its stores would) the next call
    succeeds."""
    from dram_attention_b200 import _native
    lib = _native.lib()
    world, nbytes = 2, 4 * 128 * 2
    words = nbytes // 4
    total = lib.da_gather_heads_buffer_bytes(nbytes, world)
    assert total == 2 * world * 2 * nbytes
    bufs = [torch.zeros(total, dtype=torch.uint8, device=DEV) for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    g = _g(11)
    local = torch.randn(4, 128, generator=g).bfloat16().to(DEV)
    out = torch.zeros(world * 4, 128, dtype=torch.bfloat16, device=DEV)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _native.check(lib.da_gather_heads(local.data_ptr(), nbytes, ptrs.data_ptr(), seq.data_ptr(), 0, world,
                                      out.data_ptr(), 2000, status.data_ptr(), _native.stream_ptr()))
    t1.record()
    torch.cuda.synchronize()
    assert int(status) == _native.STATUS_WAIT_TIMEOUT
    assert 1.5 <= t0.elapsed_time(t1) <= 50.0          # about the 2 ms it was given
    assert torch.equal(out[:4], local)
    assert bool(torch.isnan(out[4:].float()).all())     # nobody can take these rows for a result
    assert int(seq) == 1
    # rank 0's own rows went into both buffers as {payload, tag 1} words of slot 0, rank 0's place
    sent = bufs[1].view(torch.int32).view(2, world, words, 2)
    assert bool((sent[0, 0, :, 1] == 1).all()) and bool((sent[0, 1] == 0).all()) and bool((sent[1] == 0).all())
    assert torch.equal(sent[0, 0, :, 0].contiguous().view(torch.bfloat16).view(4, 128), local)
    # the peer shows up for the next step (seq 1 -> slot 1, tag 2)
    status.zero_()
    peer_rows = torch.randn(4, 128, generator=g).bfloat16().to(DEV)
    mine = bufs[0].view(torch.int32).view(2, world, words, 2)
    mine[1, 1, :, 0] = peer_rows.view(torch.int32).view(-1)
    mine[1, 1, :, 1] = 2
    local2 = torch.randn(4, 128, generator=g).bfloat16().to(DEV)
    _native.check(lib.da_gather_heads(local2.data_ptr(), nbytes, ptrs.data_ptr(), seq.data_ptr(), 0, world,
                                      out.data_ptr(), 2000, status.data_ptr(), _native.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status) == 0 and int(seq) == 2
    assert torch.equal(out[:4], local2) and torch.equal(out[4:], peer_rows)
    # bad arguments are refused on the host
    assert lib.da_gather_heads(local.data_ptr(), nbytes, ptrs.data_ptr(), seq.data_ptr(), 2, world, out.data_ptr(),
                               0, status.data_ptr(), _native.stream_ptr()) == -2
    assert lib.da_gather_heads(local.data_ptr(), 24, ptrs.data_ptr(), seq.data_ptr(), 0, world, out.data_ptr(),
                               0, status.data_ptr(), _native.stream_ptr()) == -2

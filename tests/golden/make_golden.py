"""Generate the golden fixtures in this directory by running the reference's
own code on the CPU (see oracle/ref_harness.py for how).  Run from the
repository root, in a container that has the reference tree:

    python tests/golden/make_golden.py

Outputs (all small .npz files, committed):
  scorer_values.npz   inputs and outputs of the reference's scorer, both its
                      torch statement and its Triton kernel run in the
                      interpreter, at the shape of its own value test.
  lru_kernel_cases.npz  random LRU tables stepped through the reference's own
                      LRU kernels (duplicates in the list, several steps).
  plumbing_traj.npz   16 generate steps of the reference's DRAMAttention on
                      the float32 plumbing workload: per-step outputs, page
                      lists and table snapshots; inputs are regenerated from
                      the seed and guarded by a checksum.
  mini_traj.npz       a smaller trajectory whose inputs are multiples of 1/8
                      stored as int8 (many exact score ties), inputs included.
  multi_traj_*.npz    generate calls with several tokens each (2, 3, 1, 4, 2 tokens) on the
                      same kind of inputs: outputs of every token, page lists, tables.  Two
                      head layouts, the ones the reference's selector accepts with more than
                      one token (its `view` after `swapaxes`, topk_selector.py:52-55, needs
                      one KV head or a GQA group of one; anything else raises there).
  rope_values.npz     the rotary embedding of the reference's caller
                      (evaluation/dram-attention/model.py: precompute_freqs_cis, apply_rotary_emb)
                      on float32 and bfloat16 queries and keys at scattered positions.
"""

from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
os.environ["TRITON_INTERPRET"] = "1"

import torch  # noqa: E402

from oracle.ref_harness import reference_on_cpu  # noqa: E402
from dram_attention_b200.synthetic import plumbing_workload  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def checksum(*tensors) -> np.ndarray:
    """Order-sensitive 64-bit checksum of the raw bytes of the tensors."""
    acc = np.uint64(1469598103934665603)
    for t in tensors:
        b = np.frombuffer(t.contiguous().view(torch.uint8).numpy().tobytes(), dtype=np.uint8)
        pad = (-b.size) % 8
        w = np.frombuffer(np.concatenate([b, np.zeros(pad, np.uint8)]).tobytes(), dtype=np.uint64)
        idx = np.arange(1, w.size + 1, dtype=np.uint64)
        with np.errstate(over="ignore"):
            acc = acc * np.uint64(1099511628211) + np.bitwise_xor.reduce(w * (idx * np.uint64(2) + np.uint64(1)))
    return np.array([acc], dtype=np.uint64)


def scorer_values(ref):
    from dram_attention.max_ip_triton_kernel import _max_inner_product_kernel, max_ip_ref
    g = torch.Generator().manual_seed(0)
    n, h, d, l = 2, 4, 64, 16
    q = torch.randn(n, h, d, generator=g)
    mm = torch.randn(h, l, 2, d, generator=g)
    out_ref = max_ip_ref(q, mm)
    out_tri = torch.empty(n, h, l)
    grid = ((l + 1) // 2, (n + 1) // 2, (h + 1) // 2)
    _max_inner_product_kernel.fn[grid](
        q, q.stride(0), q.stride(1), mm, mm.stride(0), mm.stride(1), mm.stride(2),
        out_tri, out_tri.stride(0), out_tri.stride(1), L=l, N=n, H=h, D=d,
        BLOCK_SIZE_L=2, BLOCK_SIZE_N=2, BLOCK_SIZE_H=2)
    print("scorer: torch statement vs interpreter kernel max abs diff",
          float((out_ref - out_tri).abs().max()))
    np.savez(os.path.join(HERE, "scorer_values.npz"), q=q.numpy(), min_max=mm.numpy(),
             out_ref=out_ref.numpy(), out_triton=out_tri.numpy())


def lru_kernel_cases(ref):
    from dram_attention.lru_triton_kernel import load_lru_cache_
    rng = np.random.default_rng(0)
    cases = {}
    n_cases = 12
    for c in range(n_cases):
        hk = int(rng.integers(1, 4))
        ld = int(rng.integers(16, 80))
        nh = int(rng.integers(6, min(ld, 24)))
        kk = int(rng.integers(1, nh + 1))          # list length <= slots
        page_dim = 8
        steps = 5
        dram = torch.from_numpy(rng.standard_normal((hk, ld, page_dim)).astype(np.float32))
        hbm = dram[:, ld - nh:].clone()
        times = torch.zeros(hk, nh, dtype=torch.int32)
        d2h = torch.full((hk, ld), -1, dtype=torch.int32)
        d2h[:, ld - nh:] = torch.arange(nh, dtype=torch.int32)[None]
        h2d = torch.arange(ld - nh, ld, dtype=torch.int32)[None].repeat(hk, 1).contiguous()
        step = torch.zeros(1, dtype=torch.int32)
        lists, snaps = [], []
        for s in range(steps):
            # draws with replacement from a small pool -> duplicates and re-hits
            pool = rng.choice(ld, size=min(ld, max(2, kk)), replace=False)
            lst = torch.from_numpy(rng.choice(pool, size=(hk, kk)).astype(np.int32))
            step.add_(1)
            load_lru_cache_(dram_kv_cache=dram, page_access_time=times,
                            dram_page_to_hbm_page_mapping=d2h,
                            hbm_page_to_dram_page_mapping=h2d,
                            topk_dram_page_index=lst, current_step=step, hbm_kv_cache=hbm)
            lists.append(lst.numpy().copy())
            snaps.append((d2h.numpy().copy(), h2d.numpy().copy(), times.numpy().copy(),
                          hbm.numpy().copy()))
        cases[f"c{c}_dram"] = dram.numpy()
        cases[f"c{c}_lists"] = np.stack(lists)
        cases[f"c{c}_d2h"] = np.stack([s[0] for s in snaps])
        cases[f"c{c}_h2d"] = np.stack([s[1] for s in snaps])
        cases[f"c{c}_time"] = np.stack([s[2] for s in snaps])
        cases[f"c{c}_hbm"] = np.stack([s[3] for s in snaps])
    cases["n_cases"] = np.array([n_cases])
    np.savez_compressed(os.path.join(HERE, "lru_kernel_cases.npz"), **cases)
    print("lru kernel cases:", n_cases)


def run_trajectory(ref, ctor, k, v, xq, xk, xv, dtype):
    """Prefill-free trajectory: init_cache on the given KV, then generate."""
    m = ref.DRAMAttention(device="cpu", dtype=dtype, **ctor)
    m.init_cache(k, v)
    s = k.shape[1]
    outs, lists, h2ds, d2hs, times = [], [], [], [], []
    lc = m.lru_cache
    orig_load = lc.load_

    def spy(idx):
        lists.append(idx.numpy().copy())
        return orig_load(idx)

    lc.load_ = spy
    for i in range(xq.shape[0]):
        out = m(xq[i], xk[i], xv[i], start_pos=s + i, stage="generate")
        outs.append(out[0, 0].float().numpy().copy())
        h2ds.append(lc.hbm_page_to_dram_page_mapping.numpy().copy())
        d2hs.append(lc.dram_page_to_hbm_page_mapping.numpy().copy())
        times.append(lc.page_access_time.numpy().copy())
    return dict(out=np.stack(outs), lists=np.stack(lists), h2d=np.stack(h2ds),
                d2h_final=d2hs[-1], time=np.stack(times),
                dram_tokens=np.array([m.dram_kv_cache_size]),
                step=np.array([int(lc.current_step)]))


def plumbing_traj(ref):
    w = plumbing_workload(seed=0, steps=16)
    res = run_trajectory(ref, w.ctor_kwargs(), w.k, w.v, w.xq, w.xk, w.xv, torch.float32)
    res["input_checksum"] = checksum(w.k, w.v, w.xq, w.xk, w.xv)
    np.savez_compressed(os.path.join(HERE, "plumbing_traj.npz"), **res)
    print("plumbing trajectory: out", res["out"].shape, "lists", res["lists"].shape)


def mini_traj(ref):
    g = torch.Generator().manual_seed(1)
    hq, hk, d, p = 4, 2, 64, 16
    local, lru, top_k, max_out, steps = 64, 256, 64, 8, 8
    s = 640 + local - p
    k8 = torch.randint(-16, 17, (1, s, hk, d), generator=g, dtype=torch.int8)
    v8 = torch.randint(-16, 17, (1, s, hk, d), generator=g, dtype=torch.int8)
    q8 = torch.randint(-8, 9, (steps, 1, 1, hq, d), generator=g, dtype=torch.int8)
    xk8 = torch.randint(-16, 17, (steps, 1, 1, hk, d), generator=g, dtype=torch.int8)
    xv8 = torch.randint(-16, 17, (steps, 1, 1, hk, d), generator=g, dtype=torch.int8)
    f = lambda t: t.float() / 8.0
    ctor = dict(max_output_length=max_out, lru_hbm_cache_size=lru, local_cache_size=local,
                page_size=p, top_k=top_k, n_kv_heads=hk, head_dim=d)
    res = run_trajectory(ref, ctor, f(k8), f(v8), f(q8), f(xk8), f(xv8), torch.float32)
    res.update(k8=k8.numpy(), v8=v8.numpy(), q8=q8.numpy(), xk8=xk8.numpy(), xv8=xv8.numpy(),
               ctor=np.array([max_out, lru, local, p, top_k, hk, d]))
    np.savez_compressed(os.path.join(HERE, "mini_traj.npz"), **res)
    print("mini trajectory: out", res["out"].shape)


def multi_traj(ref, hq, hk):
    """Generate calls that carry several tokens each (the reference's generate stage takes
    seq_len > 1: dram_attention/topk_selector.py:48-61, lru_cache.py:260-264,
    dram_attention.py:191-223)."""
    g = torch.Generator().manual_seed(2 + hq)
    d, p = 64, 16
    local, lru, top_k, max_out = 64, 384, 64, 16
    counts = [2, 3, 1, 4, 2]
    s = 640 + local - p
    k8 = torch.randint(-16, 17, (1, s, hk, d), generator=g, dtype=torch.int8)
    v8 = torch.randint(-16, 17, (1, s, hk, d), generator=g, dtype=torch.int8)
    n_tok = sum(counts)
    q8 = torch.randint(-8, 9, (1, n_tok, hq, d), generator=g, dtype=torch.int8)
    xk8 = torch.randint(-16, 17, (1, n_tok, hk, d), generator=g, dtype=torch.int8)
    xv8 = torch.randint(-16, 17, (1, n_tok, hk, d), generator=g, dtype=torch.int8)
    f = lambda t: t.float() / 8.0
    ctor = dict(max_output_length=max_out, lru_hbm_cache_size=lru, local_cache_size=local,
                page_size=p, top_k=top_k, n_kv_heads=hk, head_dim=d)
    m = ref.DRAMAttention(device="cpu", dtype=torch.float32, **ctor)
    m.init_cache(f(k8), f(v8))
    lc = m.lru_cache
    lists = []
    orig_load = lc.load_

    def spy(idx):
        lists.append(idx.numpy().copy())
        return orig_load(idx)

    lc.load_ = spy
    outs, h2ds, times = [], [], []
    pos, a = s, 0
    for c in counts:
        out = m(f(q8[:, a:a + c]), f(xk8[:, a:a + c]), f(xv8[:, a:a + c]), start_pos=pos, stage="generate")
        outs.append(out[0].float().numpy().copy())            # (c, Hq, D)
        h2ds.append(lc.hbm_page_to_dram_page_mapping.numpy().copy())
        times.append(lc.page_access_time.numpy().copy())
        pos += c
        a += c
    res = dict(out=np.concatenate(outs), h2d=np.stack(h2ds), time=np.stack(times),
               d2h_final=lc.dram_page_to_hbm_page_mapping.numpy().copy(),
               cache_k=m.cache_k[0].numpy().copy(), counts=np.array(counts),
               k8=k8.numpy(), v8=v8.numpy(), q8=q8.numpy(), xk8=xk8.numpy(), xv8=xv8.numpy(),
               ctor=np.array([max_out, lru, local, p, top_k, hk, d]),
               dram_tokens=np.array([m.dram_kv_cache_size]))
    for i, l in enumerate(lists):
        res[f"list{i}"] = l
    res["heads"] = np.array([hq, hk])
    np.savez_compressed(os.path.join(HERE, f"multi_traj_hq{hq}_hk{hk}.npz"), **res)
    print("multi-token trajectory: out", res["out"].shape, "lists", [l.shape for l in lists])


def rope_values(ref):
    """apply_rotary_emb of the reference's model file, float32 and bfloat16."""
    import importlib.util
    from oracle.ref_harness import REFERENCE_ROOT
    spec = importlib.util.spec_from_file_location(
        "ref_caller_model", os.path.join(REFERENCE_ROOT, "evaluation", "dram-attention", "model.py"))
    model = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(model)
    g = torch.Generator().manual_seed(7)
    hq, hk, d, s = 8, 2, 128, 5
    freqs_all = model.precompute_freqs_cis(d, 200000, 500000.0)
    pos = torch.tensor([0, 1, 4097, 131071, 199999])
    freqs = freqs_all[pos]
    res = dict(pos=pos.numpy(), freqs=torch.view_as_real(freqs).numpy())
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        xq = torch.randn(1, s, hq, d, generator=g).to(dt)
        xk = (torch.randn(1, s, hk, d, generator=g) * 3).to(dt)
        oq, ok = model.apply_rotary_emb(xq, xk, freqs_cis=freqs)
        assert oq.dtype == dt and ok.dtype == dt
        as_np = (lambda t: t.numpy()) if dt == torch.float32 else (lambda t: t.view(torch.int16).numpy())
        res.update({f"xq_{name}": as_np(xq), f"xk_{name}": as_np(xk), f"oq_{name}": as_np(oq), f"ok_{name}": as_np(ok)})
    np.savez_compressed(os.path.join(HERE, "rope_values.npz"), **res)
    print("rope values:", {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    with reference_on_cpu() as ref:
        if "--only-rope" in sys.argv:
            rope_values(ref)
            sys.exit(0)
        if "--only-multi" in sys.argv:
            multi_traj(ref, 4, 1)
            multi_traj(ref, 2, 2)
            sys.exit(0)
        scorer_values(ref)
        lru_kernel_cases(ref)
        mini_traj(ref)
        plumbing_traj(ref)
        multi_traj(ref, 4, 1)
        multi_traj(ref, 2, 2)
        rope_values(ref)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")

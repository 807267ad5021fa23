#!/usr/bin/env python
"""Benchmark of the generate stage on the Llama-3-8B-shaped 128K-context decode layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" = one generate step (one new token) of one attention layer: page
scoring, top-k selection, LRU update, miss fetch, decode attention.  Prints one
JSON line.

Set-up (untimed): cache construction, then --settle-steps decode steps, so that the slot
table holds what the query stream uses (steady-state decode), then W warm-up steps.

value   decode tok/s with every input resident in HBM: the K timed steps are
        captured, with their own device-resident inputs, in one CUDA graph, the
        graph is uploaded, and one replay is timed with CUDA events (max over ranks).
e2e     the same metric through the operator API with HOST inputs: per step the
        query/key/value are written into a pinned staging buffer, one captured graph
        (host->device copy, the step, device->host copy of the output) is replayed
        and the stream is synchronised.
roofline  attention kernel (the dominant launch): algorithmic bytes / its launch
        time, measured as the difference of two replayed graphs (L2 eviction +
        kernel, eviction alone); peak = the measured HBM copy bandwidth of this pool.
fetch_report, scorer_sweep, prefill  the miss fetch (exposed share of a step, a cold
        step against the host link), scorer/top-k over 512..65536 pages, and the
        prefill kernel's TFLOP/s; extras, not part of the metric.
cpu_baseline  the CPU oracle (a port of the reference's pure-PyTorch path) timed on
        a bounded sample of the same workload on this box's host cores.

With --gpus N > 1 (launched by torchrun, one rank per GPU) every GPU decodes a sequence
of its own (same layer shape, its own seed): no collective on the path, weak scaling,
value = N sequences' tokens / max-over-ranks time.  The same run also times ONE sequence
with its KV heads sharded over the ranks ("kv_head_sharded"; per-head outputs all-gathered
by a peer-memory kernel over NVLink, or by the process group's all-gather where symmetric
memory is not available); --shard kv-heads makes that the headline instead (strong
scaling).  --impl reference times the CPU port of the reference path on rank 0 only.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode tok/s at 128K ctx (Llama-3-8B attn shape)"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch at the default workload, from the ncu
# capture summarised in profiles/decode_attention_mma_llama128k.md
ATTN_TRAFFIC_BYTES_128K = 154.4e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--dram-tokens", type=int, default=131072, help="prefix tokens kept in DRAM")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", default="sequence", choices=["sequence", "kv-heads"],
                    help="N > 1: one independent sequence per GPU, no collective (weak scaling, default; the "
                         "KV-head-sharded step is timed as well and reported beside it), or only the KV heads "
                         "of ONE sequence sharded over the GPUs (strong scaling)")
    ap.add_argument("--library-gather", action="store_true",
                    help="N > 1: all-gather through the process group instead of the peer-memory kernel")
    ap.add_argument("--prefill-tokens", type=int, default=32768, help="prompt length of the prefill report")
    ap.add_argument("--only-prefill", action="store_true",
                    help="time just the prefill kernel at --prefill-tokens (a small launch to profile) and exit")
    ap.add_argument("--settle-steps", type=int, default=192,
                    help="untimed decode steps before the warm-up, so that the slot table holds what the query "
                         "stream uses rather than the warm start of the cache construction (steady-state decode)")
    ap.add_argument("--clock-period-ms", type=float, default=2.0,
                    help="NVML polling period while the GPU works alone; the end-to-end loop is polled 10x slower")
    ap.add_argument("--no-sweep", action="store_true", help="skip the scorer / top-k sweep over page counts")
    ap.add_argument("--profile-steps", type=int, default=16, help="un-captured steps timed stage by stage")
    return ap.parse_args()


def workload_config(args, w):
    return {
        "workload": w.name,
        "batch": 1, "n_q_heads": w.n_q_heads, "n_kv_heads": w.n_kv_heads, "head_dim": w.head_dim,
        "dram_prefix_tokens": w.dram_tokens, "page_size": w.page_size,
        "lru_hbm_cache_size": w.lru_hbm_cache_size, "local_cache_size": w.local_cache_size,
        "top_k": w.top_k, "prefill_len": w.prefill_len,
        "l2": "inputs larger than L2 (185 MB touched per step vs 126 MB)",
    }


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) in a thread."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples = []  # (t, sm_mhz, reasons)
        self.period = period_s
        self.stop_flag = False
        self.thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report that, do not fail the bench
            self.nv = None
            self.err = repr(e)

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def sample_now(self):
        """One sample taken by the caller's thread (brackets a region the poller is kept slow in)."""
        if self.nv is None:
            return
        nv = self.nv
        try:
            mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
            try:
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            self.samples.append((time.perf_counter(), mhz, reasons))
        except Exception:
            pass

    def start(self):
        if self.nv is not None and self.period > 0:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join()

    def summary(self, windows):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + self.err]}
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in windows)]
        use = inside if inside else self.samples
        names = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}
        bits = 0
        for s in use:
            bits |= s[2]
        return {"sm_mhz": statistics.median(s[1] for s in use) if use else None,
                "sm_max_mhz": self.max_mhz,
                "reasons": [n for b, n in names.items() if bits & b],
                "samples_in_timed_regions": len(inside), "samples": len(self.samples)}


def upload_graph(graph, torch):
    """Places the instantiated graph on the device before it is timed (otherwise its first
    launch pays a one-time set-up of several microseconds per captured step).  Returns False
    when the handle or the binding is not available; the caller then parks the GPU behind a
    spin while the host launches instead."""
    try:
        from cuda.bindings import runtime as rt
        exec_handle = rt.cudaGraphExec_t(int(graph.raw_cuda_graph_exec()))
        (err,) = rt.cudaGraphUpload(exec_handle, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return int(err) == 0
    except Exception:
        return False


def tensor_peak_tflops():
    """Measured dense bf16 throughput of this pool's GPUs (burst figure: the kernel is timed alone)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def hbm_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------------
# CPU port of the reference path (oracle) -- cpu_baseline leg and --impl reference
# --------------------------------------------------------------------------------

def cpu_reference_steps(w, n_warm, n_timed, budget_s=None):
    """Steps of the CPU oracle on workload w; returns (tok/s, steps timed, threads)."""
    import torch
    from oracle import dram_attention_oracle as orc
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    o = orc.OracleDRAMAttention(dtype=torch.float32, **w.ctor_kwargs())
    o.init_cache(w.k.float(), w.v.float())
    s = w.k.shape[1]
    for i in range(n_warm):
        o.generate(w.xq[i].float(), w.xk[i].float(), w.xv[i].float(), s + i)
    t0 = time.perf_counter()
    done = 0
    for i in range(n_warm, n_warm + n_timed):
        o.generate(w.xq[i].float(), w.xk[i].float(), w.xv[i].float(), s + i)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s and done >= 2:
            break
    dt = time.perf_counter() - t0
    return done / dt, done, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from dram_attention_b200.synthetic import llama_layer_workload
    k, wu = args.steps, args.warmup
    w = llama_layer_workload(seed=0, steps=k + wu, dram_tokens=args.dram_tokens, max_out=k + wu)
    tps, done, threads = cpu_reference_steps(w, wu, k)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": done, "warmup": wu, "ms_per_step": 1e3 / tps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, w),
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{done} full generate steps of the same layer after {wu} warm-up steps, "
                                   "CPU port of the reference's pure-PyTorch path (fp32 scores, fp64 attention)"},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=RESULT_OUT, flush=True)


# --------------------------------------------------------------------------------
# B200 arm
# --------------------------------------------------------------------------------

def run_b200(args):
    import torch
    import torch.distributed as dist
    import dram_attention_b200 as da
    from dram_attention_b200.sharded import KVHeadShardedDRAMAttention, head_range
    from dram_attention_b200.synthetic import llama_layer_workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # stdout carries the JSON line only
        dist.init_process_group("nccl", device_id=dev)

    if args.only_prefill:
        # one small job for a profiler: three launches of the prefill kernel, checked for finiteness
        op = da.DRAMAttention(max_output_length=8, lru_hbm_cache_size=2048, local_cache_size=512, page_size=16,
                              top_k=512, n_kv_heads=8, head_dim=128, device=dev, dtype=torch.bfloat16)
        g = torch.Generator(device=dev).manual_seed(2)
        s_pf = args.prefill_tokens
        q, k, v = (torch.randn(1, s_pf, h, 128, generator=g, device=dev).to(torch.bfloat16) for h in (32, 8, 8))
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        out = op._prefill_attention(q, k, v)
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(2):
            out = op._prefill_attention(q, k, v)
        ev1.record()
        torch.cuda.synchronize()
        op.check_status()
        ms = ev0.elapsed_time(ev1) / 2
        print(json.dumps({"prefill_tokens": s_pf, "ms": ms, "tflops": 4.0 * s_pf * s_pf / 2 * 32 * 128 / ms / 1e9,
                          "finite": bool(torch.isfinite(out.float()).all())}), file=RESULT_OUT, flush=True)
        return
    K, W = args.steps, max(args.warmup, 3)
    P = max(0, args.profile_steps)
    settle = max(0, args.settle_steps)
    total = settle + (W + K) * 2 + 2 * P + K + 4
    # N > 1, default: every GPU decodes its own sequence (same shapes, its own seed); no collective
    by_seq = world > 1 and args.shard == "sequence"
    n_seq = world if by_seq else 1
    w = llama_layer_workload(seed=(rank if by_seq else 0), steps=total, dram_tokens=args.dram_tokens, max_out=total)
    hk_all, rep, D = w.n_kv_heads, w.n_q_heads // w.n_kv_heads, w.head_dim
    lo, hi = (0, hk_all) if by_seq else head_range(hk_all, rank, world)
    hk = hi - lo
    esz = 2

    ctor = w.ctor_kwargs()
    ctor.pop("n_kv_heads")
    if world == 1 or by_seq:
        op = da.DRAMAttention(n_kv_heads=hk_all, device=dev, dtype=w.dtype, **ctor)
        inner = op
    else:
        op = KVHeadShardedDRAMAttention(n_kv_heads=hk_all, presliced=True, device=dev, dtype=w.dtype,
                                        peer_gather=not args.library_gather, **ctor)
        inner = op.inner
    inner.init_cache(w.k[:, :, lo:hi].to(dev), w.v[:, :, lo:hi].to(dev))
    lc = inner.lru_cache
    S = w.prefill_len

    # this rank's slice of every step's inputs: pinned host copies and device copies
    hq = w.xq[:, :, :, lo * rep:hi * rep].contiguous().pin_memory()
    hkk = w.xk[:, :, :, lo:hi].contiguous().pin_memory()
    hv = w.xv[:, :, :, lo:hi].contiguous().pin_memory()
    dq, dk, dv = hq.to(dev), hkk.to(dev), hv.to(dev)

    sampler = ClockSampler(local_rank, period_s=args.clock_period_ms * 1e-3)
    sampler.start()
    windows = []

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---------------- value: K captured steps, inputs resident in HBM -----------------
    step = 0
    for _ in range(settle + W):     # the settle steps are part of the set-up, the last W are the warm-up
        op(dq[step], dk[step], dv[step], start_pos=S + step, stage="generate")
        step += 1
    torch.cuda.synchronize()
    # every call returns a tensor of its own (inside a capture: of the graph's memory pool), so the K
    # outputs are kept by reference and no copy kernel sits between two steps
    outs = []
    graph = torch.cuda.CUDAGraph()
    captured = True
    first = step
    try:
        with torch.cuda.graph(graph):
            for i in range(K):
                outs.append(op(dq[first + i], dk[first + i], dv[first + i], start_pos=S + first + i,
                               stage="generate"))
    except Exception as e:  # e.g. a collective that cannot be captured: time eager launches instead
        captured = False
        capture_error = repr(e)
        torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The graph can be timed only once (a second replay of the same steps finds its pages resident),
    # so its one-time device set-up is done before the timed region.
    uploaded = captured and upload_graph(graph, torch)
    barrier()
    t_a = time.perf_counter()
    if captured and not uploaded:
        torch.cuda._sleep(20_000_000)
    ev0.record()
    if captured:
        graph.replay()
    else:
        outs = [op(dq[first + i], dk[first + i], dv[first + i], start_pos=S + first + i, stage="generate")
                for i in range(K)]
    ev1.record()
    barrier()
    windows.append((t_a, time.perf_counter()))
    step += K
    ms_value = ev0.elapsed_time(ev1)
    assert len(outs) == K and all(bool(torch.isfinite(o.float()).all()) for o in outs), "a timed step left no output"

    # ---------------- e2e: host inputs, one captured step per call ----------------------
    # q, k and v of a step sit back to back in one pinned buffer and cross the link in one copy
    nq, nk = dq[0].numel(), dk[0].numel()
    h_in = torch.cat([hq.reshape(total, -1), hkk.reshape(total, -1), hv.reshape(total, -1)], dim=1).pin_memory()
    d_in = torch.empty(nq + 2 * nk, dtype=w.dtype, device=dev)
    xq_s = d_in[:nq].view(dq[0].shape)
    xk_s = d_in[nq:nq + nk].view(dk[0].shape)
    xv_s = d_in[nq + nk:].view(dv[0].shape)
    out_h = torch.empty(1, 1, w.n_q_heads, D, dtype=w.dtype).pin_memory()
    pos = torch.tensor([S + step], dtype=torch.int32, device=dev)
    # The captured step includes the two copies across the host link: q|k|v from a fixed pinned
    # staging buffer, the output into a fixed pinned buffer.  Per step the host writes the next
    # inputs into the staging buffer, replays, and synchronises.
    h_stage = torch.empty_like(h_in[0]).pin_memory()
    step_graph = torch.cuda.CUDAGraph()
    step_captured = True
    try:
        with torch.cuda.graph(step_graph):
            d_in.copy_(h_stage, non_blocking=True)
            out_h.copy_(op(xq_s, xk_s, xv_s, start_pos=pos, stage="generate"), non_blocking=True)
            pos.add_(1)
    except Exception:
        step_captured = False
        torch.cuda.synchronize()

    h_rows = list(h_in.unbind(0))          # one view per step, made once
    cur_stream = torch.cuda.current_stream()

    def e2e_step(i):
        if step_captured:
            h_stage.copy_(h_rows[i])        # host-side, 12 KiB
            step_graph.replay()
        else:
            d_in.copy_(h_rows[i], non_blocking=True)
            out_h.copy_(op(xq_s, xk_s, xv_s, start_pos=pos, stage="generate"), non_blocking=True)
            pos.add_(1)
        cur_stream.synchronize()

    # NVML queries take driver locks that the launch path also wants: polled every 2 ms they cost
    # this host-bound loop ~20 us per step.  So the poller is slowed tenfold here and the region is
    # bracketed by one sample on each side, taken outside the events.
    fast_period = sampler.period
    sampler.period = 10 * fast_period
    for _ in range(W):
        e2e_step(step)
        step += 1
    barrier()
    t_a = time.perf_counter()
    sampler.sample_now()
    ev0.record()
    for _ in range(K):
        e2e_step(step)
        step += 1
    ev1.record()
    barrier()
    sampler.sample_now()
    windows.append((t_a, time.perf_counter()))
    sampler.period = fast_period
    ms_e2e = ev0.elapsed_time(ev1)

    # ---------------- per-stage timing of un-captured steps (roofline) -------------------
    fused = bool(getattr(inner, "_can_fuse", False) and inner.fused_fetch)
    stage_names = ["score", "topk", "lru", "fetch", "attention"]
    stage_ms = {n: [] for n in stage_names}
    misses = []
    k_pages = w.top_k // w.page_size
    list_len = rep * k_pages
    out_p = torch.empty(1, 1, hk * rep, D, dtype=w.dtype, device=dev)
    miss_dev = torch.zeros(max(P, 1), dtype=torch.int32, device=dev)
    events = []
    t_a = time.perf_counter()
    # Park the GPU behind a ~50 ms spin so that every launch and event of the P steps is
    # already queued when it starts: the event intervals then hold kernel time, not the
    # host's launch latency (a stage takes longer to launch from Python than to run).
    torch.cuda.synchronize()
    if P:
        torch.cuda._sleep(100_000_000)
    for i in range(P):
        q, kk, vv = dq[step], dk[step], dv[step]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        ev[0].record()
        lc.top_k_selector.score_(q, k_pages)
        ev[1].record()
        page_list = lc.top_k_selector.select_(1, rep, k_pages)
        ev[2].record()
        lc.update_tables_(page_list)
        ev[3].record()
        if not fused:
            lc.fetch_(list_len)
        ev[4].record()
        inner.attend_(q, kk, vv, S + step, out_p, fetch=fused)
        ev[5].record()
        miss_dev[i].copy_(lc.last_miss_counts(list_len).sum())
        events.append(ev)
        step += 1
    torch.cuda.synchronize()
    for ev in events:
        for j, n in enumerate(stage_names):
            stage_ms[n].append(ev[j].elapsed_time(ev[j + 1]))
    misses = miss_dev[:P].tolist()
    windows.append((t_a, time.perf_counter()))

    # ---------------- timeline of the overlapped step (two streams), same parking trick ----------
    overlapped = bool(fused and inner.overlap and getattr(inner, "_can_overlap", False)
                      and inner._overlap_supported(rep, w.dtype))
    timeline = None
    if overlapped and P:
        side = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream()
        recs = []
        torch.cuda.synchronize()
        torch.cuda._sleep(100_000_000)
        for i in range(P):
            q, kk, vv = dq[step], dk[step], dv[step]
            e = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
            a = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            e[0].record(main)
            lc.top_k_selector.score_(q, k_pages)
            e[1].record(main)
            page_list = lc.top_k_selector.select_(1, rep, k_pages)
            e[2].record(main)
            side.wait_event(e[1])
            with torch.cuda.stream(side):
                a[0].record(side)
                inner.attend_(q, kk, vv, S + step, out_p, phase=1)
                a[1].record(side)
            lc.update_tables_(page_list, advance_split=False)
            e[3].record(main)
            inner.attend_(q, kk, vv, S + step, out_p, phase=2)
            e[4].record(main)
            main.wait_event(a[1])
            recs.append((e, a))
            step += 1
        torch.cuda.synchronize()
        avg = lambda f: sum(f(e, a) for e, a in recs) / len(recs) * 1e3
        timeline = {
            "score": avg(lambda e, a: e[0].elapsed_time(e[1])),
            "topk": avg(lambda e, a: e[1].elapsed_time(e[2])),
            "lru": avg(lambda e, a: e[2].elapsed_time(e[3])),
            "attention_phase1_start_after_score": avg(lambda e, a: e[1].elapsed_time(a[0])),
            "attention_phase1": avg(lambda e, a: a[0].elapsed_time(a[1])),
            "attention_phase1_end_after_score": avg(lambda e, a: e[1].elapsed_time(a[1])),
            "attention_phase2_after_lru": avg(lambda e, a: e[3].elapsed_time(e[4])),
            "step": avg(lambda e, a: e[0].elapsed_time(e[4])),
        }
    inner.check_status()

    # ---------------- launch time of the two streaming kernels, for the roofline ---------------
    # R launches of one kernel, each behind a read sweep over 256 MB that evicts L2, captured in a graph and
    # timed with CUDA events; the same graph without the kernel is subtracted.  (Event pairs
    # around single eager launches, as in stage_us above, carry ~10-20 us of event overhead.)
    def launch_us(fn, reps=10):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        graphs = []
        for with_kernel in (True, False):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(reps):
                    flush.max()          # read-only sweep: evicts L2 without leaving dirty lines behind
                    if with_kernel:
                        fn()
            graphs.append(g)
        best = []
        for g in graphs:
            ts = []
            for _ in range(4):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            best.append(min(ts[1:]))
        del graphs
        return (best[0] - best[1]) / reps * 1e3

    kernel_us = {}
    if P:
        qf, kf, vf = dq[step - 1], dk[step - 1], dv[step - 1]
        pos_fixed = S + step - 1          # re-appends the token of the last step: same bytes, same place
        t_a = time.perf_counter()
        kernel_us["attention"] = launch_us(lambda: inner.attend_(qf, kf, vf, pos_fixed, out_p))
        kernel_us["score"] = launch_us(lambda: lc.top_k_selector.score_(qf, k_pages))
        windows.append((t_a, time.perf_counter()))
        inner.check_status()

    # ---------------- miss fetch: what it costs in a steady step, and a cold step against the host link ----
    fetch_report = None
    if world == 1 and P and captured:
        t_a = time.perf_counter()
        page_bytes = w.page_size * 2 * D * esz
        # (1) the same K-step graph with ONE query repeated: after the first step nothing misses,
        #     so the difference to `value` is the time the fetch leaves exposed.
        g0 = torch.cuda.CUDAGraph()
        first0 = step
        with torch.cuda.graph(g0):
            outs0 = [op(dq[first0], dk[first0 + i], dv[first0 + i], start_pos=S + first0 + i, stage="generate")
                     for i in range(K)]
        g0.replay()                      # brings the repeated query's pages in; also sets the graph up
        torch.cuda.synchronize()
        ev0.record()
        g0.replay()
        ev1.record()
        torch.cuda.synchronize()
        ms_nomiss = ev0.elapsed_time(ev1)
        step += K
        # (2) one step whose query is re-drawn from N(0,1): most of its pages are not resident
        gq = torch.Generator().manual_seed(1)
        q_cold = torch.randn(1, 1, hk * rep, D, generator=gq).to(w.dtype).to(dev)
        torch.cuda.synchronize()
        torch.cuda._sleep(20_000_000)    # the step is queued before the GPU starts it
        ev0.record()
        op(q_cold, dk[step], dv[step], start_pos=S + step, stage="generate")
        ev1.record()
        torch.cuda.synchronize()
        cold_us = ev0.elapsed_time(ev1) * 1e3
        cold_misses = int(lc.last_miss_counts(list_len).sum())
        step += 1
        inner.check_status()
        # (3) the host link itself: one pinned-host -> device copy of 64 MiB
        hbuf = torch.zeros(64 << 20, dtype=torch.uint8).pin_memory()
        dbuf = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
        link = []
        for _ in range(6):
            torch.cuda.synchronize()
            ev0.record()
            dbuf.copy_(hbuf, non_blocking=True)
            ev1.record()
            torch.cuda.synchronize()
            link.append((64 << 20) / (ev0.elapsed_time(ev1) * 1e-3) / 1e9)
        link_gbs = max(link[1:])
        steady_us = ms_value / K * 1e3
        fetch_us = max(cold_us - steady_us, 1e-3)
        fetch_report = {
            "steady_misses_per_step": (sum(misses) / len(misses)) if misses else None,
            "steady_bytes_per_step": (sum(misses) / len(misses) * page_bytes) if misses else None,
            "step_us_without_misses": ms_nomiss / K * 1e3,
            "exposed_fraction_of_step": max(0.0, 1.0 - ms_nomiss / ms_value),
            "cold_step": {"query": "re-drawn from N(0,1)", "misses": cold_misses,
                          "bytes": cold_misses * page_bytes, "step_us": cold_us,
                          "fetch_gbs": cold_misses * page_bytes / (fetch_us * 1e-6) / 1e9,
                          "host_link_gbs": link_gbs,
                          "frac_of_host_link": cold_misses * page_bytes / (fetch_us * 1e-6) / 1e9 / link_gbs,
                          "host_link_peak": "best of 5 pinned host -> device copies of 64 MiB on this box "
                                            "(PCIe Gen5 x16: 63 GB/s nominal)"},
        }
        windows.append((t_a, time.perf_counter()))

    # ---------------- page scorer + top-k over a sweep of page counts (8 KV heads, GQA 4, bf16) -----------
    sweep = None
    if world == 1 and P and not args.no_sweep:
        from dram_attention_b200.topk_selector import IPUpperboundTopKSelector
        t_a = time.perf_counter()
        peak_now, _ = hbm_peak_gbs()
        gs = torch.Generator(device=dev).manual_seed(0)
        s_hk, s_rep, s_pg, l_max = 8, 4, 16, 65536
        mm = torch.empty(s_hk, l_max, 2, D, dtype=torch.bfloat16, device=dev)
        for h in range(s_hk):
            keys = torch.randn(l_max, s_pg, D, generator=gs, device=dev).to(torch.bfloat16)
            mn, mx = torch.aminmax(keys, dim=1)
            mm[h, :, 0], mm[h, :, 1] = mn, mx
            del keys
        q_s = torch.randn(1, 1, s_hk * s_rep, D, generator=gs, device=dev).to(torch.bfloat16)
        sweep = []
        for n_pages in (512, 2048, 8192, 32768, 65536):
            shape_only = torch.empty(s_hk, n_pages * s_pg, D, dtype=torch.bfloat16, device="meta")
            sel = IPUpperboundTopKSelector(shape_only, n_pages, device=dev, _summaries=mm[:, :n_pages].contiguous())
            kk_pages = min(256, n_pages)
            sel.score_(q_s, kk_pages)
            sel.select_(1, s_rep, kk_pages)
            t_score = launch_us(lambda: sel.score_(q_s, kk_pages))
            t_topk = launch_us(lambda: sel.select_(1, s_rep, kk_pages))
            nbytes = s_hk * n_pages * 2 * D * 2 + s_hk * s_rep * D * 2
            sweep.append({"pages": n_pages, "score_us": t_score, "score_gbs": nbytes / (t_score * 1e-6) / 1e9,
                          "score_frac_of_peak": nbytes / (t_score * 1e-6) / 1e9 / peak_now,
                          "topk_us": t_topk, "k": kk_pages})
            del sel
        del mm
        windows.append((t_a, time.perf_counter()))
    # ---------------- prefill stage (off the decode path): the tcgen05 causal attention kernel ---------------
    prefill = None
    if world == 1 and P and not args.no_sweep:
        t_a = time.perf_counter()
        pf_s = args.prefill_tokens
        gp = torch.Generator(device=dev).manual_seed(2)
        pq = torch.randn(1, pf_s, w.n_q_heads, D, generator=gp, device=dev).to(w.dtype)
        pk = torch.randn(1, pf_s, hk_all, D, generator=gp, device=dev).to(w.dtype)
        pv = torch.randn(1, pf_s, hk_all, D, generator=gp, device=dev).to(w.dtype)
        flops = 4.0 * pf_s * pf_s / 2 * w.n_q_heads * D          # causal: half of the square
        peak_tf, peak_tf_kind = tensor_peak_tflops()

        def time_prefill(use_kernel):
            inner.prefill_kernel = use_kernel
            for _ in range(2):
                inner._prefill_attention(pq, pk, pv)
            torch.cuda.synchronize()
            ev0.record()
            for _ in range(3):
                inner._prefill_attention(pq, pk, pv)
            ev1.record()
            torch.cuda.synchronize()
            return ev0.elapsed_time(ev1) / 3

        ms_own, ms_lib = time_prefill(True), time_prefill(False)
        inner.prefill_kernel = True
        inner.check_status()
        prefill = {"what": f"causal attention of a {pf_s}-token prompt, {w.n_q_heads}/{hk_all} heads, bf16 "
                           "(stage=\"prefill\"; not part of the decode metric)",
                   "kernel": "prefill_attention_kernel (tcgen05.mma, TMEM accumulators, TMA operands)",
                   "ms": ms_own, "tflops": flops / ms_own / 1e9, "peak_tflops": peak_tf,
                   "peak_kind": peak_tf_kind + " cuBLAS bf16 GEMM (burst)", "frac": flops / ms_own / 1e9 / peak_tf,
                   "library_ms": ms_lib, "library_tflops": flops / ms_lib / 1e9,
                   "library": "torch scaled_dot_product_attention on the same tensors"}
        del pq, pk, pv
        windows.append((t_a, time.perf_counter()))

    # ---------------- N > 1, by sequence: the KV-head-sharded step of ONE sequence, timed beside it -------
    sharded_report = None
    if by_seq:
        t_a = time.perf_counter()
        n_sh = settle + W + K + 2
        w0 = w if rank == 0 else llama_layer_workload(seed=0, steps=n_sh, dram_tokens=args.dram_tokens,
                                                      max_out=n_sh)
        lo0, hi0 = head_range(hk_all, rank, world)
        sh = KVHeadShardedDRAMAttention(n_kv_heads=hk_all, presliced=True, device=dev, dtype=w.dtype,
                                        peer_gather=not args.library_gather,
                                        **dict(ctor, max_output_length=max(ctor["max_output_length"], n_sh)))
        sh.inner.init_cache(w0.k[:, :, lo0:hi0].to(dev), w0.v[:, :, lo0:hi0].to(dev))
        sq = w0.xq[:n_sh, :, :, lo0 * rep:hi0 * rep].contiguous().to(dev)
        sk = w0.xk[:n_sh, :, :, lo0:hi0].contiguous().to(dev)
        sv = w0.xv[:n_sh, :, :, lo0:hi0].contiguous().to(dev)
        S0 = w0.prefill_len
        w_sh = settle + W
        for i in range(w_sh):
            sh(sq[i], sk[i], sv[i], start_pos=S0 + i, stage="generate")
        torch.cuda.synchronize()
        g_sh = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_sh):
            outs_sh = [sh(sq[w_sh + i], sk[w_sh + i], sv[w_sh + i], start_pos=S0 + w_sh + i, stage="generate")
                       for i in range(K)]
        up = upload_graph(g_sh, torch)
        barrier()
        if not up:
            torch.cuda._sleep(20_000_000)
        ev0.record()
        g_sh.replay()
        ev1.record()
        barrier()
        sh.check_status()
        ms_sh = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
        dist.all_reduce(ms_sh, op=dist.ReduceOp.MAX)
        ms_sh = float(ms_sh[0])
        sharded_report = {
            "what": f"ONE sequence, its {hk_all} KV heads sharded {world}-way, K steps in one graph per rank, max over ranks",
            "value": K / (ms_sh * 1e-3), "unit": "tok/s", "ms_per_step": ms_sh / K, "scaling": "strong",
            "gather": ("peer stores over NVLink (da_gather_heads)" if sh._peer is not None
                       else "NCCL all_gather_into_tensor"),
        }
        windows.append((t_a, time.perf_counter()))
    sampler.stop()
    if world > 1:
        op.check_status()     # includes the gather kernel's bounded waits

    # ---------------- reduce over ranks -------------------------------------------------
    t = torch.tensor([ms_value, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_value, ms_e2e = float(t[0]), float(t[1])

    mean = lambda xs: (sum(xs) / len(xs)) if xs else None
    stage_us = {n: (mean(v) * 1e3 if v else None) for n, v in stage_ms.items()}
    if fused:
        stage_us["fetch"] = None   # no such launch: the attention kernel reads the missed pages itself
    t_local = (S + step - 1) - w.dram_tokens          # local tokens at the last profiled step
    n_slots_tokens = w.lru_hbm_cache_size
    b_attn = hk * (n_slots_tokens + t_local + 1) * 2 * D * esz + 2 * hk * rep * D * esz
    b_score = hk * (w.dram_tokens // w.page_size) * 2 * D * esz + hk * rep * D * esz
    peak, peak_kind = hbm_peak_gbs()
    roofline = None
    if kernel_us.get("attention"):
        ach = b_attn / (kernel_us["attention"] * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": "decode_attention_mma_kernel", "achieved": ach, "peak": peak,
                    "peak_kind": peak_kind + " HBM copy bandwidth", "unit": "GB/s", "frac": ach / peak,
                    "traffic": (ATTN_TRAFFIC_BYTES_128K if (world == 1 and args.dram_tokens == 131072) else None),
                    "algorithmic_bytes_per_launch": b_attn,
                    "launch_us": kernel_us["attention"],
                    "timing": "CUDA events around a graph of 10 launches, each behind an L2-evicting 256 MB read; "
                              "same graph without the launches subtracted"}
    roofline_score = None
    if kernel_us.get("score"):
        ach = b_score / (kernel_us["score"] * 1e-6) / 1e9
        roofline_score = {"bound": "hbm", "kernel": "score_pages_mma_kernel", "achieved": ach, "peak": peak,
                          "unit": "GB/s", "frac": ach / peak, "algorithmic_bytes_per_launch": b_score,
                          "launch_us": kernel_us["score"]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": n_seq * K / (ms_value * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_value / K, "higher_is_better": True,
            "scaling": ("weak" if (world == 1 or by_seq) else "strong"), "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": dict(workload_config(args, w), batch=n_seq,
                           parallelism=("single GPU" if world == 1 else
                                        f"{world} independent sequences, one per GPU, no collective on the path"
                                        if by_seq else f"KV heads sharded {world}-way, " +
                                        ("all-gather of per-head outputs by peer stores over NVLink (da_gather_heads)"
                                         if getattr(op, "_peer", None) is not None else
                                         "NCCL all-gather of per-head outputs")),
                           settle_steps=settle,
                           timed_region=("one CUDA graph of K steps, " +
                                         ("uploaded to the device" if uploaded else "launched behind a spin kernel") +
                                         " before the first event" if captured else
                                         "K eager steps (graph capture failed: " + capture_error + ")")),
            "clocks": sampler.summary(windows),
            "e2e": {"value": n_seq * K / (ms_e2e * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": (hq[0].numel() + hkk[0].numel() + hv[0].numel()) * esz * world,
                    "d2h_bytes_per_step": out_h.numel() * esz * world, "ms_per_step": ms_e2e / K,
                    "per_step": "host writes q|k|v into a pinned staging buffer; one graph replay = H2D copy, the step, "
                                "D2H copy of the output; stream sync"},
            "gpu_launches": ((5 if (overlapped or not fused) else 4) + (1 if (world > 1 and not by_seq) else 0))
                            * K * world,
            "kv_head_sharded": sharded_report,
            "roofline": roofline,
            "roofline_score": roofline_score,
            "stage_us_with_event_overhead": stage_us,
            "overlapped_timeline_us": timeline,
            "step_layout": ("{score -> top-k -> LRU || attention phase 1} -> attention phase 2 (+fetch)"
                            if overlapped else ("score -> top-k -> LRU -> attention (+fetch)" if fused else
                                                "score -> top-k -> LRU -> fetch -> attention")),
            "misses_per_step": mean(misses),
            "fetch": ("inside the attention kernel" if fused else "separate gather-copy launch"),
            "fetch_report": fetch_report,
            "scorer_sweep": sweep,
            "prefill": prefill,
            "fetch_fraction_of_step": (stage_us["fetch"] / sum(v for v in stage_us.values() if v)
                                       if stage_us["fetch"] else None),
        }
        if world == 1 and not args.no_cpu_baseline:
            tps, done, threads = cpu_reference_steps(w, 1, min(32, total - 1), budget_s=15.0)
            line["cpu_baseline"] = {
                "value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                "sample": f"{done} full generate steps of the same layer (1 warm-up) on the host cores: "
                          "CPU port of the reference's pure-PyTorch path"}
        print(json.dumps(line), file=RESULT_OUT, flush=True)
    if world > 1:
        # No collective follows the timing all-reduce, so every rank can leave on its own.  The
        # process group is not torn down: the captured graphs still reference the communicator,
        # and destroying it under them has been seen to block at exit.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


RESULT_OUT = sys.stdout


def main():
    global RESULT_OUT
    args = parse_args()
    # The JSON line must be the only thing on stdout, but libraries (the NCCL version banner, for one)
    # write to file descriptor 1 directly: keep a private copy of it for the result and point
    # descriptor 1 at stderr for everything else.
    sys.stdout.flush()
    RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()

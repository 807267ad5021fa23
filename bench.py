#!/usr/bin/env python
"""Benchmark of the generate stage of DRAM Attention on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config cfg2|cfg4|cfg5]

One "step" = one generate step (one new token) of one attention layer: page scoring, top-k
selection, LRU update (with the copy of the few missed pages), decode attention.  Prints ONE
JSON line.

Headline (default, --config cfg2): the Llama-3-8B-shaped 128K-context decode layer, one sequence
per GPU (N > 1: N independent sequences, no collective on the path, weak scaling).

value    decode tok/s with every input resident in HBM.  K timed steps, each with its own
         device-resident inputs, are captured in one CUDA graph, the graph is uploaded, and one
         replay is timed with CUDA events (max over ranks).  That is done for several disjoint
         windows of K consecutive steps; `value` is the median window, `windows` lists them all.
e2e      the same metric through the operator API with HOST inputs: per step the query/key/value
         are written into a pinned staging buffer, one captured graph (host->device copy, the
         step, device->host copy of the output) is replayed and the stream is synchronised.
roofline  the attention launch that carries most of the bytes as the step really runs it (phase 1
         of the two-launch layout), from device-side time stamps of the last step of an extra,
         untimed window; roofline_phase2, roofline_score, roofline_step (all algorithmic bytes of
         a step / ms_per_step) and roofline_single_launch (the same attention as one launch,
         timed alone by graph difference) beside it.  Fractions are of the measured HBM copy
         bandwidth of this pool and, separately, of the nominal 8 TB/s.
timeline_us  where the time of a step goes: start and end of every kernel of the step's last
         replayed step, from the same stamps.
cpu_baseline  the CPU oracle (a port of the reference's pure-PyTorch path, float32) timed on a
         bounded sample of the same workload on this box's host cores.

Extras in the same line (skipped with --no-extras): rope_in_call (the step with the caller's
rotary embedding done by the operator), fetch_report (miss fetch against the host link),
scorer_sweep (config 3), prefill, and the two other multi-GPU configurations:
cfg4     8 independent 64K-token sequences, 128 steps with a query re-draw every 32 steps,
         sequences dealt round-robin to the N GPUs (no collective) and, on a GPU, to up to four
         streams (they are independent); the one-stream figure is in the object as well.
cfg5     a 32-layer stack at a 1,048,576-token prefix per layer, KV heads sharded N-way with the
         per-head outputs all-gathered by a peer-memory kernel over NVLink; the whole token step
         (all layers) in one CUDA graph.
kv_head_sharded (N > 1)  ONE 128K sequence with its KV heads sharded N-way, with its efficiency
         against the one-GPU step of the same run.
--config cfg4 / cfg5 makes that configuration the headline instead.
--impl reference times the CPU port of the reference path on rank 0 only.
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
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one single-launch attention at the default workload, from
# the ncu capture summarised in profiles/decode_attention_mma_llama128k.md
ATTN_TRAFFIC_BYTES_128K = 154.4e6
# the same counters for the phase-1 launch form of the default step (same profile file)
PHASE1_TRAFFIC_BYTES_128K = 151.3e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="cfg2", choices=["cfg2", "cfg4", "cfg5"],
                    help="which BASELINE configuration is the headline of the line")
    ap.add_argument("--dram-tokens", type=int, default=131072, help="cfg2: prefix tokens kept in DRAM")
    ap.add_argument("--windows", type=int, default=5, help="cfg2: disjoint windows of K steps that are timed")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline configuration (no cfg4 / cfg5 / sweep / prefill / fetch report)")
    ap.add_argument("--shard", default="sequence", choices=["sequence", "kv-heads"],
                    help="cfg2, N > 1: one independent sequence per GPU (weak scaling, default; the KV-head-"
                         "sharded step is timed as well), or only ONE sequence with its KV heads sharded")
    ap.add_argument("--library-gather", action="store_true",
                    help="N > 1: all-gather through the process group instead of the peer-memory kernel")
    ap.add_argument("--prefill-tokens", type=int, default=32768, help="prompt length of the prefill report")
    ap.add_argument("--only-prefill", action="store_true",
                    help="time just the prefill kernel at --prefill-tokens (a small launch to profile) and exit")
    ap.add_argument("--only-sweep", action="store_true",
                    help="run just the page scorer and the selection at 8 KV heads x 65536 pages (config 3's largest "
                         "case) three times and exit: a small job to profile")
    ap.add_argument("--settle-steps", type=int, default=0,
                    help="cfg2: untimed decode steps before the warm-up (0: the timed windows start right after "
                         "the warm-up, inside the 64 steps the configuration names)")
    ap.add_argument("--clock-period-ms", type=float, default=2.0,
                    help="NVML polling period while the GPU works alone; the end-to-end loop is polled 10x slower")
    ap.add_argument("--reference-gpu", action="store_true",
                    help="also time the UNMODIFIED reference package on this GPU (its Triton kernels and flash-attn), "
                         "if a copy of it lies under the git-ignored baseline/_ref/; one data point, off by default")
    ap.add_argument("--cfg4-sequences", type=int, default=8)
    ap.add_argument("--cfg4-steps", type=int, default=128)
    ap.add_argument("--cfg4-redraw", type=int, default=32)
    ap.add_argument("--cfg4-streams", type=int, default=4,
                    help="the sequences of a GPU are dealt to this many streams (they are independent: one "
                         "sequence's selection chain then overlaps another's attention); the one-stream figure is "
                         "measured as well, on the steps that follow")
    ap.add_argument("--cfg5-layers", type=int, default=32)
    ap.add_argument("--cfg5-steps", type=int, default=32)
    ap.add_argument("--cfg5-prefixes", type=int, default=4,
                    help="distinct synthetic prefixes (pinned DRAM copies) the layers of the stack share; "
                         "32 = every layer its own 4 GiB (128 GiB of pinned host memory unsharded)")
    ap.add_argument("--cfg5-streams", type=int, default=0,
                    help="layers of a token step alternate over this many streams (their synthetic inputs make "
                         "them independent), so that one layer's chain overlaps the next ones' attention; 0 = by "
                         "shard size: 2 streams with 8 KV heads per GPU, 4 with 4 or 2, 8 with 1 (the smaller the "
                         "shard, the less of the GPU one layer's chain can keep busy)")
    return ap.parse_args()


# --------------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------------

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

    def sample_now(self):
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

    def _run(self):
        while not self.stop_flag:
            self.sample_now()
            time.sleep(self.period)

    def start(self):
        if self.nv is not None and self.period > 0:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join()

    def median_mhz(self, window):
        inside = [s[1] for s in self.samples if window[0] <= s[0] <= window[1]]
        return statistics.median(inside) if inside else None

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
    """Places the instantiated graph on the device before it is timed (otherwise its first launch
    pays a one-time set-up of several microseconds per captured step)."""
    try:
        from cuda.bindings import runtime as rt
        exec_handle = rt.cudaGraphExec_t(int(graph.raw_cuda_graph_exec()))
        (err,) = rt.cudaGraphUpload(exec_handle, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return int(err) == 0
    except Exception:
        return False


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {}


def hbm_peak_gbs():
    p = _peaks()
    return (float(p["hbm_gbs"]), "measured") if "hbm_gbs" in p else (FALLBACK_HBM_GBS, "fallback")


def tensor_peak_tflops():
    p = _peaks()
    return (float(p["bf16_tflops"]), "measured") if "bf16_tflops" in p else (1590.0, "fallback")


def roofline_obj(kernel, nbytes, us, **extra):
    """bytes / time against the measured copy bandwidth (and the nominal 8 TB/s beside it)."""
    if not us or us <= 0:
        return None
    peak, kind = hbm_peak_gbs()
    ach = nbytes / (us * 1e-6) / 1e9
    obj = {"bound": "hbm", "kernel": kernel, "achieved": ach, "peak": peak,
           "peak_kind": kind + " HBM copy bandwidth", "unit": "GB/s", "frac": ach / peak,
           "frac_of_nominal_8tbs": ach / NOMINAL_HBM_GBS, "algorithmic_bytes_per_launch": nbytes, "launch_us": us}
    obj.update(extra)
    return obj


class Ctx:
    """Process / device context of one rank."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torchrun for N > 1")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # stdout carries the JSON line only
            # plain rings / trees and plain peer stores: nothing of this process is bound to an NVLink
            # multicast object when it exits
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.sampler = ClockSampler(self.local_rank, period_s=args.clock_period_ms * 1e-3)
        self.windows = []

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def sum_over_ranks(self, values):
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return [float(x) for x in t]


def time_graph(ctx, capture_fn):
    """Captures capture_fn() into a CUDA graph, uploads it, replays it once between two events.
    Returns (ms on this rank, outputs of capture_fn, uploaded, wall-clock window, graph)."""
    torch = ctx.torch
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = capture_fn()
    uploaded = upload_graph(graph, torch)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.barrier()
    t_a = time.perf_counter()
    if not uploaded:
        torch.cuda._sleep(20_000_000)    # the launch is queued before the GPU starts it
    ev0.record()
    graph.replay()
    ev1.record()
    ctx.barrier()
    window = (t_a, time.perf_counter())
    ctx.windows.append(window)
    return ev0.elapsed_time(ev1), outs, uploaded, window, graph


# --------------------------------------------------------------------------------
# device-side time line of a step (da_trace_set)
# --------------------------------------------------------------------------------

class StepTrace:
    KERNELS = ["score", "topk", "lru", "attention_phase1", "attention_phase2", "gather"]

    def __init__(self, ctx):
        from dram_attention_b200 import _native
        self.lib = _native.lib()
        self.torch = ctx.torch
        self.buf = ctx.torch.zeros(self.lib.da_trace_bytes() // 8, dtype=ctx.torch.int64, device=ctx.dev)

    def __enter__(self):
        self.torch.cuda.synchronize()
        self.buf.zero_()
        rc = self.lib.da_trace_set(self.buf.data_ptr())
        assert rc == 0, rc
        return self

    def __exit__(self, *exc):
        self.torch.cuda.synchronize()
        self.lib.da_trace_set(0)

    def timeline(self):
        """Start / end of every kernel of the last step that ran, in microseconds after the first
        CTA of the step got onto an SM."""
        import numpy as np
        n = len(self.KERNELS)
        t = self.buf.cpu().numpy().reshape(n, 1024, 4)
        live = [t[k][:, 0] > 0 for k in range(n)]
        starts = [t[k][live[k], 0] for k in range(n - 1) if live[k].any()]   # the gather's CTA may sit on its SM from
                                                                             # before the step's first kernel
        if not starts:
            return None
        t0 = min(int(s.min()) for s in starts)
        us = lambda x: (int(x) - t0) / 1e3
        out = {}
        for k, name in enumerate(self.KERNELS):
            m = live[k]
            if not m.any():
                continue
            e = {"ctas": int(m.sum()), "first_cta_on_sm": us(t[k][m, 0].min()), "last_cta_on_sm": us(t[k][m, 0].max()),
                 "end": us(t[k][m, 1].max())}
            if k in (1, 2):
                w = t[k][m, 2]
                e["predecessor_done"] = us(w[w > 0].max()) if (w > 0).any() else None
            if k in (3, 4):
                le = t[k][m, 2]
                e["units_done_min"], e["units_done_median"], e["units_done_max"] = \
                    us(le.min()), us(np.median(le)), us(le.max())
                e["last_ticket"] = us(t[k][m, 3].max())
            if k == 5:
                e = {"on_sm": us(t[k][0, 0]), "rows_ready": us(t[k][0, 2]), "sent": us(t[k][0, 3]),
                     "all_ranks_there_and_copied": us(t[k][0, 1]), "end": us(t[k][0, 1])}
            out[name] = e
        out["step_end"] = max(v["end"] for v in out.values())
        return out


# --------------------------------------------------------------------------------
# CPU port of the reference path (oracle) -- cpu_baseline leg and --impl reference
# --------------------------------------------------------------------------------

def cpu_reference_steps(w, n_warm, n_timed, budget_s=None):
    """Steps of the CPU oracle on workload w, float32 throughout (what the reference's pure-PyTorch
    path computes in); returns (tok/s, steps timed, threads)."""
    import torch
    from oracle import dram_attention_oracle as orc
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    o = orc.OracleDRAMAttention(dtype=torch.float32, **w.ctor_kwargs())
    o.attn_dtype = torch.float32
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


def cfg2_config(w):
    """The workload description both arms print (identical, so that the two lines compare)."""
    return {
        "workload": w.name,
        "batch": 1, "n_q_heads": w.n_q_heads, "n_kv_heads": w.n_kv_heads, "head_dim": w.head_dim,
        "dram_prefix_tokens": w.dram_tokens, "page_size": w.page_size,
        "lru_hbm_cache_size": w.lru_hbm_cache_size, "local_cache_size": w.local_cache_size,
        "top_k": w.top_k, "prefill_len": w.prefill_len,
        "l2": "inputs larger than L2 (185 MB touched per step vs 126 MB)",
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from dram_attention_b200.synthetic import llama_layer_workload
    k, wu = args.steps, args.warmup
    w = llama_layer_workload(seed=0, steps=k + wu, dram_tokens=args.dram_tokens, max_out=k + wu)
    tps, done, threads = cpu_reference_steps(w, wu, k)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": done, "warmup": wu, "ms_per_step": 1e3 / tps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg2_config(w),
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{done} full generate steps of the same layer after {wu} warm-up steps, "
                                   "CPU port of the reference's pure-PyTorch path, float32 scores and attention"},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=RESULT_OUT, flush=True)


# --------------------------------------------------------------------------------
# cfg2: the 128K-context layer
# --------------------------------------------------------------------------------

def layer_bytes(hk, rep, d, n_pages, n_slots, page, t_local, esz=2):
    b_score = hk * n_pages * 2 * d * esz + hk * rep * d * esz
    b_attn = hk * (n_slots * page + t_local + 1) * 2 * d * esz + 2 * hk * rep * d * esz
    return b_score, b_attn


def total_misses(lru_cache) -> float:
    return float(lru_cache.evict_redo[1].sum().item())


def bench_cfg2(args, ctx):
    torch, dist = ctx.torch, ctx.dist
    import dram_attention_b200 as da
    from dram_attention_b200.sharded import KVHeadShardedDRAMAttention, head_range
    from dram_attention_b200.synthetic import llama_layer_workload
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    K, W = args.steps, max(args.warmup, 3)
    NW = max(1, args.windows)
    settle = max(0, args.settle_steps)
    total = settle + W + (NW + 1) * K + (W + K) + 3 * K + 8 + (W + 2 * K + 4 if args.reference_gpu else 0)
    by_seq = world > 1 and args.shard == "sequence"
    n_seq = world if by_seq else 1
    w = llama_layer_workload(seed=(rank if by_seq else 0), steps=total, dram_tokens=args.dram_tokens, max_out=total)
    hk_all, rep, D = w.n_kv_heads, w.n_q_heads // w.n_kv_heads, w.head_dim
    lo, hi = (0, hk_all) if (world == 1 or by_seq) else head_range(hk_all, rank, world)
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
    n_pages, n_slots = w.dram_tokens // w.page_size, w.lru_hbm_cache_size // w.page_size

    hq = w.xq[:, :, :, lo * rep:hi * rep].contiguous().pin_memory()
    hkk = w.xk[:, :, :, lo:hi].contiguous().pin_memory()
    hv = w.xv[:, :, :, lo:hi].contiguous().pin_memory()
    dq, dk, dv = hq.to(dev), hkk.to(dev), hv.to(dev)

    # ---------------- value: windows of K captured steps, inputs resident in HBM -----------------
    step = 0
    for _ in range(settle + W):     # set-up steps, the last W of them the warm-up
        op(dq[step], dk[step], dv[step], start_pos=S + step, stage="generate")
        step += 1
    torch.cuda.synchronize()
    if hasattr(op, "check_status"):
        op.check_status()           # also: a gather's first (eager) call has set its buffers up

    def capture_steps(first):
        return [op(dq[first + i], dk[first + i], dv[first + i], start_pos=S + first + i, stage="generate")
                for i in range(K)]

    win_ms, win_mhz, win_first = [], [], []
    uploaded = True
    miss_before = total_misses(lc)
    for _ in range(NW):
        first = step
        ms, outs, up, window, _g = time_graph(ctx, lambda: capture_steps(first))
        uploaded = uploaded and up
        assert len(outs) == K and all(bool(torch.isfinite(o.float()).all()) for o in outs), "a timed step left no output"
        win_ms.append(ms)
        win_mhz.append(ctx.sampler.median_mhz(window))
        win_first.append(first)
        step += K
        del outs, _g
    misses_per_step = (total_misses(lc) - miss_before) / (NW * K)
    redo_steps = int(lc.evict_redo[2].max().item())
    win_ms = ctx.max_over_ranks(win_ms)
    ms_value = statistics.median(win_ms)

    # ---------------- one more, untimed window with the device-side time stamps switched on -------
    tr = StepTrace(ctx)
    g = torch.cuda.CUDAGraph()
    first = step
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        outs_t = capture_steps(first)
    ctx.barrier()
    with tr:
        g.replay()
    timeline = tr.timeline()
    ctx.barrier()
    step += K
    del g, outs_t
    inner.check_status()

    # ---------------- e2e: host inputs, one captured step per call ----------------------
    nq, nk = dq[0].numel(), dk[0].numel()
    h_in = torch.cat([hq.reshape(total, -1), hkk.reshape(total, -1), hv.reshape(total, -1)], dim=1).pin_memory()
    d_in = torch.empty(nq + 2 * nk, dtype=w.dtype, device=dev)
    xq_s = d_in[:nq].view(dq[0].shape)
    xk_s = d_in[nq:nq + nk].view(dk[0].shape)
    xv_s = d_in[nq + nk:].view(dv[0].shape)
    out_h = torch.empty(1, 1, hk * rep * (world if not by_seq and world > 1 else 1), D, dtype=w.dtype).pin_memory()
    pos = torch.tensor([S + step], dtype=torch.int32, device=dev)
    h_stage = torch.empty_like(h_in[0]).pin_memory()
    step_graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(step_graph):
        d_in.copy_(h_stage, non_blocking=True)
        out_h.copy_(op(xq_s, xk_s, xv_s, start_pos=pos, stage="generate"), non_blocking=True)
        pos.add_(1)
    h_rows = list(h_in.unbind(0))
    cur_stream = torch.cuda.current_stream()

    def e2e_step(i):
        h_stage.copy_(h_rows[i])        # host-side, 12 KiB
        step_graph.replay()
        cur_stream.synchronize()

    # NVML queries take driver locks that the launch path also wants: polled every 2 ms they cost this
    # host-bound loop ~20 us per step.  So the poller is slowed tenfold here and the region is bracketed by
    # one sample on each side, taken outside the events.
    fast_period = ctx.sampler.period
    ctx.sampler.period = 10 * fast_period
    for _ in range(W):
        e2e_step(step)
        step += 1
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.barrier()
    t_a = time.perf_counter()
    ctx.sampler.sample_now()
    ev0.record()
    for _ in range(K):
        e2e_step(step)
        step += 1
    ev1.record()
    ctx.barrier()
    ctx.sampler.sample_now()
    ctx.windows.append((t_a, time.perf_counter()))
    ctx.sampler.period = fast_period
    (ms_e2e,) = ctx.max_over_ranks([ev0.elapsed_time(ev1)])

    # ---------------- rooflines ------------------------------------------------------------
    t_local = (S + step - 1) - w.dram_tokens
    b_score, b_attn = layer_bytes(hk, rep, D, n_pages, n_slots, w.page_size, t_local, esz)
    n_front = int(lc.split_cap)
    tok_bytes = 2 * D * esz
    b_phase1 = hk * ((n_slots - n_front) * w.page_size + t_local + 1) * tok_bytes
    b_phase2 = hk * n_front * w.page_size * tok_bytes
    roof = {}
    if timeline:
        p1, p2, sc = timeline.get("attention_phase1"), timeline.get("attention_phase2"), timeline.get("score")
        stamp_note = ("device time stamps (first CTA on an SM -> last CTA done) of the last step of an untimed "
                      "window of K steps replayed as one graph")
        if p1:
            roof["roofline"] = roofline_obj(
                "decode_attention_mma_kernel, phase 1 of the default two-launch step", b_phase1,
                p1["end"] - p1["first_cta_on_sm"], timing=stamp_note,
                streaming_us=p1["units_done_median"] - p1["first_cta_on_sm"],
                traffic=(PHASE1_TRAFFIC_BYTES_128K if (hk == 8 and args.dram_tokens == 131072) else None),
                traffic_note="dram__bytes_read.sum + dram__bytes_write.sum of one phase-1 launch of this workload "
                             "(ncu capture summarised in profiles/decode_attention_mma_llama128k.md)")
        if p2:
            roof["roofline_phase2"] = roofline_obj("decode_attention_mma_kernel, phase 2 (eviction front + merge of both)",
                                                   b_phase2, p2["end"] - p2["first_cta_on_sm"], timing=stamp_note,
                                                   waits_for="the LRU update: its CTAs are on their SMs early and wait")
        if sc:
            roof["roofline_score"] = roofline_obj("score_pages_mma_kernel", b_score, sc["end"] - sc["first_cta_on_sm"],
                                                  timing=stamp_note)
    roof["roofline_step"] = roofline_obj("whole generate step (all five launches)", b_score + b_attn,
                                         ms_value / K * 1e3, timing="the headline: ms_per_step of the median window")

    # the same attention as ONE launch over everything, timed alone: R launches, each behind a read sweep
    # over 256 MB that evicts L2, captured in a graph; the same graph without the launches subtracted
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

    out_p = torch.empty(1, 1, hk * rep, D, dtype=w.dtype, device=dev)
    qf, kf, vf = dq[step - 1], dk[step - 1], dv[step - 1]
    pos_fixed = S + step - 1          # re-appends the token of the last step: same bytes, same place
    t_a = time.perf_counter()
    us_single = launch_us(lambda: inner.attend_(qf, kf, vf, pos_fixed, out_p))
    ctx.windows.append((t_a, time.perf_counter()))
    roof["roofline_single_launch"] = roofline_obj(
        "decode_attention_mma_kernel as one launch over all slots and the local window (not what the default step runs)",
        b_attn, us_single,
        traffic=(ATTN_TRAFFIC_BYTES_128K if (world == 1 and args.dram_tokens == 131072) else None),
        timing="CUDA events around a graph of 10 launches, each behind an L2-evicting 256 MB read; same graph "
               "without the launches subtracted")
    inner.check_status()

    return {
        "w": w, "op": op, "inner": inner, "K": K, "W": W, "n_seq": n_seq, "by_seq": by_seq, "hk": hk, "rep": rep,
        "ms_value": ms_value, "ms_e2e": ms_e2e, "win_ms": win_ms, "win_mhz": win_mhz, "win_first": win_first,
        "uploaded": uploaded, "timeline": timeline, "roof": roof, "misses_per_step": misses_per_step,
        "redo_steps": redo_steps, "h2d": (hq[0].numel() + hkk[0].numel() + hv[0].numel()) * esz * world,
        "d2h": out_h.numel() * esz * (world if by_seq or world == 1 else 1), "dq": dq, "dk": dk, "dv": dv,
        "step": step, "S": S, "launch_us": launch_us, "b_score": b_score, "b_attn": b_attn,
    }


def cfg2_extras(args, ctx, r):
    """fetch report, scorer / top-k sweep (config 3), prefill: a one-GPU run only."""
    torch, dev = ctx.torch, ctx.dev
    w, op, inner, K = r["w"], r["op"], r["inner"], r["K"]
    dq, dk, dv, S, step = r["dq"], r["dk"], r["dv"], r["S"], r["step"]
    lc = inner.lru_cache
    hk, rep, D, esz = r["hk"], r["rep"], w.head_dim, 2
    launch_us = r["launch_us"]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = {}

    # ---------------- the caller's rotary embedding inside the call (freqs_cis=) ----------------------
    t_a = time.perf_counter()
    # angle 0 everywhere: the kernel runs and the arithmetic is done, but queries and keys stay what they are,
    # so both graphs see the same pages (the synthetic prefix was not rotated by position; real angles would
    # turn the query stream into a different, unrelated one and the difference would be its misses)
    rope_us = {}
    for name in ("without", "with_freqs_cis"):
        first_r = step
        fr = [torch.polar(torch.ones(1, D // 2, device=dev), torch.zeros(1, D // 2, device=dev)) for i in range(K)]
        torch.cuda.synchronize()
        g_r = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_r):
            outs_r = [op(dq[first_r + i], dk[first_r + i], dv[first_r + i], start_pos=S + first_r + i, stage="generate",
                         **({"freqs_cis": fr[i]} if name == "with_freqs_cis" else {})) for i in range(K)]
        upload_graph(g_r, torch)
        torch.cuda.synchronize()
        ev0.record()
        g_r.replay()
        ev1.record()
        torch.cuda.synchronize()
        rope_us[name] = ev0.elapsed_time(ev1) / K * 1e3
        step += K
        del outs_r, g_r
    inner.check_status()
    out["rope_in_call"] = {"what": "K captured steps with the operator applying the caller's rotary embedding itself "
                                   "(da_rope_qk, one launch in front of the scorer; rotation by angle 0, see the code) and K steps "
                                   "without, us per step",
                           "us_per_step": rope_us}
    ctx.windows.append((t_a, time.perf_counter()))

    # ---------------- miss fetch: a steady step without misses, and a cold step against the host link ----
    t_a = time.perf_counter()
    page_bytes = w.page_size * 2 * D * esz
    first0 = step
    g0 = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(g0):
        outs0 = [op(dq[first0], dk[first0 + i], dv[first0 + i], start_pos=S + first0 + i, stage="generate")
                 for i in range(K)]
    g0.replay()                      # ONE query repeated: after this replay nothing misses any more
    torch.cuda.synchronize()
    # (the replay appends the same K tokens to the same places again)
    ev0.record()
    g0.replay()
    ev1.record()
    torch.cuda.synchronize()
    ms_nomiss = ev0.elapsed_time(ev1)
    step += K
    del outs0, g0
    gq = torch.Generator().manual_seed(1)
    q_cold = torch.randn(1, 1, hk * rep, D, generator=gq).to(w.dtype).to(dev)
    miss0 = total_misses(lc)
    torch.cuda.synchronize()
    torch.cuda._sleep(20_000_000)    # the step is queued before the GPU starts it
    ev0.record()
    op(q_cold, dk[step], dv[step], start_pos=S + step, stage="generate")
    ev1.record()
    torch.cuda.synchronize()
    cold_us = ev0.elapsed_time(ev1) * 1e3
    cold_misses = int(total_misses(lc) - miss0)
    step += 1
    inner.check_status()
    # the host link itself: pinned host -> device copies of 256 MiB (median and best of 10), and the
    # library's own gather-copy kernel reading the same pinned buffer through the mapping, page by page
    nb = 256 << 20
    hbuf = torch.zeros(nb, dtype=torch.uint8).pin_memory()
    dbuf = torch.empty(nb, dtype=torch.uint8, device=dev)
    link = []
    for _ in range(11):
        torch.cuda.synchronize()
        ev0.record()
        dbuf.copy_(hbuf, non_blocking=True)
        ev1.record()
        torch.cuda.synchronize()
        link.append(nb / (ev0.elapsed_time(ev1) * 1e-3) / 1e9)
    link = link[1:]
    from dram_attention_b200 import _native
    n_pg = nb // page_bytes
    pages = torch.arange(n_pg, dtype=torch.int32, device=dev)[None].contiguous()
    nmiss = torch.tensor([n_pg], dtype=torch.int32, device=dev)
    zc = []
    for _ in range(6):
        torch.cuda.synchronize()
        ev0.record()
        _native.check(_native.lib().da_fetch_pages(hbuf.data_ptr(), dbuf.data_ptr(), pages.data_ptr(), pages.data_ptr(),
                                                   nmiss.data_ptr(), n_pg, 1, n_pg, n_pg, page_bytes, _native.stream_ptr()))
        ev1.record()
        torch.cuda.synchronize()
        zc.append(nb / (ev0.elapsed_time(ev1) * 1e-3) / 1e9)
    del hbuf, dbuf
    link_peak = max(link)
    steady_us = r["ms_value"] / K * 1e3
    fetch_us = max(cold_us - steady_us, 1e-3)
    fetch_gbs = cold_misses * page_bytes / (fetch_us * 1e-6) / 1e9
    out["fetch_report"] = {
        "steady_misses_per_step": r["misses_per_step"],
        "steady_bytes_per_step": r["misses_per_step"] * page_bytes,
        "step_us_without_misses": ms_nomiss / K * 1e3,
        "exposed_fraction_of_step": max(0.0, 1.0 - ms_nomiss / r["ms_value"]),
        "host_link": {"copy_256MiB_gbs_median": statistics.median(link), "copy_256MiB_gbs_best": link_peak,
                      "gather_kernel_zero_copy_gbs_best": max(zc[1:]),
                      "what": "pinned host -> device cudaMemcpyAsync of 256 MiB, 10 repeats; and da_fetch_pages reading "
                              "the same pinned buffer through its device mapping in 8 KiB pages"},
        "cold_step": {"query": "re-drawn from N(0,1)", "misses": cold_misses, "bytes": cold_misses * page_bytes,
                      "step_us": cold_us, "fetch_gbs": fetch_gbs, "frac_of_host_link": fetch_gbs / link_peak},
    }
    ctx.windows.append((t_a, time.perf_counter()))

    # ---------------- page scorer + top-k over a sweep of page counts (config 3) -----------
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
    out["scorer_sweep"] = sweep
    ctx.windows.append((t_a, time.perf_counter()))

    # ---------------- prefill stage (off the decode path): the tcgen05 causal attention kernel -------
    t_a = time.perf_counter()
    pf_s = args.prefill_tokens
    gp = torch.Generator(device=dev).manual_seed(2)
    pq = torch.randn(1, pf_s, w.n_q_heads, D, generator=gp, device=dev).to(w.dtype)
    pk = torch.randn(1, pf_s, w.n_kv_heads, D, generator=gp, device=dev).to(w.dtype)
    pv = torch.randn(1, pf_s, w.n_kv_heads, D, generator=gp, device=dev).to(w.dtype)
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
    out["prefill"] = {"what": f"causal attention of a {pf_s}-token prompt, {w.n_q_heads}/{w.n_kv_heads} heads, bf16 "
                              "(stage=\"prefill\"; not part of the decode metric)",
                      "kernel": "prefill_attention_kernel (tcgen05.mma, TMEM accumulators, TMA operands)",
                      "ms": ms_own, "tflops": flops / ms_own / 1e9, "peak_tflops": peak_tf,
                      "peak_kind": peak_tf_kind + " cuBLAS bf16 GEMM (burst)", "frac": flops / ms_own / 1e9 / peak_tf,
                      "library_ms": ms_lib, "library_tflops": flops / ms_lib / 1e9,
                      "library": "torch scaled_dot_product_attention on the same tensors"}
    del pq, pk, pv
    ctx.windows.append((t_a, time.perf_counter()))
    return out


def bench_reference_gpu(args, ctx, w):
    """One data point for the unmodified reference on this GPU: its DRAMAttention (Triton scorer and LRU
    kernels, flash-attn for the two attention calls, torch for the rest) on the same layer, eager steps
    after a warm start; nothing of this package is on that path.  Any failure is reported as text."""
    torch, dev = ctx.torch, ctx.dev
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "dram_attention")):
        return {"unavailable": "no copy of the reference package under baseline/_ref/"}
    try:
        if ref_root not in sys.path:
            sys.path.insert(0, ref_root)
        import dram_attention as ref
        K, W = args.steps, max(args.warmup, 3)
        m = ref.DRAMAttention(device=dev, dtype=w.dtype, **w.ctor_kwargs())
        m.init_cache(w.k.to(dev), w.v.to(dev))
        S = w.prefill_len
        dq, dk, dv = w.xq.to(dev), w.xk.to(dev), w.xv.to(dev)
        for i in range(W):      # Triton compiles and autotunes here
            out = m(dq[i], dk[i], dv[i], start_pos=S + i, stage="generate")
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(W, W + K):
            out = m(dq[i], dk[i], dv[i], start_pos=S + i, stage="generate")
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / K
        res = {"what": "unmodified reference DRAMAttention on this GPU, generate steps after a warm start", "steps": K,
               "eager_ms_per_step": ms, "eager_tok_s": 1e3 / ms, "finite": bool(torch.isfinite(out.float()).all())}
        # the way its chat example decodes: ONE step captured in a CUDA graph with a device-side position,
        # replayed per token (examples/long-qa-chat/chat.py:238-249, :272)
        try:
            first = W + K
            xq, xk, xv = dq[first].clone(), dk[first].clone(), dv[first].clone()
            pos = torch.tensor([S + first], dtype=torch.int32, device=dev)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                m(xq, xk, xv, start_pos=pos, stage="generate")
            torch.cuda.current_stream().wait_stream(side)
            pos.add_(1)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out_g = m(xq, xk, xv, start_pos=pos, stage="generate")
            torch.cuda.synchronize()
            ev0.record()
            for i in range(K):
                xq.copy_(dq[first + 1 + i]); xk.copy_(dk[first + 1 + i]); xv.copy_(dv[first + 1 + i])
                g.replay()
                pos.add_(1)
            ev1.record()
            torch.cuda.synchronize()
            gms = ev0.elapsed_time(ev1) / K
            res.update(graph_ms_per_step=gms, graph_tok_s=1e3 / gms, graph_finite=bool(torch.isfinite(out_g.float()).all()))
        except Exception as e:
            res["graph_error"] = repr(e)[:400]
            torch.cuda.synchronize()
        return res
    except Exception as e:
        return {"error": repr(e)[:600]}


def bench_kv_head_sharded(args, ctx, one_gpu_ms_per_step):
    """ONE 128K sequence, its KV heads sharded over the ranks, outputs all-gathered (N > 1)."""
    torch = ctx.torch
    from dram_attention_b200.sharded import KVHeadShardedDRAMAttention, head_range
    from dram_attention_b200.synthetic import llama_layer_workload
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    K, W, NW = args.steps, max(args.warmup, 3), max(1, args.windows)
    n_sh = W + (NW + 1) * K + 4
    w0 = llama_layer_workload(seed=0, steps=n_sh, dram_tokens=args.dram_tokens, max_out=n_sh)
    hk_all, rep = w0.n_kv_heads, w0.n_q_heads // w0.n_kv_heads
    lo0, hi0 = head_range(hk_all, rank, world)
    ctor = w0.ctor_kwargs()
    ctor.pop("n_kv_heads")
    sh = KVHeadShardedDRAMAttention(n_kv_heads=hk_all, presliced=True, device=dev, dtype=w0.dtype,
                                    peer_gather=not args.library_gather, **ctor)
    sh.inner.init_cache(w0.k[:, :, lo0:hi0].to(dev), w0.v[:, :, lo0:hi0].to(dev))
    sq = w0.xq[:n_sh, :, :, lo0 * rep:hi0 * rep].contiguous().to(dev)
    sk = w0.xk[:n_sh, :, :, lo0:hi0].contiguous().to(dev)
    sv = w0.xv[:n_sh, :, :, lo0:hi0].contiguous().to(dev)
    S0 = w0.prefill_len
    for i in range(W):
        sh(sq[i], sk[i], sv[i], start_pos=S0 + i, stage="generate")
    torch.cuda.synchronize()
    sh.check_status()
    # the same windows of K consecutive steps as the one-GPU figure it is compared with
    win_us = []
    for wi in range(NW):
        first = W + wi * K
        ms, outs, up, _w, _g = time_graph(ctx, lambda: [sh(sq[first + i], sk[first + i], sv[first + i],
                                                           start_pos=S0 + first + i, stage="generate") for i in range(K)])
        (ms,) = ctx.max_over_ranks([ms])
        win_us.append(ms / K * 1e3)
        del outs, _g
    sh.check_status()
    # the same kind of steps once more with the device-side stamps: where a sharded step's time goes
    first = W + NW * K
    tr = StepTrace(ctx)
    g = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        outs_t = [sh(sq[first + i], sk[first + i], sv[first + i], start_pos=S0 + first + i, stage="generate")
                  for i in range(K)]
    ctx.barrier()
    with tr:
        g.replay()
    tl = tr.timeline()
    ctx.barrier()
    sh.check_status()
    del g, outs_t
    us = statistics.median(win_us)
    ms = us * K / 1e3
    us = ms / K * 1e3
    return {
        "what": f"ONE sequence, its {hk_all} KV heads sharded {world}-way, K steps in one graph per rank, max over ranks; "
                f"median of {NW} windows of K consecutive steps, the same windows as the one-GPU figure beside it",
        "value": K / (ms * 1e-3), "unit": "tok/s", "us_per_step": us, "us_per_step_by_window": win_us, "scaling": "strong",
        "one_gpu_us_per_step_same_run": one_gpu_ms_per_step * 1e3,
        "speedup_vs_one_gpu": one_gpu_ms_per_step * 1e3 / us,
        "efficiency_vs_one_gpu": one_gpu_ms_per_step * 1e3 / us / world,
        "gather": ("peer stores over NVLink (da_gather_heads)" if sh._peer is not None
                   else "NCCL all_gather_into_tensor"),
        "timeline_us_rank0": tl,
    }


# --------------------------------------------------------------------------------
# cfg4: batched decode, sequences dealt round-robin to the GPUs
# --------------------------------------------------------------------------------

def bench_cfg4(args, ctx):
    torch = ctx.torch
    import dram_attention_b200 as da
    from dram_attention_b200.synthetic import device_layer_inputs
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    n_seq, K4, W = args.cfg4_sequences, args.cfg4_steps, 3
    redraw = args.cfg4_redraw
    mine = list(range(rank, n_seq, world))
    hk, rep, D, page, lru, local, top_k, dram = 8, 4, 128, 16, 32768, 4096, 4096, 65536
    n_streams = max(1, min(args.cfg4_streams, max(len(range(r, n_seq, world)) for r in range(world))))
    steps = W + (2 * K4 if n_streams > 1 else K4)
    ops, inputs = [], []
    for sidx in mine:
        k, v, xq, xk, xv, _u, _ch = device_layer_inputs(dev, 1000 + sidx, steps, dram, n_kv_heads=hk, rep=rep,
                                                        local=local, page_size=page, needles=0, redraw_every=redraw)
        op = da.DRAMAttention(max_output_length=steps, lru_hbm_cache_size=lru, local_cache_size=local, page_size=page,
                              top_k=top_k, n_kv_heads=hk, head_dim=D, device=dev, dtype=torch.bfloat16)
        op.init_cache(k, v)
        del k, v
        ops.append(op)
        inputs.append((xq, xk, xv))
    S = dram + local - page
    for i in range(W):
        for op, (xq, xk, xv) in zip(ops, inputs):
            op(xq[i], xk[i], xv[i], start_pos=S + i, stage="generate")
    torch.cuda.synchronize()
    miss0 = sum(total_misses(op.lru_cache) for op in ops)
    redo0 = sum(op.lru_cache.evict_redo[2].sum().item() for op in ops)
    streams = [torch.cuda.Stream(device=dev) for _ in range(n_streams)] if n_streams > 1 else []

    def capture(first, last, use_streams):
        """Steps first .. last-1 of every sequence of this GPU, step by step; with streams, sequence j's steps go
        to stream j % n (the sequences are independent of each other)."""
        outs = []
        if use_streams and streams:
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            for st in streams:
                st.wait_event(fork)
        for i in range(first, last):
            for j, (op, (xq, xk, xv)) in enumerate(zip(ops, inputs)):
                if use_streams and streams:
                    with torch.cuda.stream(streams[j % n_streams]):
                        outs.append(op(xq[i], xk[i], xv[i], start_pos=S + i, stage="generate"))
                else:
                    outs.append(op(xq[i], xk[i], xv[i], start_pos=S + i, stage="generate"))
        if use_streams and streams:
            for st in streams:
                done = torch.cuda.Event()
                done.record(st)
                main.wait_event(done)
        return outs

    # the configuration's 128 steps over the streams; the same number of steps after them (as many re-draws)
    # on one stream, for comparison
    order = [(f"sequences_over_{n_streams}_streams" if n_streams > 1 else "sequences_on_one_stream", True, W, W + K4)]
    if n_streams > 1:
        order.append(("sequences_on_one_stream", False, W + K4, W + 2 * K4))
    by_schedule = {}
    misses_first = redos_first = 0.0
    for name, use_streams, a, b in order:
        if mine:
            ms, outs, up, _w, _g = time_graph(ctx, lambda: capture(a, b, use_streams))
            assert all(bool(torch.isfinite(o.float()).all()) for o in outs[-len(ops):])
            del outs, _g
        else:   # more GPUs than sequences: this rank only takes part in the barriers
            ctx.barrier()
            ctx.barrier()
            ms = 0.0
        (ms,) = ctx.max_over_ranks([ms])
        by_schedule[name] = ms
        if name == order[0][0]:
            misses_first = sum(total_misses(op.lru_cache) for op in ops) - miss0
            redos_first = sum(op.lru_cache.evict_redo[2].sum().item() for op in ops) - redo0
    best_name = order[0][0]          # the headline is the configuration's own 128 steps
    ms = by_schedule[best_name]
    for op in ops:
        op.check_status()
    misses, redos = ctx.sum_over_ranks([misses_first, redos_first])
    t_local = local - page + W + K4 // 2
    b_score, b_attn = layer_bytes(hk, rep, D, dram // page, lru // page, page, t_local)
    per_gpu_steps = max(len(range(r, n_seq, world)) for r in range(world)) * K4
    us_per_seq_step = ms * 1e3 / per_gpu_steps
    page_bytes = page * 2 * D * 2
    peak, kind = hbm_peak_gbs()
    redraw_steps = [i for i in range(W, W + K4) if redraw and i % redraw == 0]
    ach = (b_score + b_attn) / (us_per_seq_step * 1e-6) / 1e9
    return {
        "workload": f"batched decode: {n_seq} independent sequences x {dram}-token prefix, Llama-3-8B attention shape, "
                    f"bf16, {K4} timed steps per sequence after {W} warm-up steps, query drift N(0,0.05^2) per step and "
                    f"a re-draw from N(0,1) every {redraw} steps (steps {redraw_steps} of the timed region re-draw)",
        "metric": "decode tok/s, all sequences", "value": n_seq * K4 / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
        "scaling": "strong (fixed batch)", "parallelism": f"sequences dealt round-robin to {world} GPU(s), no collective",
        "ms_total": ms, "us_per_sequence_step": us_per_seq_step, "schedule": best_name,
        "ms_total_by_schedule": by_schedule,
        "roofline_step": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                          "frac_of_nominal_8tbs": ach / NOMINAL_HBM_GBS, "peak_kind": kind + " HBM copy bandwidth",
                          "algorithmic_bytes_per_sequence_step": b_score + b_attn,
                          "note": "includes the re-draw steps, which are bound by the host link, not by HBM"},
        "misses_per_sequence_step": misses / (n_seq * K4), "miss_bytes_total": misses * page_bytes,
        "steps_that_took_the_redo_path": redos,
        "timed_region": "one CUDA graph per rank holding every step of its sequences (step by step, the sequences dealt "
                        "to the streams of the schedule), uploaded, one replay; the one-stream schedule is timed on the "
                        "128 steps that follow (as many re-draws)",
        "data": "synthetic, generated on the device",
    }


# --------------------------------------------------------------------------------
# cfg5: 32-layer stack at a 1M-token prefix, KV heads sharded over the GPUs
# --------------------------------------------------------------------------------

def bench_cfg5(args, ctx):
    torch = ctx.torch
    import dram_attention_b200 as da
    from dram_attention_b200.sharded import KVHeadShardedDRAMAttention, head_range
    from dram_attention_b200.synthetic import device_layer_inputs, device_decode_inputs
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    L, K5, W = args.cfg5_layers, args.cfg5_steps, 3
    P = max(1, min(L, args.cfg5_prefixes))
    hk_all, rep, D, page, lru, local, top_k, dram = 8, 4, 128, 16, 65536, 8192, 8192, 1048576
    if hk_all % world:
        return {"skipped": f"{world} GPUs do not divide {hk_all} KV heads"}
    lo, hi = head_range(hk_all, rank, world)
    hk = hi - lo
    steps = W + K5 + 1
    t_setup = time.perf_counter()
    ctor = dict(max_output_length=steps, lru_hbm_cache_size=lru, local_cache_size=local, page_size=page,
                top_k=top_k, head_dim=D, device=dev, dtype=torch.bfloat16)

    def make_layer():
        if world == 1:
            op = da.DRAMAttention(n_kv_heads=hk_all, **ctor)
            return op, op
        op = KVHeadShardedDRAMAttention(n_kv_heads=hk_all, presliced=True, peer_gather=not args.library_gather, **ctor)
        return op, op.inner

    layers, inners, inputs, owners = [], [], [], []
    for l in range(L):
        op, inner = make_layer()
        if l < P:
            # this rank's KV heads of a prefix of its own (all ranks draw the same prefix, then slice)
            k, v, xq, xk, xv, u, ch = device_layer_inputs(dev, 5000 + l, steps, dram, n_kv_heads=hk_all, rep=rep,
                                                          local=local, page_size=page, needles=32)
            inner.init_cache(k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous())
            del k, v
            owners.append((inner, u, ch))
        else:
            src, u, ch = owners[l % P]
            inner.init_cache_sharing(src)
            xq, xk, xv = device_decode_inputs(dev, 6000 + l, steps, u, ch, hk_all, rep)
        inputs.append((xq[:, :, :, lo * rep:hi * rep].contiguous(), xk[:, :, :, lo:hi].contiguous(),
                       xv[:, :, :, lo:hi].contiguous()))
        layers.append(op)
        inners.append(inner)
        torch.cuda.empty_cache()
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup
    S = dram + local - page
    pinned_gib = P * hk * (dram // page) * page * 2 * D * 2 / 2 ** 30

    n_streams = args.cfg5_streams if args.cfg5_streams > 0 else {8: 2, 4: 4, 2: 4, 1: 8}[hk]
    streams = [torch.cuda.Stream(device=dev) for _ in range(n_streams)] if n_streams > 1 else []

    def token_step(i, overlap):
        """Every layer's generate step for token i.  The layers are independent here (synthetic q/k/v per
        layer), so with `overlap` they alternate over a few streams: the chain of layer l + 1 (scores ->
        page list -> LRU update) runs while layer l's attention streams."""
        outs = []
        if overlap and streams:
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            for s in streams:
                s.wait_event(fork)
            for l, (op, (xq, xk, xv)) in enumerate(zip(layers, inputs)):
                with torch.cuda.stream(streams[l % n_streams]):
                    outs.append(op(xq[i], xk[i], xv[i], start_pos=S + i, stage="generate"))
            for s in streams:
                done = torch.cuda.Event()
                done.record(s)
                main.wait_event(done)
        else:
            for op, (xq, xk, xv) in zip(layers, inputs):
                outs.append(op(xq[i], xk[i], xv[i], start_pos=S + i, stage="generate"))
        return outs

    def misses_now():
        return sum(total_misses(x.lru_cache) for x in inners)

    # every layer's peer gather sets itself up at its first use (an allocation, a rendezvous, a barrier):
    # that is construction, done here with a dummy block so that the cold step below times the step
    if world > 1:
        dummy = torch.zeros(1, 1, hk * rep, D, dtype=torch.bfloat16, device=dev)
        for op in layers:
            op.all_gather_heads(dummy)
        torch.cuda.synchronize()
    # cold start: the first token step finds only the warm start of the cache construction resident
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    miss0 = misses_now()
    ctx.barrier()
    ev0.record()
    token_step(0, False)
    ev1.record()
    ctx.barrier()
    (cold_ms,) = ctx.max_over_ranks([ev0.elapsed_time(ev1)])
    cold_misses = misses_now() - miss0
    for i in range(1, W):
        token_step(i, False)
    torch.cuda.synchronize()
    for op in layers:
        op.check_status()

    # K5 token steps, timed once with the layers in sequence and once alternating over the streams
    # (two disjoint halves of the steps, so that neither finds the other's pages resident)
    half = max(1, K5 // 2)
    results = {}
    order = [("layers_in_sequence", False, W, W + half)]
    if streams:
        order.append((f"layers_alternating_over_{n_streams}_streams", True, W + half, W + 2 * half))
    miss1 = misses_now()
    for name, overlap, a, b in order:
        ms, outs, up, _w, _g = time_graph(ctx, lambda: [token_step(i, overlap) for i in range(a, b)])
        (ms,) = ctx.max_over_ranks([ms])
        assert all(bool(torch.isfinite(o.float()).all()) for o in outs[-1])
        results[name] = ms / (b - a)
        del outs, _g
    timed_steps = sum(b - a for _n, _o, a, b in order)
    steady_misses = misses_now() - miss1
    redos = sum(x.lru_cache.evict_redo[2].sum().item() for x in inners)
    for op in layers:
        op.check_status()
    cold_misses, steady_misses, redos = ctx.sum_over_ranks([cold_misses, steady_misses, redos])
    best_name = min(results, key=results.get)
    ms_tok = results[best_name]
    b_score, b_attn = layer_bytes(hk_all, rep, D, dram // page, lru // page, page, local - page + W + K5 // 2)
    us_layer = ms_tok * 1e3 / L
    peak, kind = hbm_peak_gbs()
    page_bytes = page * 2 * D * 2
    ach = (b_score + b_attn) / world / (us_layer * 1e-6) / 1e9
    gather = "nothing (one GPU)"
    if world > 1:
        gather = ("peer stores over NVLink (da_gather_heads)" if getattr(layers[0], "_peer", None) is not None
                  else "the process group's all-gather")
    return {
        "workload": f"{L}-layer stack, 1,048,576-token prefix per layer in pinned DRAM, Llama-3-8B attention shape, bf16, "
                    f"lru_hbm_cache_size {lru}, local {local}, top_k {top_k}; synthetic q/k/v per layer (N(0,1), 8 outlier "
                    f"channels x10, 32 needle pages), projections omitted: the layers of a token step are independent",
        "metric": "decode tok/s through the whole stack", "value": 1e3 / ms_tok, "unit": "tok/s", "n_gpus": world,
        "scaling": "strong",
        "parallelism": f"{hk_all} KV heads sharded {world}-way, per-head outputs all-gathered per layer by {gather}",
        "layers": L, "timed_token_steps": timed_steps, "ms_per_token_step": ms_tok, "us_per_layer_step": us_layer,
        "ms_per_token_step_by_schedule": results, "schedule": best_name,
        "roofline_layer_step": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                                "frac_of_nominal_8tbs": ach / NOMINAL_HBM_GBS, "peak_kind": kind + " HBM copy bandwidth",
                                "algorithmic_bytes_per_layer_step_per_gpu": (b_score + b_attn) / world,
                                "floor_us_at_measured_peak": (b_score + b_attn) / world / peak / 1e3},
        "distinct_prefixes": P, "pinned_dram_gib_per_gpu": pinned_gib,
        "pinned_note": (f"{P} distinct synthetic prefixes of {4 / world:.2f} GiB per GPU, shared by the {L} layers (every "
                        f"layer has its own slot table, LRU state, local window and queries); {L} distinct prefixes "
                        f"would pin {L * 4 / world:.0f} GiB per GPU.  The bytes a layer step reads and the pages it misses "
                        "do not depend on the sharing."),
        "hbm_gib_per_gpu": (L * hk * (lru // page) * page_bytes + P * hk * (dram // page) * 2 * D * 2) / 2 ** 30,
        "cold_first_token_step": {"ms": cold_ms, "misses": cold_misses, "bytes": cold_misses * page_bytes,
                                  "host_link_gbs_all_gpus": cold_misses * page_bytes / (cold_ms * 1e-3) / 1e9},
        "steady_misses_per_layer_step": steady_misses / (timed_steps * L),
        "steady_miss_bytes_per_token_step": steady_misses * page_bytes / timed_steps,
        "layer_steps_that_took_the_redo_path": redos, "setup_s": setup_s,
        "timed_region": "all layers of the timed token steps in one CUDA graph per rank, uploaded, one replay, max over ranks",
        "data": "synthetic, generated on the device",
    }


# --------------------------------------------------------------------------------
# B200 arm
# --------------------------------------------------------------------------------

def run_b200(args):
    ctx = Ctx(args)
    torch, dist = ctx.torch, ctx.dist
    world, rank, dev = ctx.world, ctx.rank, ctx.dev

    if args.only_sweep:
        from dram_attention_b200.topk_selector import IPUpperboundTopKSelector
        gs = torch.Generator(device=dev).manual_seed(0)
        s_hk, s_rep, s_pg, n_pages, D = 8, 4, 16, 65536, 128
        mm = torch.empty(s_hk, n_pages, 2, D, dtype=torch.bfloat16, device=dev)
        for h in range(s_hk):
            keys = torch.randn(n_pages, s_pg, D, generator=gs, device=dev).to(torch.bfloat16)
            mm[h, :, 0], mm[h, :, 1] = torch.aminmax(keys, dim=1)
            del keys
        q_s = torch.randn(1, 1, s_hk * s_rep, D, generator=gs, device=dev).to(torch.bfloat16)
        sel = IPUpperboundTopKSelector(torch.empty(s_hk, n_pages * s_pg, D, dtype=torch.bfloat16, device="meta"), n_pages,
                                       device=dev, _summaries=mm)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        res = []
        for _ in range(3):
            ev[0].record()
            sel.score_(q_s, 256)
            ev[1].record()
            pl = sel.select_(1, s_rep, 256)
            ev[2].record()
            torch.cuda.synchronize()
            res.append((ev[0].elapsed_time(ev[1]) * 1e3, ev[1].elapsed_time(ev[2]) * 1e3))
        print(json.dumps({"pages": n_pages, "score_us": [r[0] for r in res], "topk_us": [r[1] for r in res],
                          "first_pages_of_head_0": pl[0, :4].tolist()}), file=RESULT_OUT, flush=True)
        return

    if args.only_prefill:
        import dram_attention_b200 as da
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

    ctx.sampler.start()
    extras = not args.no_extras
    line = None

    def guarded(fn):
        """An extra must not take the headline down with it."""
        try:
            return fn(args, ctx)
        except Exception as e:
            import traceback
            traceback.print_exc()
            return {"error": repr(e)}

    if args.config == "cfg2":
        r = bench_cfg2(args, ctx)
        w, K, W = r["w"], r["K"], r["W"]
        by_seq, n_seq = r["by_seq"], r["n_seq"]
        ms_value, ms_e2e = r["ms_value"], r["ms_e2e"]
        more = {}
        if extras and world == 1:
            more.update(cfg2_extras(args, ctx, r))
        if args.reference_gpu and world == 1:
            more["reference_gpu"] = bench_reference_gpu(args, ctx, w)
        # free the 128K layer before the other configurations are built
        for key in ("op", "inner", "dq", "dk", "dv", "launch_us"):
            r.pop(key, None)
        torch.cuda.empty_cache()
        sharded = bench_kv_head_sharded(args, ctx, ms_value / K) if by_seq else None
        torch.cuda.empty_cache()
        cfg4 = cfg5 = None
        if extras:
            cfg4 = guarded(bench_cfg4)
            torch.cuda.empty_cache()
            cfg5 = guarded(bench_cfg5)
            torch.cuda.empty_cache()
        if rank == 0:
            win_us = [m / K * 1e3 for m in r["win_ms"]]
            mhz = [m for m in r["win_mhz"] if m]
            line = {
                "metric": METRIC, "value": n_seq * K / (ms_value * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": K, "warmup": W, "ms_per_step": ms_value / K, "higher_is_better": True,
                "scaling": ("weak" if (world == 1 or by_seq) else "strong"), "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic",
                "config": cfg2_config(w),
                "parallelism": ("single GPU" if world == 1 else
                                f"{world} independent sequences, one per GPU, no collective on the path" if by_seq else
                                f"KV heads sharded {world}-way, all-gather of per-head outputs"),
                "timed_region": ("one CUDA graph of K steps, " + ("uploaded to the device" if r["uploaded"] else
                                                                   "launched behind a spin kernel") +
                                 f" before the first event; {len(win_us)} disjoint windows of K consecutive steps, the "
                                 "median one is the headline"),
                "windows": {"us_per_step": win_us, "median": statistics.median(win_us), "min": min(win_us),
                            "max": max(win_us), "first_step_of_window": r["win_first"],
                            "sm_mhz_median_per_window": r["win_mhz"],
                            "us_x_ghz_median": (statistics.median(win_us) * statistics.median(mhz) / 1e3) if mhz else None,
                            "note": "window i covers generate steps first_step .. first_step + K - 1 after the prefill; "
                                    "the first windows lie inside the 64 steps the configuration names, later ones "
                                    "find a slot table that has settled on the query stream"},
                "clocks": ctx.sampler.summary(ctx.windows),
                "e2e": {"value": n_seq * K / (ms_e2e * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": r["h2d"],
                        "d2h_bytes_per_step": r["d2h"], "ms_per_step": ms_e2e / K,
                        "per_step": "host writes q|k|v into a pinned staging buffer; one graph replay = H2D copy, the "
                                    "step, D2H copy of the output; stream sync"},
                "gpu_launches": 5 * K * world,
                "step_layout": "{score -> top-k -> LRU update (+ copy of the few missed pages) -> attention phase 2} || "
                               "attention phase 1; the CTA that finishes last merges",
                "misses_per_step": r["misses_per_step"], "steps_that_took_the_redo_path": r["redo_steps"],
                "timeline_us": r["timeline"],
                "kv_head_sharded": sharded,
                "cfg4": cfg4, "cfg5": cfg5,
            }
            line.update(r["roof"])
            line.update(more)
            if world == 1 and not args.no_cpu_baseline:
                tps, done, threads = cpu_reference_steps(w, 1, min(32, w.steps - 1), budget_s=15.0)
                line["cpu_baseline"] = {
                    "value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                    "sample": f"{done} full generate steps of the same layer (1 warm-up) on the host cores: CPU port "
                              "of the reference's pure-PyTorch path, float32 scores and attention"}
    else:
        res = bench_cfg4(args, ctx) if args.config == "cfg4" else bench_cfg5(args, ctx)
        if rank == 0:
            line = {
                "metric": res.get("metric"), "value": res.get("value"), "unit": "tok/s", "n_gpus": world,
                "steps": args.cfg4_steps if args.config == "cfg4" else res.get("timed_token_steps"), "warmup": 3,
                "ms_per_step": (res.get("us_per_sequence_step", 0) / 1e3 if args.config == "cfg4"
                                else res.get("ms_per_token_step")),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": res.get("workload")}, "clocks": ctx.sampler.summary(ctx.windows),
                "detail": res,
            }
    ctx.sampler.stop()
    if rank == 0 and line is not None:
        print(json.dumps(line), file=RESULT_OUT, flush=True)
    if world > 1:
        # Leave in step: every rank is done with its kernels and gathers before anybody exits, and the
        # process group goes down in an orderly way (no multicast binding was ever made: NVLS is off).
        ctx.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        try:
            dist.destroy_process_group()
        except Exception:
            pass
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

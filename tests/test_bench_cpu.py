"""CPU-side checks of bench.py's arithmetic: the algorithmic bytes the rooflines divide by, the
roofline object, and the command line (no GPU, no timing)."""

import importlib.util
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_algorithmic_bytes_of_the_llama_layer():
    """B_score = Hk L 2 D e + Hq D e, B_attn = Hk (Nh P + T + 1) 2 D e + 2 Hq D e: config 2 with T = 4200
    local tokens is 33.56 MB + 151.6 MB, the figures the design document quotes."""
    b = _bench()
    b_score, b_attn = b.layer_bytes(8, 4, 128, 8192, 2048, 16, 4200)
    assert b_score == 8 * 8192 * 2 * 128 * 2 + 32 * 128 * 2 == 33_562_624
    assert b_attn == 8 * (2048 * 16 + 4200 + 1) * 2 * 128 * 2 + 2 * 32 * 128 * 2
    assert abs(b_attn / 1e6 - 151.45) < 0.1
    # config 5, one layer: 65536 pages, 4096 slots, local 8192
    s5, a5 = b.layer_bytes(8, 4, 128, 65536, 4096, 16, 8192)
    assert abs((s5 + a5) / 1e6 - 570) < 3


def test_roofline_object_divides_by_the_peak_it_names():
    b = _bench()
    r = b.roofline_obj("k", 147_349_504, 31.6)
    peak, kind = b.hbm_peak_gbs()
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["peak"] == peak and kind in r["peak_kind"]
    assert abs(r["achieved"] - 147_349_504 / 31.6e-6 / 1e9) < 1e-6
    assert abs(r["frac"] - r["achieved"] / peak) < 1e-12
    assert abs(r["frac_of_nominal_8tbs"] - r["achieved"] / 8000.0) < 1e-9
    assert b.roofline_obj("k", 1, 0) is None


def test_command_line_defaults():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--config", "--windows", "--shard"):
        assert flag in out.stdout
    b = _bench()
    argv = sys.argv
    try:
        sys.argv = ["bench.py"]
        a = b.parse_args()
    finally:
        sys.argv = argv
    assert a.gpus == 1 and a.steps == 20 and a.warmup >= 3 and a.settle_steps == 0 and a.windows == 5
    assert a.config == "cfg2" and a.impl != "reference"

"""Host-side logic of the KV-head sharding, on two gloo ranks (no GPU): head
ranges, input slicing, the all-gather that reassembles (1, s, Hq, D), and a rank that
leaves between two steps."""

import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dram_attention_b200.sharded import KVHeadShardedDRAMAttention, head_range


def test_head_ranges():
    assert [head_range(8, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert head_range(8, 0, 1) == (0, 8)
    with pytest.raises(ValueError):
        head_range(8, 0, 3)
    with pytest.raises(ValueError):
        head_range(8, 4, 4)


class FakeOperator(torch.nn.Module):
    """Stands in for DRAMAttention: output = query + (sum of its KV head's new key)."""

    def __init__(self, n_kv_heads, **kw):
        super().__init__()
        self.n_kv_heads = n_kv_heads
        self.kw = kw
        self.seen_cache = None

    def init_cache(self, k, v):
        self.seen_cache = (k.clone(), v.clone())

    def forward(self, xq, xk, xv, *, start_pos, stage):
        rep = xq.shape[2] // self.n_kv_heads
        return xq + xk.sum(-1, keepdim=True).repeat_interleave(rep, dim=2) + float(start_pos)


def _worker(rank, world, port, seq):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        hk, rep, d = 4, 2, 8
        xq = torch.randn(1, seq, hk * rep, d, generator=g)
        xk = torch.randn(1, seq, hk, d, generator=g)
        xv = torch.randn(1, seq, hk, d, generator=g)
        kc = torch.randn(1, 32, hk, d, generator=g)
        op = KVHeadShardedDRAMAttention(n_kv_heads=hk, operator_factory=FakeOperator, page_size=16)
        assert (op.lo, op.hi) == (rank * 2, rank * 2 + 2) and op.inner.kw == {"page_size": 16}
        op.init_cache(kc, kc + 1)
        assert torch.equal(op.inner.seen_cache[0], kc[:, :, op.lo:op.hi])
        out = op(xq, xk, xv, start_pos=5, stage="generate")
        full = FakeOperator(hk)(xq, xk, xv, start_pos=5, stage="generate")
        assert out.shape == full.shape and torch.equal(out, full)
        # pre-sliced inputs give the same result
        op2 = KVHeadShardedDRAMAttention(n_kv_heads=hk, operator_factory=FakeOperator, presliced=True)
        out2 = op2(xq[:, :, op.lo * rep:op.hi * rep], xk[:, :, op.lo:op.hi], xv[:, :, op.lo:op.hi],
                   start_pos=5, stage="generate")
        assert torch.equal(out2, full)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq", [1, 3])
def test_two_rank_gather_reassembles_heads(seq):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, seq), nprocs=2, join=True)


def _leaver(rank, world, port, result_dir):
    """Rank 1 leaves after the first step (between steps, nothing of its own in flight); rank 0's
    next step must come back with an error within the process group's time-out, not wait for ever."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    hk, rep, d = 4, 2, 8
    g = torch.Generator().manual_seed(1)
    xq, xk, xv = torch.randn(1, 1, hk * rep, d, generator=g), torch.randn(1, 1, hk, d, generator=g), \
        torch.randn(1, 1, hk, d, generator=g)
    op = KVHeadShardedDRAMAttention(n_kv_heads=hk, operator_factory=FakeOperator)
    out = op(xq, xk, xv, start_pos=1, stage="generate")
    assert torch.equal(out, FakeOperator(hk)(xq, xk, xv, start_pos=1, stage="generate"))
    if rank == 1:
        os._exit(0)          # gone: no further call, no goodbye
    t0 = time.monotonic()
    try:
        op(xq, xk, xv, start_pos=2, stage="generate")
        verdict = "no error"
    except Exception as e:   # a closed connection or the group's time-out, depending on who notices first
        verdict = "error after %.1f s: %s" % (time.monotonic() - t0, type(e).__name__)
    with open(os.path.join(result_dir, "rank0.txt"), "w") as f:
        f.write(verdict)
    os._exit(0)


def test_rank_that_leaves_between_steps_is_an_error_not_a_hang(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    t0 = time.monotonic()
    mp.spawn(_leaver, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert time.monotonic() - t0 < 60
    verdict = (tmp_path / "rank0.txt").read_text()
    assert verdict.startswith("error after"), verdict

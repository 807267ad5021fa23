"""Run under torchrun with one rank per GPU (tests/test_multi_gpu.py launches it when the
machine has at least two GPUs): the peer-memory all-gather of the sharded operator against
the process group's all-gather, eagerly and inside a CUDA graph, and the sharded operator
against the single-GPU operator on the same inputs."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def close(a, b):
    """bf16 outputs of two different split-K partitions of the same attention (the number of
    splits follows the KV heads per GPU): 2e-2 absolute plus half a unit in the last place."""
    a, b = a.float(), b.float()
    return bool(((a - b).abs() <= 2e-2 + b.abs() * 2.0 ** -8).all())


def main():
    import dram_attention_b200 as da
    from dram_attention_b200.sharded import KVHeadShardedDRAMAttention
    from dram_attention_b200.synthetic import llama_layer_workload

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")        # nothing bound to an NVLink multicast object at exit
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    dist.init_process_group("nccl", device_id=dev)

    steps = 6
    w = llama_layer_workload(seed=0, steps=steps + 4, dram_tokens=16384, lru=4096, local=512, top_k=1024,
                             needles=4)
    kw = w.ctor_kwargs()
    hk = kw.pop("n_kv_heads")
    ops = {name: KVHeadShardedDRAMAttention(n_kv_heads=hk, device=dev, dtype=w.dtype, peer_gather=flag, **kw)
           for name, flag in (("peer", True), ("nccl", False))}
    single = da.DRAMAttention(n_kv_heads=hk, device=dev, dtype=w.dtype, **kw)
    k, v = w.k.to(dev), w.v.to(dev)
    for op in list(ops.values()) + [single]:
        op.init_cache(k, v)
    s0 = w.prefill_len
    for i in range(steps):
        args = (w.xq[i].to(dev), w.xk[i].to(dev), w.xv[i].to(dev))
        outs = {name: op(*args, start_pos=s0 + i, stage="generate") for name, op in ops.items()}
        ref = single(*args, start_pos=s0 + i, stage="generate")
        assert ops["peer"]._peer is not None, f"peer gather not in use: {ops['peer']._peer_failed}"
        assert torch.equal(outs["peer"], outs["nccl"]), f"step {i}: peer gather differs from the library gather"
        assert close(outs["peer"], ref), f"step {i}: sharded output differs from the single-GPU operator"
    # the same step inside a CUDA graph, replayed
    i = steps
    args = (w.xq[i].to(dev), w.xk[i].to(dev), w.xv[i].to(dev))
    pos = torch.tensor([s0 + i], dtype=torch.int32, device=dev)
    ref = single(*args, start_pos=s0 + i, stage="generate")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = ops["peer"](*args, start_pos=pos, stage="generate")
    graph.replay()
    torch.cuda.synchronize()
    assert close(got, ref), "captured step differs"
    first = got.clone()
    graph.replay()      # same position again: re-appends the same token, same result
    torch.cuda.synchronize()
    assert torch.equal(got, first), "replayed step differs"
    for op in ops.values():
        op.check_status()
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_GATHER_OK", world, flush=True)
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)     # the captured graph still references the communicator: leave without tearing it down


if __name__ == "__main__":
    main()

"""KV-cache files in the reference's per-layer format (examples/long-qa-chat/model.py:206-221,
chat.py:214-233): round trip, head slicing for sharded loading, and operators built from files."""

import pytest
import torch

from dram_attention_b200 import kv_files


class _Recorder:
    """Stands in for the operator: keeps what init_cache was given."""

    def __init__(self):
        self.k = self.v = None

    def init_cache(self, k, v):
        self.k, self.v = k.clone(), v.clone()


def _kv(seed, s=96, hk=4, d=8, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(1, s, hk, d, generator=g).to(dtype), torch.randn(1, s, hk, d, generator=g).to(dtype))


def test_round_trip_and_names(tmp_path):
    k, v = _kv(0)
    path = kv_files.save_layer_cache(str(tmp_path), 3, k, v)
    assert path.endswith("03_cache.pth")
    blob = torch.load(path, weights_only=True)          # readable the way the reference reads it
    assert set(blob) == {"cache_k", "cache_v"} and torch.equal(blob["cache_k"], k)
    k2, v2 = kv_files.load_layer_cache(str(tmp_path), 3)
    assert torch.equal(k2, k) and torch.equal(v2, v) and k2.dtype == torch.bfloat16


def test_head_slice_and_errors(tmp_path):
    k, v = _kv(1)
    kv_files.save_layer_cache(str(tmp_path), 0, k, v)
    k2, v2 = kv_files.load_layer_cache(str(tmp_path), 0, heads=(1, 3))
    assert torch.equal(k2, k[:, :, 1:3]) and torch.equal(v2, v[:, :, 1:3])
    with pytest.raises(ValueError):
        kv_files.load_layer_cache(str(tmp_path), 0, heads=(2, 9))
    with pytest.raises(FileNotFoundError):
        kv_files.load_layer_cache(str(tmp_path), 1)
    torch.save({"cache_k": k}, kv_files.layer_cache_path(str(tmp_path), 1))
    with pytest.raises(KeyError):
        kv_files.load_layer_cache(str(tmp_path), 1)
    with pytest.raises(AssertionError):
        kv_files.save_layer_cache(str(tmp_path), 2, k[0], v[0])


@pytest.mark.parametrize("world", [1, 2, 4])
def test_attach_gives_every_rank_its_heads(tmp_path, world):
    layers = [_kv(10 + i) for i in range(3)]
    for i, (k, v) in enumerate(layers):
        kv_files.save_layer_cache(str(tmp_path), i, k, v)
    assert kv_files.count_layer_caches(str(tmp_path)) == 3
    for rank in range(world):
        ops, cache_len = kv_files.attach_layer_caches(str(tmp_path), lambda layer: _Recorder(),
                                                      rank=rank, world_size=world)
        assert cache_len == 96 and len(ops) == 3
        per = 4 // world
        for (k, v), op in zip(layers, ops):
            assert torch.equal(op.k, k[:, :, rank * per:(rank + 1) * per])
            assert torch.equal(op.v, v[:, :, rank * per:(rank + 1) * per])


def test_attach_rejects_ragged_layers(tmp_path):
    kv_files.save_layer_cache(str(tmp_path), 0, *_kv(0, s=96))
    kv_files.save_layer_cache(str(tmp_path), 1, *_kv(1, s=80))
    with pytest.raises(ValueError):
        kv_files.attach_layer_caches(str(tmp_path), lambda layer: _Recorder())
    with pytest.raises(FileNotFoundError):
        kv_files.attach_layer_caches(str(tmp_path / "empty"), lambda layer: _Recorder())


@pytest.mark.gpu
def test_operator_from_files_equals_operator_from_tensors(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dram_attention_b200 as da
    from dram_attention_b200.synthetic import plumbing_workload
    w = plumbing_workload(seed=0, steps=3)
    kw = w.ctor_kwargs()
    for layer in range(2):
        kv_files.save_layer_cache(str(tmp_path), layer, w.k.flip(1) if layer else w.k, w.v)
    ops, cache_len = kv_files.attach_layer_caches(
        str(tmp_path), lambda layer: da.DRAMAttention(device="cuda", dtype=w.dtype, **kw))
    assert cache_len == w.k.shape[1]
    direct = da.DRAMAttention(device="cuda", dtype=w.dtype, **kw)
    direct.init_cache(w.k.cuda(), w.v.cuda())
    for i in range(3):
        args = (w.xq[i].cuda(), w.xk[i].cuda(), w.xv[i].cuda())
        a = ops[0](*args, start_pos=cache_len + i, stage="generate")
        b = direct(*args, start_pos=cache_len + i, stage="generate")
        assert torch.equal(a, b)
        assert torch.isfinite(ops[1](*args, start_pos=cache_len + i, stage="generate")).all()
    for op in ops:
        op.check_status()

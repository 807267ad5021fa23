"""Per-layer KV-cache files: the format the reference's chat example writes after a
prefill and reads back before decoding (examples/long-qa-chat/model.py:206-221,
examples/long-qa-chat/chat.py:214-233).

One file per layer, `NN_cache.pth` (NN = two-digit layer index), a `torch.save`d dict
{"cache_k": (1, S, Hk, D), "cache_v": (1, S, Hk, D)} of CPU tensors, keys already rotated.

The reference loads every file whole onto the GPU before `init_cache`.  Here the file is
memory-mapped, the KV heads of this rank are sliced out first (KV-head sharding), and only
that slice travels to the device, where one pass builds the pinned DRAM pages, the page
summaries and the warm-start slots.
"""

from __future__ import annotations

import os
from typing import Callable, List, Optional, Tuple

import torch

CACHE_FILE = "{index:02d}_cache.pth"


def layer_cache_path(cache_dir: str, index: int) -> str:
    return os.path.join(cache_dir, CACHE_FILE.format(index=index))


def save_layer_cache(cache_dir: str, index: int, xk: torch.Tensor, xv: torch.Tensor) -> str:
    """Write one layer's prefill keys/values (1, S, Hk, D) in the reference's format."""
    assert xk.dim() == 4 and xk.shape == xv.shape and xk.shape[0] == 1, "expects (1, S, Hk, D) tensors"
    os.makedirs(cache_dir, exist_ok=True)
    path = layer_cache_path(cache_dir, index)
    torch.save({"cache_k": xk.detach().to("cpu"), "cache_v": xv.detach().to("cpu")}, path)
    return path


def load_layer_cache(cache_dir: str, index: int, heads: Optional[Tuple[int, int]] = None,
                     mmap: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """(cache_k, cache_v) of one layer as CPU tensors (1, S, Hk', D).  With `heads` =
    (lo, hi) only those KV heads are returned (a view of the mapped file: nothing else is
    read from disk)."""
    path = layer_cache_path(cache_dir, index)
    if not os.path.exists(path):
        raise FileNotFoundError(f"no KV cache file for layer {index}: {path}")
    blob = torch.load(path, map_location="cpu", mmap=mmap, weights_only=True)
    for name in ("cache_k", "cache_v"):
        if name not in blob:
            raise KeyError(f"{path}: missing '{name}'")
    k, v = blob["cache_k"], blob["cache_v"]
    if k.dim() != 4 or k.shape != v.shape or k.shape[0] != 1:
        raise ValueError(f"{path}: expected two (1, S, Hk, D) tensors, got {tuple(k.shape)} / {tuple(v.shape)}")
    if heads is not None:
        lo, hi = heads
        if not (0 <= lo < hi <= k.shape[2]):
            raise ValueError(f"head range {heads} outside 0..{k.shape[2]}")
        k, v = k[:, :, lo:hi], v[:, :, lo:hi]
    return k, v


def count_layer_caches(cache_dir: str) -> int:
    """Number of consecutive layer files 00_cache.pth, 01_cache.pth, ... present."""
    n = 0
    while os.path.exists(layer_cache_path(cache_dir, n)):
        n += 1
    return n


def attach_layer_caches(cache_dir: str, make_operator: Callable[[int], "torch.nn.Module"],
                        n_layers: Optional[int] = None, rank: int = 0, world_size: int = 1,
                        n_kv_heads: Optional[int] = None) -> Tuple[List["torch.nn.Module"], int]:
    """Build one operator per layer from the files of `cache_dir`, as the chat example does
    before it captures its decode graph.  `make_operator(layer)` returns a fresh
    DRAMAttention (or KVHeadShardedDRAMAttention built with presliced=True) for that layer;
    with world_size > 1 every rank loads only its own KV heads.  Returns (operators,
    cache_len) with cache_len = S, the position of the first generated token."""
    from .sharded import head_range
    if n_layers is None:
        n_layers = count_layer_caches(cache_dir)
    if n_layers < 1:
        raise FileNotFoundError(f"no layer cache files in {cache_dir}")
    ops, cache_len = [], None
    for layer in range(n_layers):
        heads = None
        if world_size > 1:
            if n_kv_heads is None:
                probe_k, _ = load_layer_cache(cache_dir, layer)
                n_kv_heads = probe_k.shape[2]
            heads = head_range(n_kv_heads, rank, world_size)
        k, v = load_layer_cache(cache_dir, layer, heads=heads)
        if cache_len is None:
            cache_len = k.shape[1]
        elif k.shape[1] != cache_len:
            raise ValueError(f"layer {layer} holds {k.shape[1]} tokens, layer 0 holds {cache_len}")
        op = make_operator(layer)
        op.init_cache(k, v)
        ops.append(op)
        del k, v
    return ops, cache_len

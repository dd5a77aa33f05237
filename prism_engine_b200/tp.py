"""Tensor-parallel sharding plan for the palettized linears (host side).

Column-parallel tensors (q, k, v, gate, up, lm_head) are split by output rows
-- a row's palette travels with it.  Row-parallel tensors (o, down) are split
by input columns in units of 32 (one 16-byte index chunk at 4 bit) and every
rank keeps the full palette of every row; their partial sums are all-reduced
in fp32 before the fp16 rounding.  The reference has no tensor parallelism;
these helpers define the shard geometry both the CUDA engine and the tests use.
"""
from __future__ import annotations

from typing import Dict, Tuple

import numpy as np


def split_units(total_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Balanced contiguous split of ``total_units`` items; returns [u0, u1)."""
    return total_units * rank // world, total_units * (rank + 1) // world


def shard_plan(cfg: dict, world: int, rank: int) -> Dict[str, Tuple[int, int, int, int]]:
    """role -> (row0, rows, col0, cols) of this rank's shard of each layer tensor."""
    H, hd = cfg["hidden_size"], cfg["head_dim"]
    nh, nkv, I, V = cfg["num_heads"], cfg["num_kv_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    if nh % world or nkv % world:
        raise ValueError("tensor parallel degree must divide the head counts")
    nh_l, nkv_l = nh // world, nkv // world
    u0, u1 = split_units(I // 32, world, rank)
    i0, il = u0 * 32, (u1 - u0) * 32
    w0, w1 = split_units((V + 31) // 32, world, rank)
    v0, vl = w0 * 32, min(V, w1 * 32) - w0 * 32
    return {
        "q": (rank * nh_l * hd, nh_l * hd, 0, H),
        "k": (rank * nkv_l * hd, nkv_l * hd, 0, H),
        "v": (rank * nkv_l * hd, nkv_l * hd, 0, H),
        "o": (0, H, rank * nh_l * hd, nh_l * hd),
        "gate": (i0, il, 0, H),
        "up": (i0, il, 0, H),
        "down": (0, H, i0, il),
        "lm_head": (v0, vl, 0, H),
    }


def slice_payload(payload: np.ndarray, dim_m: int, dim_n: int, bits: int, row0: int, rows: int, col0: int,
                  cols: int) -> np.ndarray:
    """The reference-format payload of rows [row0,row0+rows) x columns [col0,col0+cols)."""
    n_ent = 1 << bits
    per_byte = 8 // bits
    assert col0 % per_byte == 0 and cols % per_byte == 0
    pal = payload[: dim_m * n_ent * 2].reshape(dim_m, n_ent * 2)
    idx = payload[dim_m * n_ent * 2: dim_m * n_ent * 2 + dim_m * (dim_n // per_byte)].reshape(dim_m, dim_n // per_byte)
    return np.concatenate([pal[row0:row0 + rows].reshape(-1),
                           idx[row0:row0 + rows, col0 // per_byte:(col0 + cols) // per_byte].reshape(-1)])


def exchange_unique_id(make_id, group=None) -> bytes:
    """Rank 0 creates the NCCL unique id (``make_id()``), every rank receives it through
    ``torch.distributed`` (any backend: gloo on CPU, nccl on GPU)."""
    import torch
    import torch.distributed as dist

    rank = dist.get_rank(group)
    box = [make_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0, group=group)
    assert isinstance(box[0], (bytes, bytearray)) and len(box[0]) == 128
    return bytes(box[0])

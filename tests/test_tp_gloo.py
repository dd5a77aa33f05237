"""Tensor-parallel host logic on CPU: world_size-2 gloo ranks.

Each rank takes its shard of a column-parallel and a row-parallel palettized
tensor, computes with the CPU oracle, and the exchange step (fp32 all-reduce /
gather) reproduces the unsharded result.  Also exercises the unique-id
exchange the NCCL bootstrap uses.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from oracle import oracle as orc
    from prism_engine_b200 import synth, tp

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = dict(hidden_size=128, head_dim=32, num_heads=4, num_kv_heads=2, intermediate_size=352, vocab_size=1000)
        plan = tp.shard_plan(cfg, world, rank)
        H, I = cfg["hidden_size"], cfg["intermediate_size"]
        # unique id travels rank0 -> all
        uid = tp.exchange_unique_id(lambda: bytes(range(128)))
        assert uid == bytes(range(128))
        x = synth.make_activation(H, seed=5)
        wg = synth.make_payload(I, H, seed=11)
        wd = synth.make_payload(H, I, seed=12)
        # column-parallel gate: rows of the result are this rank's slice
        r0, rows, c0, cols = plan["gate"]
        assert rows % 32 == 0 and c0 == 0 and cols == H
        g_local = orc.lut_gemv(x, tp.slice_payload(wg, I, H, 4, r0, rows, c0, cols), rows, H)
        g_full = orc.lut_gemv(x, wg, I, H)
        assert np.array_equal(g_local, g_full[r0:r0 + rows])
        # row-parallel down over the local activation slice: fp32 partials, all-reduce, then round
        d0, drows, dc0, dcols = plan["down"]
        assert (dc0, dcols) == (r0, rows) and d0 == 0 and drows == H
        shard = tp.slice_payload(wd, H, I, 4, 0, H, dc0, dcols)
        W = orc.f16_vals(orc.dequant(shard, H, dcols)).astype(np.float32)
        part = torch.from_numpy(W @ orc.f16_vals(g_full[dc0:dc0 + dcols]).astype(np.float32))
        dist.all_reduce(part)
        full = orc.f16_vals(orc.lut_gemv(g_full, wd, H, I))
        got = part.numpy().astype(np.float16).astype(np.float32)
        rel = np.linalg.norm(got - full) / np.linalg.norm(full)
        assert rel < 1e-3, rel
        # shards tile the tensor exactly
        spans = [None] * world
        dist.all_gather_object(spans, (r0, rows))
        assert spans[0][0] == 0 and sum(s[1] for s in spans) == I
        assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_sharded_linears():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def test_shard_plan_72b():
    from prism_engine_b200 import QWEN25_72B, tp

    for world in (1, 2, 4, 8):
        tot_i = tot_v = 0
        for r in range(world):
            p = tp.shard_plan(QWEN25_72B, world, r)
            assert p["gate"][1] % 32 == 0 and p["down"][3] == p["gate"][1] and p["down"][2] == p["gate"][0]
            assert p["o"][3] == 8192 // world and p["o"][2] % 32 == 0
            assert p["k"][1] == 1024 // world
            tot_i += p["gate"][1]
            tot_v += p["lm_head"][1]
        assert tot_i == 29568 and tot_v == 152064

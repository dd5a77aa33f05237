"""Tensor-parallel decode on two GPUs against the single-GPU engine (skipped on a one-GPU box).

Each rank generates its shard of the same seeded weights; column/row-sharded linears with an fp32
all-reduce (the peer-memory kernel, and ncclAllReduce with the peer path switched off) must
reproduce the single-GPU greedy tokens (the only difference is the order in which the fp32 partial
sums of o_proj / down_proj are added).
"""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = dict(num_layers=3, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=352,
           vocab_size=1024, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)


def _worker(rank, world, port, q, peer_ar):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist

    import prism_engine_b200 as p
    from prism_engine_b200 import synth, tp

    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        be = p.CudaBackend(device=rank)
        be.tp_init(world, rank, tp.exchange_unique_id(p.CudaBackend.tp_unique_id))
        be.set_option("tp_peer_ar", peer_ar)
        peer = be.tp_peer_ready()
        eng = p.PrismEngine(be, p.model_config(**CFG, max_seq=64, max_batch=2, profile="baseline"))
        eng.synth_weights(seed=21)
        prompts = np.stack([synth.make_prompt(7, CFG["vocab_size"], seed=s) for s in (1, 2)])
        got = eng.generate(prompts, 24)
        eng.close()
        be.close()
        if rank == 0:
            ref_be = p.CudaBackend(device=0)
            ref = p.PrismEngine(ref_be, p.model_config(**CFG, max_seq=64, max_batch=2, profile="baseline"))
            ref.synth_weights(seed=21)
            want = ref.generate(prompts, 24)
            ref.close()
            ref_be.close()
            q.put((rank, "ok" if np.array_equal(got, want) else f"tokens differ: {got.tolist()} vs {want.tolist()}", peer))
        else:
            q.put((rank, "ok", peer))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e), False))


@pytest.mark.timeout(600)
@pytest.mark.parametrize("peer_ar", [1, 0])
def test_tp2_matches_single_gpu(peer_ar):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000 + peer_ar
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, peer_ar)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = [q.get(timeout=500) for _ in procs]
    for pr in procs:
        pr.join(60)
    assert sorted(r[:2] for r in res) == [(0, "ok"), (1, "ok")], res
    # both ranks agree on whether peer memory could be mapped; on an NVLink box it can
    assert len({r[2] for r in res}) == 1, res
    print("peer-memory all-reduce set up:", res[0][2], "used:", bool(peer_ar) and res[0][2])

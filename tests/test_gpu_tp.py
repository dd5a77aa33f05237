"""Tensor-parallel decode on two GPUs against the single-GPU engine AND the CPU oracle (skipped on a
one-GPU box), and the bounded wait of the peer-memory all-reduce running out (one GPU is enough).

Each rank generates its shard of the same seeded weights; column/row-sharded linears with an fp32
all-reduce (the peer-memory kernel, and ncclAllReduce with the peer path switched off) must
reproduce the greedy tokens of the oracle's PrismEngine twin and of the single-GPU engine (the only
difference is the order in which the fp32 partial sums of o_proj / down_proj are added).  Run on a toy
model and on a 2-layer model at the 72B benchmark's widths.
"""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = dict(num_layers=3, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=352,
           vocab_size=1024, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)


WIDE = dict(num_layers=2, hidden_size=8192, num_heads=64, num_kv_heads=8, head_dim=128, intermediate_size=29568,
            vocab_size=152064, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)


def _worker(rank, world, port, q, peer_ar, wide=False, batch=2, fused=1):
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
        be.set_option("tp_fused_ar", fused)
        peer = be.tp_peer_ready()
        cfg = WIDE if wide else CFG
        max_seq, n_new = (512, 33) if wide else (64, 33)
        eng = p.PrismEngine(be, p.model_config(**cfg, max_seq=max_seq, max_batch=2, profile="baseline"))
        eng.synth_weights(seed=21)
        # one sequence: the row-parallel matmuls all-reduce inside the GEMV kernel; two: through the stand-alone kernel
        prompts = np.stack([synth.make_prompt(7, cfg["vocab_size"], seed=s) for s in (1, 2)[:batch]])
        got = eng.generate(prompts, n_new)
        eng.close()
        be.close()
        if rank == 0:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            from oracle import oracle as orc
            from test_gpu_engine import oracle_twin

            ref_be = p.CudaBackend(device=0)
            mc = p.model_config(**cfg, max_seq=max_seq, max_batch=2, profile="baseline")
            ref = p.PrismEngine(ref_be, mc)
            ref.synth_weights(seed=21)   # the same seeded tensors, whole: the ranks' shards are slices of these
            want = ref.generate(prompts, n_new)
            twin = oracle_twin(orc, ref_be, cfg, mc, threads=orc.max_threads())
            msg = "ok" if np.array_equal(got, want) else f"tokens differ from one GPU: {got.tolist()} vs {want.tolist()}"
            for b in range(batch):
                w, margins = twin.generate(prompts[b], n_new)
                if not np.array_equal(got[b][:32], w[:32]):
                    msg = f"sequence {b} differs from the oracle: {got[b].tolist()} vs {w.tolist()} (min margin {float(margins.min()):.5f})"
            twin.close()
            ref.close()
            ref_be.close()
            q.put((rank, msg, peer))
        else:
            q.put((rank, "ok", peer))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e), False))


@pytest.mark.timeout(1500)
# fused (one sequence only): 0 = GEMV leaves fp32 partial sums, a kernel pushes and reduces them; 1 = the GEMV delivers
# into the peers' receive areas, a kernel publishes flags and reduces; 2 = everything inside the GEMV kernel; 3 = the GEMV delivers 8-byte words
# that carry their epoch, a kernel polls the words and reduces (no flags, no fence); 4 = flagged words polled and reduced
# at the end of the GEMV kernel itself
@pytest.mark.parametrize("peer_ar,fused,wide,batch", [(1, 1, False, 2), (0, 1, False, 2), (1, 0, False, 1), (1, 1, False, 1),
                                                       (1, 2, False, 1), (0, 1, False, 1), (1, 1, True, 1), (1, 2, True, 1),
                                                       (1, 3, False, 1), (1, 3, True, 1), (1, 3, False, 2), (1, 4, False, 1), (1, 4, True, 1)])
def test_tp2_matches_single_gpu_and_oracle(peer_ar, fused, wide, batch):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000 + peer_ar + 2 * int(wide) + 4 * batch + 16 * fused
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, peer_ar, wide, batch, fused)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = [q.get(timeout=1200) for _ in procs]
    for pr in procs:
        pr.join(60)
    assert sorted(r[:2] for r in res) == [(0, "ok"), (1, "ok")], res
    # both ranks agree on whether peer memory could be mapped; on an NVLink box it can
    assert len({r[2] for r in res}) == 1, res
    print("peer-memory all-reduce set up:", res[0][2], "used:", bool(peer_ar) and res[0][2])


def test_peer_all_reduce_wait_runs_out_and_is_reported():
    """Failure detection without faulting anything: a rank whose peers never deliver.  On one GPU a
    loopback group stands for the peers (rank 0 of 2, nobody plays rank 1); the all-reduce kernel gives up
    after `wait_limit_polls` polls, the device keeps running, the next synchronising call returns
    PRISM_E_TIMEOUT once, and the context goes on serving GEMVs."""
    import torch

    import prism_engine_b200 as p
    from prism_engine_b200 import synth

    be = p.CudaBackend(device=0)
    try:
        be.set_option("wait_limit_polls", 2000)          # a few milliseconds
        be.tp_init_loopback(2, 0)
        assert be.tp_peer_ready()
        with pytest.raises(p.PrismCudaError):             # no model can run on a group without peers
            p.PrismEngine(be, p.model_config(**CFG, max_seq=8))
        n = 8192
        part = torch.ones(n, dtype=torch.float32, device="cuda")
        h = torch.zeros(n, dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        be.tp_all_reduce_resid_dev(part.data_ptr(), h.data_ptr(), n)
        with pytest.raises(p.PrismCudaError) as e:
            be.synchronize()
        assert e.value.code == -8 and "peer" in e.value.msg, (e.value.code, e.value.msg)
        be.synchronize()                                   # reported once; the error word was cleared
        m, k = 256, 128
        pay = synth.make_payload(m, k, seed=1)
        hnd = be.upload("after.timeout", pay, m, k)
        y = be.gemv(hnd, synth.make_activation(k, seed=2))
        assert y.size == m and np.any(y != 0)
    finally:
        be.close()


def _leaver(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist

    import prism_engine_b200 as p
    from prism_engine_b200 import tp

    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        be = p.CudaBackend(device=rank)
        be.tp_init(world, rank, tp.exchange_unique_id(p.CudaBackend.tp_unique_id))
        be.set_option("wait_limit_polls", 20000)
        ok = be.tp_peer_ready()
        n = 8192
        part = torch.full((n,), float(rank + 1), dtype=torch.float32, device="cuda")
        h = torch.zeros(n, dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        msg = "ok"
        if ok:
            # step 1: both ranks take part -> 1 + 2 = 3 everywhere
            be.tp_all_reduce_resid_dev(part.data_ptr(), h.data_ptr(), n)
            be.synchronize()
            if not bool((h == 3).all()):
                msg = "first all-reduce wrong"
            dist.barrier()
            # between steps rank 1 leaves (nothing of it in flight); rank 0's next all-reduce must give up
            if rank == 0:
                be.tp_all_reduce_resid_dev(part.data_ptr(), h.data_ptr(), n)
                try:
                    be.synchronize()
                    msg = "no timeout reported"
                except p.PrismCudaError as e:
                    if e.code != -8:
                        msg = f"wrong code {e.code}: {e.msg}"
                be.synchronize()   # context still answers
        dist.barrier()
        be.close()
        q.put((rank, msg, ok))
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e), False))


@pytest.mark.timeout(600)
def test_rank_that_leaves_between_steps_is_detected():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29950 + os.getpid() % 40
    procs = [ctx.Process(target=_leaver, args=(r, 2, port, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = [q.get(timeout=500) for _ in procs]
    for pr in procs:
        pr.join(60)
    assert sorted(r[:2] for r in res) == [(0, "ok"), (1, "ok")], res

"""Greedy-token parity at the widths the 72B decode benchmark runs: a 2-layer model with hidden 8192,
64 query / 8 KV heads of 128, intermediate 29568, vocabulary 152064 (untied head), max_seq >= 512 --
the folded-RMSNorm boundary of the warp-specialised GEMV (8192 values), the 8-CTA attention clusters
with head_dim 128, the cluster argmax over 152064 logits, the batched GEMV at batch 8 and the
tensor-core GEMM path at batch 12 -- against the oracle's PrismEngine twin fed with the same bytes.
"""
import numpy as np
import pytest

import prism_engine_b200 as p
from prism_engine_b200 import synth
from test_gpu_engine import oracle_twin

pytestmark = pytest.mark.gpu

WIDE = dict(p.QWEN25_72B, num_layers=2)
N_PROMPT, N_NEW = 5, 34


@pytest.fixture(scope="module")
def wide(oracle):
    be = p.CudaBackend(device=0)
    mc = p.model_config(**WIDE, max_seq=512, max_batch=12, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=72)
    twin = oracle_twin(oracle, be, WIDE, mc, threads=oracle.max_threads())
    prompts = np.stack([synth.make_prompt(N_PROMPT, WIDE["vocab_size"], seed=100 + b) for b in range(12)])
    want = {}

    def expect(b):
        if b not in want:
            want[b] = twin.generate(prompts[b], N_NEW)
        return want[b]

    yield be, eng, prompts, expect
    eng.close()
    twin.close()
    be.close()


def _check(got_row, expect_pair, what):
    want, margins = expect_pair
    n_same = int(np.argmax(np.concatenate([got_row != want, [True]])))
    print(f"{what}: {n_same}/{len(want)} tokens identical, min oracle top-1/top-2 margin {float(margins.min()):.5f}")
    assert np.array_equal(got_row[:32], want[:32]), (what, n_same, float(margins[min(n_same, len(margins) - 1)]))


@pytest.mark.timeout(1800)
def test_wide_batch1_matches_oracle(wide):
    be, eng, prompts, expect = wide
    got = eng.generate(prompts[0], N_NEW)
    assert eng.kernels_per_step() == 2 * 5 + 4      # embed, per layer qkv/attention/o/gate-up/down, head, argmax, advance
    _check(got, expect(0), "batch 1 (warp-specialised GEMV, 8-CTA attention clusters)")


@pytest.mark.timeout(1800)
def test_wide_batch8_matches_oracle(wide):
    be, eng, prompts, expect = wide
    got = eng.generate(prompts[:8], N_NEW)
    for b in (0, 7):
        _check(got[b], expect(b), f"batch 8 (batched GEMV), sequence {b}")


@pytest.mark.timeout(1800)
def test_wide_batch12_gemm_path_matches_oracle(wide):
    be, eng, prompts, expect = wide
    got = eng.generate(prompts, N_NEW)
    for b in (0, 11):
        _check(got[b], expect(b), f"batch 12 (tensor-core GEMM), sequence {b}")


def test_option_change_rebuilds_the_step_graph(oracle):
    """A captured decode graph is good for one option epoch: flipping batch_gemv_max between two generate
    calls on one engine must change what a step launches, not replay the old graph."""
    cfg = dict(num_layers=2, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=256,
               vocab_size=1024, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
    be = p.CudaBackend(device=0)
    eng = p.PrismEngine(be, p.model_config(**cfg, max_seq=64, max_batch=9, profile="baseline"))
    eng.synth_weights(seed=5)
    prompts = np.stack([synth.make_prompt(4, cfg["vocab_size"], seed=s) for s in range(9)])
    a = eng.generate(prompts, 12)
    k_gemm = eng.kernels_per_step()          # batch 9 > batch_gemv_max 8: tensor-core GEMM path
    be.set_option("batch_gemv_max", 16)
    l0 = be.launch_count()
    b = eng.generate(prompts, 12)
    k_gemv = eng.kernels_per_step()          # now the batched GEMV in groups of 8
    assert k_gemv != k_gemm and be.launch_count() > l0
    twin = oracle_twin(oracle, be, cfg, eng.cfg)
    want, _ = twin.generate(prompts[8], 12)
    assert np.array_equal(a[8], want) and np.array_equal(b[8], want)
    eng.close(); twin.close(); be.close()

"""End-to-end greedy decode: the device engine against the oracle's PrismEngine twin.

Weights are generated on the device, read back through the C ABI in the
reference's payload format and handed to the oracle, so both sides see the
same bytes.  Greedy tokens must be identical for the first 32 steps.
"""
import ctypes as C

import numpy as np
import pytest

import prism_engine_b200 as p
from prism_engine_b200 import synth

pytestmark = pytest.mark.gpu

TINY = dict(num_layers=3, hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
            vocab_size=512, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
ROLES = ["q", "k", "v", "o", "gate", "up", "down"]
SUFFIX = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight",
          "o": "self_attn.o_proj.weight", "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight",
          "down": "mlp.down_proj.weight"}


def oracle_twin(orc, be, cfg_dict, mc, threads=8):
    """Oracle model fed with the payloads read back from the device."""
    oc = orc.Cfg(mc.num_layers, mc.hidden_size, mc.num_heads, mc.num_kv_heads, mc.head_dim, mc.intermediate_size,
                 mc.vocab_size, mc.norm_eps, mc.rope_theta, mc.bits, mc.tie_word_embeddings, mc.rope_use_theta,
                 mc.rope_k, mc.kv_int8, mc.down_guard, threads)
    m = orc.Model(oc)
    for l in range(mc.num_layers):
        for r in ROLES:
            m.set_tensor(r, l, be.download_payload(be.find(f"model.layers.{l}.{SUFFIX[r]}")))
    m.set_tensor("embed", 0, be.download_payload(be.find("model.embed_tokens.weight")))
    if not mc.tie_word_embeddings:
        m.set_tensor("lm_head", 0, be.download_payload(be.find("model.lm_head.weight")))
    return m


def run_parity(oracle, cfg_dict, profile, n_prompt, max_new, seed, max_seq=256, variant=1, fuse=1, tie=None):
    d = dict(cfg_dict)
    if tie is not None:
        d["tie_word_embeddings"] = tie
    be = p.CudaBackend(device=0)
    try:
        be.set_option("gemv_variant", variant)
        be.set_option("fuse", fuse)
        mc = p.model_config(**d, max_seq=max_seq, max_batch=1, profile=profile)
        eng = p.PrismEngine(be, mc)
        eng.synth_weights(seed=seed)
        prompt = synth.make_prompt(n_prompt, d["vocab_size"], seed=seed)
        got, logits = eng.generate(prompt, max_new, return_logits=True)
        twin = oracle_twin(oracle, be, d, mc)
        want, margins = twin.generate(prompt, max_new)
        n_same = int(np.argmax(np.concatenate([got != want, [True]])))
        assert np.array_equal(got[:32], want[:32]), (
            f"tokens diverge at step {n_same}; oracle top-1/top-2 margin there {margins[min(n_same, max_new - 1)]:.5f}; "
            f"min margin over run {margins.min():.5f}")
        eng.close()
        twin.close()
        return got, want, margins
    finally:
        be.close()


@pytest.mark.parametrize("profile", ["baseline", "reference_cpu"])
@pytest.mark.parametrize("variant,fuse", [(2, 1), (1, 1), (0, 0), (0, 1), (4, 1)])
def test_tiny_model_token_parity(oracle, profile, variant, fuse):
    got, want, margins = run_parity(oracle, TINY, profile, n_prompt=9, max_new=40, seed=3, variant=variant, fuse=fuse)
    assert np.array_equal(got, want)


def test_tiny_square_mlp_under_guard(oracle):
    """inter == hidden: the reference's dim test lets DownProj run and the layer counter advance."""
    cfg = dict(TINY, intermediate_size=64)
    got, want, _ = run_parity(oracle, cfg, "reference_cpu", n_prompt=5, max_new=36, seed=4)
    assert np.array_equal(got, want)


def test_untied_head_and_empty_prompt(oracle):
    got, want, _ = run_parity(oracle, TINY, "baseline", n_prompt=0, max_new=34, seed=5, tie=False)
    assert np.array_equal(got, want)


def test_out_of_range_token_embeds_zeros(oracle):
    be = p.CudaBackend(device=0)
    mc = p.model_config(**TINY, max_seq=64, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=6)
    twin = oracle_twin(oracle, be, TINY, mc)
    eng.reset(1)
    nxt, lg = eng.step([TINY["vocab_size"] + 5], want_logits=True)   # engine_impl.rs:1423-1425
    want = twin.step(TINY["vocab_size"] + 5, 0)
    assert int(nxt[0]) == oracle.argmax(want)
    assert np.mean(lg[0] == want) > 0.9
    eng.close(); twin.close(); be.close()


def test_kv_capacity_is_checked(oracle):
    be = p.CudaBackend(device=0)
    eng = p.PrismEngine(be, p.model_config(**TINY, max_seq=8, profile="baseline"))
    eng.synth_weights(seed=1)
    with pytest.raises(p.PrismCudaError) as e:
        eng.generate(np.arange(6, dtype=np.uint32), 8)
    assert e.value.code == -5 and "KV cache full" in e.value.msg
    eng.close(); be.close()


def test_unbound_engine_refuses(oracle):
    be = p.CudaBackend(device=0)
    eng = p.PrismEngine(be, p.model_config(**TINY, max_seq=8))
    with pytest.raises(p.PrismCudaError) as e:
        eng.generate(np.arange(3, dtype=np.uint32), 2)
    assert "emb miss" in e.value.msg          # engine_impl.rs:1417 "emb miss: {key}"
    eng.close(); be.close()


def test_cimage_load_and_generate(oracle, tmp_path):
    """PrismEngine::load path: a reference-format .cimage written by the Python twin of CImageWriter."""
    cfg = dict(TINY, num_layers=2)
    graph = p.ModelGraph.build(p.UnifiedConfig(
        vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"],
        num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, norm_eps=1e-6, rope_theta=1e6,
        tie_word_embeddings=True))
    path = str(tmp_path / "tiny.cimage")
    w = p.CImageWriter(path)
    payloads = {}
    for i, (key, dm, dn) in enumerate(graph.palettized_tensors() + [graph.embedding()]):
        payloads[key] = synth.make_payload(dm, dn, seed=100 + i)
        w.append_palettized(key, payloads[key], dm, dn)
    w.set_execution_plan('{"nodes":[]}')
    w.finalize()
    be = p.CudaBackend(device=0)
    mc = p.model_config(**cfg, max_seq=64, profile="baseline")
    eng = p.PrismEngine.load(be, path, mc)
    twin = oracle_twin(oracle, be, cfg, mc)
    prompt = synth.make_prompt(7, cfg["vocab_size"], seed=2)
    got = eng.generate(prompt, 33)
    want, _ = twin.generate(prompt, 33)
    assert np.array_equal(got, want)
    assert np.array_equal(be.download_payload(be.find("model.embed_tokens.weight")), payloads["model.embed_tokens.weight"])
    eng.close(); twin.close(); be.close()


def test_batched_sequences_match_single(oracle):
    be = p.CudaBackend(device=0)
    mc = p.model_config(**TINY, max_seq=64, max_batch=3, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=8)
    prompts = np.stack([synth.make_prompt(6, TINY["vocab_size"], seed=s) for s in (1, 2, 3)])
    both = eng.generate(prompts, 20)
    for b in range(3):
        assert np.array_equal(eng.generate(prompts[b], 20), both[b])
    eng.close(); be.close()


@pytest.mark.parametrize("batch_gemv_max,batch", [(8, 8), (1, 8), (8, 5), (24, 11), (8, 11)])
def test_batched_decode_matches_the_oracle(oracle, batch_gemv_max, batch):
    """Several sequences per step.  Up to `batch_gemv_max` sequences every linear is one pass of the batched
    GEMV (groups of 8 beyond that), above it one tensor-core GEMM over the batch; tokens of each sequence must
    still be the oracle's."""
    cfg = dict(TINY, hidden_size=128, intermediate_size=256, head_dim=32, vocab_size=1024)
    be = p.CudaBackend(device=0)
    be.set_option("batch_gemv_max", batch_gemv_max)
    mc = p.model_config(**cfg, max_seq=64, max_batch=batch, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=13)
    prompts = np.stack([synth.make_prompt(5, cfg["vocab_size"], seed=s) for s in range(batch)])
    l0 = be.launch_count()
    got = eng.generate(prompts, 33)
    assert be.launch_count() > l0
    twin = oracle_twin(oracle, be, cfg, mc)
    for b in (0, 3, batch - 1):
        want, margins = twin.generate(prompts[b], 33)
        assert np.array_equal(got[b][:32], want[:32]), (b, float(margins.min()))
    eng.close(); twin.close(); be.close()


@pytest.mark.parametrize("chunk", [512, 16, 0])
def test_batched_prefill_matches_the_oracle(oracle, chunk):
    """generate() puts the prompt through the layers in chunks of `prefill_chunk` tokens (tensor-core GEMMs, causal
    attention over the cache); 0 is the reference's one step per prompt token.  All must continue with the oracle's tokens."""
    cfg = dict(num_layers=3, hidden_size=256, num_heads=8, num_kv_heads=2, head_dim=32, intermediate_size=640,
               vocab_size=2048, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    be = p.CudaBackend(device=0)
    be.set_option("prefill_chunk", chunk)
    mc = p.model_config(**cfg, max_seq=128, max_batch=3, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=17)
    prompts = np.stack([synth.make_prompt(41, cfg["vocab_size"], seed=s) for s in range(3)])
    l0 = be.launch_count()
    got = eng.generate(prompts, 33)
    n_launch = be.launch_count() - l0
    twin = oracle_twin(oracle, be, cfg, mc)
    for b in range(3):
        want, margins = twin.generate(prompts[b], 33)
        assert np.array_equal(got[b][:32], want[:32]), (chunk, b, float(margins.min()))
    print("prefill_chunk", chunk, "launches", n_launch)
    eng.close(); twin.close(); be.close()


@pytest.mark.timeout(900)
def test_context_beyond_the_reference_limit(oracle):
    """A 5000-token prompt (the reference stops at MAX_SEQ = 4096, engine_impl.rs:30): batched prefill in chunks,
    then decode with every cluster rank of the attention kernel walking several tiles of cached rows."""
    cfg = dict(num_layers=2, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=256,
               vocab_size=1024, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
    be = p.CudaBackend(device=0)
    mc = p.model_config(**cfg, max_seq=6000, max_batch=1, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=23)
    prompt = synth.make_prompt(5000, cfg["vocab_size"], seed=4)
    got = eng.generate(prompt, 33)
    assert eng.position() == 5033
    twin = oracle_twin(oracle, be, cfg, mc)
    want, margins = twin.generate(prompt, 33)
    assert np.array_equal(got[:32], want[:32]), float(margins.min())
    eng.close(); twin.close(); be.close()


def test_paged_kv_cache(oracle):
    """The fp16 cache as a pool of 16-position pages shared by the sequences: same tokens as the oracle, pages
    returned on reset, and a clear error when the pool runs out."""
    cfg = dict(TINY, hidden_size=128, intermediate_size=256, head_dim=32, vocab_size=1024)
    be = p.CudaBackend(device=0)
    # 3 sequences x 64 positions would be 12 pages of 16; the pool has 9: enough for 3 x 45 positions, not for 3 x 64
    mc = p.model_config(**cfg, max_seq=64, max_batch=3, profile="baseline", kv_page_size=16, kv_pool_pages=9)
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=31)
    prompts = np.stack([synth.make_prompt(11, cfg["vocab_size"], seed=s) for s in range(3)])
    got = eng.generate(prompts, 33)                       # 44 positions per sequence: 3 pages each
    twin = oracle_twin(oracle, be, cfg, mc)
    for b in range(3):
        want, margins = twin.generate(prompts[b], 33)
        assert np.array_equal(got[b][:32], want[:32]), (b, float(margins.min()))
    with pytest.raises(p.PrismCudaError) as e:
        eng.generate(prompts, 50)                         # 61 positions: 4 pages each = 12 > 9
    assert e.value.code == -5 and "page pool exhausted" in e.value.msg
    one = eng.generate(prompts[1], 50)                    # a single sequence may use what three could not
    want, _ = twin.generate(prompts[1], 50)
    assert np.array_equal(one[:32], want[:32])
    # token-serial prefill and stepwise decode go through the same page table
    be.set_option("prefill_chunk", 0)
    again = eng.generate(prompts, 33)
    assert np.array_equal(again, got)
    eng.close(); twin.close(); be.close()


def test_more_than_32_sequences(oracle):
    """40 concurrent sequences (the reference decodes one): every linear is one tensor-core GEMM over the batch."""
    cfg = dict(TINY, hidden_size=128, intermediate_size=256, head_dim=32, vocab_size=1024)
    be = p.CudaBackend(device=0)
    mc = p.model_config(**cfg, max_seq=64, max_batch=40, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=29)
    prompts = np.stack([synth.make_prompt(9, cfg["vocab_size"], seed=s) for s in range(40)])
    got = eng.generate(prompts, 33)
    twin = oracle_twin(oracle, be, cfg, mc)
    for b in (0, 17, 39):
        want, margins = twin.generate(prompts[b], 33)
        assert np.array_equal(got[b][:32], want[:32]), (b, float(margins.min()))
    eng.close(); twin.close(); be.close()


@pytest.mark.timeout(1500)
def test_qwen25_0p5b_first_32_tokens(oracle):
    """The 0.5B-architecture model of the benchmark configuration: identical greedy tokens for 32 steps."""
    got, want, margins = run_parity(oracle, p.QWEN25_0P5B, "baseline", n_prompt=16, max_new=32, seed=11, max_seq=64)
    assert np.array_equal(got, want)
    print("0.5B parity: min top-1/top-2 margin", float(margins.min()))

"""Loader parity on the GPU: re-lay round trip and bit-exact dequantisation (through the C ABI)."""
import numpy as np
import pytest

from prism_engine_b200 import PrismCudaError, synth, tp

pytestmark = pytest.mark.gpu

SHAPES = [(2, 8, 4), (33, 40, 4), (64, 32, 4), (100, 96, 4), (4864, 896, 4), (896, 4864, 4), (128, 896, 4),
          (65, 64, 2), (512, 3584, 2), (31, 16, 2)]


@pytest.mark.parametrize("m,k,bits", SHAPES)
def test_relay_roundtrip_and_dequant_bit_exact(backend, oracle, m, k, bits):
    pay = synth.make_payload(m, k, bits, seed=m + k)
    h = backend.upload(f"t_{m}_{k}_{bits}", pay, m, k, bits)
    assert backend.dims(h) == (m, k, bits)
    assert np.array_equal(backend.download_payload(h), pay)          # inverse re-lay is the identity
    assert np.array_equal(backend.dequant(h), oracle.dequant(pay, m, k, bits))  # bit-exact weights
    backend.free(h)


def test_reference_kat_payload(backend):
    # compute-core/src/lut/evaluator.rs:231-246: row 0 palette all 1.0, row 1 all 2.0, indices 0
    p = np.concatenate([np.full(16, 0x3C00, "<u2").view(np.uint8), np.full(16, 0x4000, "<u2").view(np.uint8),
                        np.zeros(8, np.uint8)])
    h = backend.upload("kat", p, 2, 8)
    y = backend.gemv(h, np.full(8, 0x3C00, np.uint16))
    assert y.tolist() == [0x4800, 0x4C00]
    for variant in (0, 1, 2):
        backend.set_option("gemv_variant", variant)
        assert backend.gemv("kat", np.full(8, 0x3C00, np.uint16)).tolist() == [0x4800, 0x4C00]
    backend.free(h)


def test_shard_upload_matches_slice(backend, oracle):
    m, k = 160, 256
    pay = synth.make_payload(m, k, 4, seed=9)
    for (r0, rows, c0, cols) in [(32, 96, 0, 256), (0, 160, 64, 128), (64, 33, 32, 224)]:
        h = backend.upload("shard", pay, m, k, 4, shard=(r0, rows, c0, cols))
        want = tp.slice_payload(pay, m, k, 4, r0, rows, c0, cols)
        assert np.array_equal(backend.download_payload(h), want)
        backend.free(h)


def test_device_synth_is_deterministic_and_sorted(backend, oracle):
    h1 = backend.synth("s1", 96, 128, 4, seed=7)
    h2 = backend.synth("s2", 96, 128, 4, seed=7)
    h3 = backend.synth("s3", 96, 128, 4, seed=8)
    p1, p2, p3 = (backend.download_payload(h) for h in (h1, h2, h3))
    assert np.array_equal(p1, p2) and not np.array_equal(p1, p3)
    pal = p1[: 96 * 32].view("<u2").view(np.float16).reshape(96, 16).astype(np.float32)
    assert np.all(np.diff(pal, axis=1) >= 0) and 0.005 < pal.std() < 0.05
    idx = p1[96 * 32:]
    assert idx.size == 96 * 64 and 100 < idx.astype(np.float64).mean() < 155
    for h in (h1, h2, h3):
        backend.free(h)


def test_rejects_bad_arguments(backend):
    pay = synth.make_payload(8, 32, 4, seed=1)
    with pytest.raises(PrismCudaError) as e:
        backend.upload("short", pay[:-1], 8, 32)
    assert e.value.code == -2 and "truncated" in e.value.msg
    with pytest.raises(PrismCudaError):
        backend.upload("bits", pay, 8, 32, bits=3)
    with pytest.raises(PrismCudaError):
        backend.upload("k", pay, 8, 36)       # 36*4 bits is not a whole number of index words
    with pytest.raises(PrismCudaError) as e:
        backend.gemv("no.such.tensor", np.zeros(32, np.uint16))
    assert e.value.code == -3 and "miss no.such.tensor" in e.value.msg   # MetalBackend::gemv's "miss {key}"
    h = backend.upload("ok", pay, 8, 32)
    with pytest.raises(PrismCudaError):
        backend.gemv(h, np.zeros(31, np.uint16))
    backend.free(h)
    with pytest.raises(PrismCudaError):
        backend.dims(h)                          # freed handle


def _write_tiny_cimage(path, plan):
    import prism_engine_b200 as p

    graph = p.ModelGraph.build(p.UnifiedConfig(vocab_size=256, hidden_size=64, intermediate_size=96, num_layers=2,
                                               num_heads=4, num_kv_heads=2, head_dim=16, tie_word_embeddings=True))
    w = p.CImageWriter(path)
    payloads = {}
    for i, (key, dm, dn) in enumerate(graph.palettized_tensors() + [graph.embedding()]):
        payloads[key] = synth.make_payload(dm, dn, seed=300 + i)
        w.append_palettized(key, payloads[key], dm, dn)
    w.append_blob("tokenizer.blob", np.arange(100, dtype=np.uint8))
    if plan == "reference":
        w.set_execution_plan(p.generate_plan(graph, has_gpu=True))
    elif plan is not None:
        w.set_execution_plan(plan)
    w.finalize()
    return graph, payloads


def test_cimage_execution_plan_is_parsed_and_bad_plans_tolerated(tmp_path):
    import prism_engine_b200 as p

    for plan, want_version in (("reference", 1), (None, 0), ('{"schema":"compute-core","ops":[1,2]}', 0), ("{not json", 0)):
        be = p.CudaBackend(device=0)
        path = str(tmp_path / f"m{want_version}{abs(hash(plan)) % 97}.cimage")
        graph, payloads = _write_tiny_cimage(path, plan)
        assert be.load_cimage(path) == len(payloads)            # the load itself never depends on the plan
        pl = be.cimage_plan()
        assert pl["version"] == want_version
        if want_version:
            assert pl["num_layers"] == 2 and pl["n_nodes"] == len(graph.nodes) and pl["n_gemm_nodes"] == 14
            assert pl["kv_cache"] == "Fp16" and pl["attention_strategy"] == "MetalKernel" and pl["lm_head_backend"] == "metal"
        be.close()


def test_cimage_relaid_cache_round_trip(tmp_path):
    """First load writes the device layout beside the container; the second load takes it from there (no
    re-lay kernels) and holds byte-identical tensors; a changed container invalidates the cache."""
    import os

    import prism_engine_b200 as p

    path = str(tmp_path / "m.cimage")
    graph, payloads = _write_tiny_cimage(path, "reference")
    be = p.CudaBackend(device=0)
    n, hit = be.load_cimage(path, cache="")
    assert n == len(payloads) and not hit and os.path.exists(path + ".b200relay")
    be.close()
    be = p.CudaBackend(device=0)
    l0 = be.launch_count()
    n, hit = be.load_cimage(path, cache="")
    assert n == len(payloads) and hit and be.launch_count() == l0       # copies only
    for key, pay in payloads.items():
        assert np.array_equal(be.download_payload(be.find(key)), pay), key
    x = synth.make_activation(64, seed=1)
    key = "model.layers.1.mlp.gate_proj.weight"
    y_cached = be.gemv(key, x)
    be.close()
    be = p.CudaBackend(device=0)
    be.load_cimage(path)
    assert np.array_equal(be.gemv(key, x), y_cached)
    be.close()
    # another model under the same name: the key (header + size) differs, the stale cache is replaced
    _write_tiny_cimage(path, None)                                     # same tensors, different header bytes
    be = p.CudaBackend(device=0)
    n, hit = be.load_cimage(path, cache="")
    assert not hit
    be.close()
    # option-driven use by the engine loader
    be = p.CudaBackend(device=0)
    be.set_option("cimage_cache", 1)
    mc = p.model_config(num_layers=2, hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                        vocab_size=256, tie_word_embeddings=True, max_seq=32, profile="baseline")
    eng = p.PrismEngine.load(be, path, mc)
    toks = eng.generate(np.array([1, 2, 3], np.uint32), 5)
    assert toks.shape == (5,)
    eng.close(); be.close()

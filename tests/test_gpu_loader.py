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

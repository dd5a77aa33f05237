"""The oracle against every known-answer test the reference holds for this path.

Each test names the reference test it restates (paths relative to the
reference repository root).  These run on CPU.
"""
import numpy as np


def _h(v):
    return np.array(v, dtype=np.float32).astype(np.float16).view(np.uint16)


def test_lut_gemv_kat(oracle):
    # compute-core/src/lut/evaluator.rs:231-246 (same at compute-core/src/lut/engine.rs:752-767)
    p = bytearray()
    for _ in range(16):
        p += (0x3C00).to_bytes(2, "little")
    for _ in range(16):
        p += (0x4000).to_bytes(2, "little")
    p += bytes(8)
    x = np.full(8, 0x3C00, np.uint16)
    y = oracle.lut_gemv(x, np.frombuffer(bytes(p), np.uint8), 2, 8)
    assert abs(oracle.f16_vals(y)[0] - 8.0) < 0.01
    assert y[0] == 0x4800 and y[1] == 0x4C00  # 8.0, 16.0 exactly


def test_rms_kat(oracle):
    # compute-core/src/lut/evaluator.rs:248-255
    out = oracle.rms_norm(np.full(4, 0x3C00, np.uint16), 1e-6)
    assert np.all(np.abs(oracle.f16_vals(out) - 1.0) < 1e-4)


def test_vec_add_kat(oracle):
    # compute-core/src/lut/evaluator.rs:257-265
    out = oracle.vec_add(_h([1.0] * 4), _h([2.0] * 4))
    assert np.all(np.abs(oracle.f16_vals(out) - 3.0) < 1e-4)


def test_lut_embed_kat(oracle):
    # compute-core/src/lut/evaluator.rs:267-284; src/lut/engine_impl.rs:1531-1571
    payload = np.concatenate([np.full(2 * 16, 0x3C00, "<u2").view(np.uint8), np.zeros(2 * 4, np.uint8)])
    v = oracle.embed(0, payload, 2, 8)
    assert v.size == 8 and np.all(v == 0x3C00)
    v2 = oracle.embed(5, payload, 2, 8)
    assert v2.size == 8 and np.all(v2 == 0)


def test_silu_mul_kat(oracle):
    # compute-core/src/lut/evaluator.rs:286-298
    g = oracle.mul(oracle.silu(_h([2.0] * 4)), _h([3.0] * 4))
    expected = 2.0 / (1.0 + np.exp(np.float32(-2.0))) * 3.0
    assert abs(oracle.f16_vals(g)[0] - expected) < 0.01


def test_gelu_kat(oracle):
    # compute-core/src/lut/evaluator.rs:300-308
    g = oracle.f16_vals(oracle.gelu(_h([1.0, 1.0])))[0]
    assert 0.8 < g < 0.9


def test_encode_channel_kat(oracle):
    # src/quantization/palette.rs:410-425 -- pins the nibble order
    packed, mse = oracle.encode_channel([1.0, 2.0, 3.0, 4.0], [1.0, 2.0, 3.0, 4.0] + [0.0] * 12)
    assert packed.tolist() == [0x10, 0x32] and mse < 1e-3


def test_fit_palette_kat(oracle):
    # src/quantization/palette.rs:371-408
    data = [-5.0] * 5 + [0.0] * 5 + [5.0] * 5
    cb = np.sort(oracle.fit_palette(data, 3, 50))
    assert cb.size == 3 and np.all(np.abs(cb - np.array([-5.0, 0.0, 5.0])) < 0.1)


def test_palettize_roundtrip_kat(oracle):
    # src/quantization/palette.rs:427-456: 3x4 matrix, k = 4
    w = np.arange(1, 13, dtype=np.float32)
    payload = oracle.palettize_to_payload(w, 3, 4, k=4, max_iter=50)
    pal = payload[: 3 * 32].view("<u2").reshape(3, 16)
    assert np.all(pal[:, :4] != 0)
    deq = oracle.f16_vals(oracle.dequant(payload, 3, 4)).reshape(-1)
    assert np.mean((deq - w) ** 2) < 2.0


def test_int8_kv_roundtrip_kat(oracle):
    # compute-core/src/lut/quantization.rs:94-108: round-trip error < 0.02 on values in [-1, 1]
    x = _h(np.linspace(-1.0, 1.0, 64))
    blk = oracle.kv_quant(x)
    back = oracle.f16_vals(oracle.kv_dequant(blk, 1, 64))
    assert np.max(np.abs(back - oracle.f16_vals(x))) < 0.02


def test_f16_conversion_exhaustive(oracle):
    # half::f16::{to_f32,from_f32}: numpy's float16 is the same IEEE binary16
    L = oracle.lib()
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    got = np.array([L.po_f16_to_f32(int(b)) for b in bits], np.float32)
    ok = (got == ref) | (np.isnan(got) & np.isnan(ref))
    assert ok.all()
    rng = np.random.default_rng(1)
    f = np.concatenate([rng.normal(0, 1, 20000), rng.normal(0, 1e-6, 5000), rng.normal(0, 7e4, 5000),
                        [0.0, -0.0, 65504.0, 65520.0, 65519.9, 5.9604645e-08, 2.9802322e-08, 2.98023224e-08 * 1.0001,
                         np.inf, -np.inf, 6.1035156e-05, 6.0975552e-05]]).astype(np.float32)
    want = f.astype(np.float16).view(np.uint16)
    have = np.array([L.po_f32_to_f16(float(v)) for v in f], np.uint16)
    assert np.array_equal(want, have)

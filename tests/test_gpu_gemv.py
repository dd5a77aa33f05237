"""Palettized GEMV / fused SwiGLU / MLP / GEMM parity against the CPU oracle, through the C ABI.

Tolerance: 1e-3 relative L2 on fp16 outputs of fp32-accumulated sums (the
summation order differs from the oracle's strictly serial one); exact equality
is required wherever the sum has a single non-zero term.
"""
import numpy as np
import pytest

from conftest import rel_l2
from prism_engine_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-3

SAMPLED_TOKENS = [0, 1, 127, 128, 255, 256, 1000, 2047]   # first, last, and both sides of the 128- and 256-token tile edges

GEMV_SHAPES = [(64, 32), (33, 64), (100, 96), (4864, 896), (896, 4864), (128, 896), (896, 896), (1000, 8),
               (72, 40), (8192, 1024), (2368, 8192), (3712, 256),
               (640, 29568), (20000, 512), (9000, 1312)]


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("m,k", GEMV_SHAPES)
def test_gemv_matches_oracle(backend, oracle, variant, m, k):
    backend.set_option("gemv_variant", variant)
    pay = synth.make_payload(m, k, 4, seed=m * 7 + k)
    x = synth.make_activation(k, seed=k)
    h = backend.upload("g", pay, m, k)
    y = backend.gemv(h, x)
    want = oracle.lut_gemv(x, pay, m, k, threads=8)
    assert rel_l2(y, want) <= TOL
    # fp32 accumulation error is far below an fp16 ulp: almost every element is bit-identical
    assert np.mean(y == want) > 0.9
    big = (want & 0x7FFF) > 0x2800  # |y| > 2^-5: one fp16 ulp there dwarfs the fp32 summation error
    if big.any():
        assert np.max(np.abs(y.astype(np.int64) - want.astype(np.int64))[big]) <= 1
    backend.free(h)
    backend.set_option("gemv_variant", 1)


@pytest.mark.parametrize("m,k", [(8192, 8192), (8256, 8192), (4160, 29568), (10240, 8192)])
def test_gemv_large_shapes(backend, oracle, m, k):
    """The persistent warp-specialised kernel at 72B-sized shapes (8256 rows = 129 blocks: an odd count)."""
    h = backend.synth("big", m, k, seed=m + k)
    pay = backend.download_payload(h)
    x = synth.make_activation(k, seed=7)
    y = backend.gemv(h, x)
    want = oracle.lut_gemv(x, pay, m, k, threads=oracle.max_threads())
    assert rel_l2(y, want) <= TOL
    assert np.mean(y == want) > 0.9
    backend.free(h)


def test_fused_gate_up_large(backend, oracle):
    hidden, inter = 8192, 9248           # 289 gate/up half-blocks: an odd number of blocks
    hg, hu = backend.synth("bg", inter, hidden, seed=1), backend.synth("bu", inter, hidden, seed=2)
    x = synth.make_activation(hidden, seed=3)
    act = backend.fused_gate_up(hg, hu, x)
    _, want = oracle.mlp(backend.download_payload(hg), backend.download_payload(hu), None, x, hidden, inter,
                         threads=oracle.max_threads())
    assert rel_l2(act, want) <= TOL and np.mean(act == want) > 0.9
    backend.free(hg); backend.free(hu)


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("m,k", [(65, 64), (512, 3584), (96, 128), (100, 48), (3584, 18944), (18944, 3584), (4864, 896)])
def test_gemv_2bit(backend, oracle, variant, m, k):
    """2-bit indices / 4-entry palettes (no such format in the reference: the oracle's generalisation is the pin).
    variant 1 takes the pair-table tensor-core kernel when K is a whole number of 64-weight chunks, the plain
    kernel otherwise; variant 0 is always the plain kernel."""
    backend.set_option("gemv_variant", variant)
    pay = synth.make_payload(m, k, 2, seed=m + k)
    x = synth.make_activation(k, seed=3)
    h = backend.upload("g2", pay, m, k, bits=2)
    y = backend.gemv(h, x)
    want = oracle.lut_gemv(x, pay, m, k, bits=2, threads=8)
    assert rel_l2(y, want) <= TOL
    assert np.mean(y == want) > 0.9
    backend.free(h)
    backend.set_option("gemv_variant", 1)


def test_gemv_2bit_one_hot_is_exact(backend, oracle):
    m, k = 512, 3584
    pay = synth.make_payload(m, k, 2, seed=9)
    W = oracle.dequant(pay, m, k, bits=2)
    h = backend.upload("oh2", pay, m, k, bits=2)
    for j in (0, 1, 2, 3, 63, 64, 1000, 3583):
        x = np.zeros(k, np.uint16)
        x[j] = 0x3C00
        want = W[:, j].copy()
        want[want == 0x8000] = 0
        assert np.array_equal(backend.gemv(h, x), want), j
    backend.free(h)


@pytest.mark.parametrize("name,m,k", [("kv", 512, 3584), ("q", 3584, 3584), ("gate_up", 18944, 3584), ("down", 3584, 18944)])
def test_gemm_2bit_prefill_shapes_match_oracle(backend, oracle, name, m, k):
    """The 2-bit variant of the prefill configuration through the tensor-core GEMM (parity unpinned by the reference)."""
    m_tok = 2048
    pay = synth.make_payload(m, k, 2, seed=70 + m % 5)
    h = backend.upload(f"c4b2.{name}", pay, m, k, bits=2)
    X = synth.make_activation((m_tok, k), seed=m + 2 * k)
    Y = backend.gemm(h, X)
    want = oracle.lut_gemm(X[SAMPLED_TOKENS], pay, m, k, bits=2, threads=oracle.max_threads())
    got = Y[SAMPLED_TOKENS]
    assert rel_l2(got.reshape(-1), want.reshape(-1)) <= TOL
    assert np.mean(got == want) > 0.9
    backend.free(h)


@pytest.mark.parametrize("m,k,m_tok", [(192, 256, 37), (130, 128, 9), (640, 1024, 300)])
def test_gemm_2bit_small_shapes(backend, oracle, m, k, m_tok):
    pay = synth.make_payload(m, k, 2, seed=8)
    X = synth.make_activation((m_tok, k), seed=8)
    h = backend.upload("gm2", pay, m, k, bits=2)
    Y = backend.gemm(h, X)
    want = oracle.lut_gemm(X, pay, m, k, bits=2, threads=8)
    assert rel_l2(Y.reshape(-1), want.reshape(-1)) <= TOL and np.mean(Y == want) > 0.9
    backend.free(h)


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4, 5])
def test_gemv_one_hot_is_exact(backend, oracle, variant):
    """x = e_j picks column j of the dequantised matrix: a single-term sum, so bit-exact at full size."""
    backend.set_option("gemv_variant", variant)
    m, k = 4864, 896
    pay = synth.make_payload(m, k, 4, seed=42)
    W = oracle.dequant(pay, m, k)
    h = backend.upload("oh", pay, m, k)
    for j in (0, 1, 31, 32, 445, 895):
        x = np.zeros(k, np.uint16)
        x[j] = 0x3C00
        y = backend.gemv(h, x)
        # +0.0 sums: a column entry of -0.0 reads back as +0.0 after accumulation with zeros
        want = W[:, j].copy()
        want[want == 0x8000] = 0
        assert np.array_equal(y, want), j
    backend.free(h)
    backend.set_option("gemv_variant", 1)


def test_gemv_linearity_full_size(backend, oracle):
    """GEMV(2x) == 2*GEMV(x) exactly: scaling by two is exact in fp16 and fp32 as long as the fp16
    result is a normal number (a subnormal result has already lost bits the doubled sum keeps)."""
    m, k = 4864, 896
    h = backend.synth("lin", m, k, seed=5)
    x = synth.make_activation(k, seed=8, scale=0.25)
    x2 = (x.view(np.float16) * np.float16(2)).view(np.uint16)
    y, y2 = backend.gemv(h, x), backend.gemv(h, x2)
    normal = (y & 0x7C00) != 0
    assert normal.mean() > 0.99
    assert np.array_equal((y.view(np.float16) * np.float16(2)).view(np.uint16)[normal], y2[normal])
    backend.free(h)


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("hidden,inter", [(64, 96), (896, 4864), (256, 1000 // 8 * 8)])
def test_fused_gate_up_and_mlp(backend, oracle, variant, hidden, inter):
    backend.set_option("gemv_variant", variant)
    wg, wu = synth.make_payload(inter, hidden, seed=1), synth.make_payload(inter, hidden, seed=2)
    wd = synth.make_payload(hidden, inter, seed=3)
    x = synth.make_activation(hidden, seed=4)
    hg, hu, hd = backend.upload("gate", wg, inter, hidden), backend.upload("up", wu, inter, hidden), \
        backend.upload("down", wd, hidden, inter)
    want_out, want_act = oracle.mlp(wg, wu, wd, x, hidden, inter, threads=8)
    act = backend.fused_gate_up("gate", "up", x)
    assert rel_l2(act, want_act) <= TOL
    assert np.mean(act == want_act) > 0.9
    out = backend.mlp(hg, hu, hd, x)
    assert rel_l2(out, want_out) <= TOL
    for h in (hg, hu, hd):
        backend.free(h)
    backend.set_option("gemv_variant", 1)


@pytest.mark.parametrize("gemm_variant", [0, 1])
@pytest.mark.parametrize("m,k,m_tok", [(192, 256, 37), (256, 512, 300), (130, 64, 32), (512, 3584, 96),
                                        (4864, 896, 2), (896, 4864, 3), (2368, 8192, 7), (192, 256, 9), (640, 29568, 5)])
def test_gemm_rows_are_gemvs(backend, oracle, gemm_variant, m, k, m_tok):
    backend.set_option("gemm_variant", gemm_variant)
    pay = synth.make_payload(m, k, seed=6)
    X = synth.make_activation((m_tok, k), seed=6)
    h = backend.upload("gm", pay, m, k)
    Y = backend.gemm(h, X)
    want = oracle.lut_gemm(X, pay, m, k, threads=8)
    assert Y.shape == (m_tok, m) and rel_l2(Y.reshape(-1), want.reshape(-1)) <= TOL
    assert np.mean(Y == want) > 0.9
    backend.free(h)
    backend.set_option("gemm_variant", 1)


def test_gemm_full_size_rows_match_gemv(backend):
    """Qwen2.5-7B q-projection shape, M = 2048 tokens: sampled rows of the tensor-core GEMM equal the GEMV
    of the same activation row up to fp32 summation order."""
    m, k, m_tok = 3584, 3584, 2048
    h = backend.synth("gm.full", m, k, seed=3)
    X = synth.make_activation((m_tok, k), seed=4)
    Y = backend.gemm(h, X)
    for t in (0, 1, 255, 256, 1000, 2047):
        y = backend.gemv(h, X[t])
        assert rel_l2(Y[t], y) <= TOL and np.mean(Y[t] == y) > 0.9, t
    backend.free(h)


CONFIG4 = [("q", 3584, 3584), ("kv", 512, 3584), ("gate_up", 18944, 3584), ("down", 3584, 18944)]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("name,m,k", CONFIG4)
def test_gemm_prefill_shapes_match_oracle(backend, oracle, name, m, k):
    """The Qwen2.5-7B prefill shapes at M = 2048 tokens of N(0,1) activations through the tensor-core GEMM:
    sampled token rows against prefill_cpu (one lut_gemv_cpu per row, engine_impl.rs:1046-1053)."""
    m_tok = 2048
    pay = synth.make_payload(m, k, 4, seed=40 + m % 7)
    h = backend.upload(f"c4.{name}", pay, m, k)
    X = synth.make_activation((m_tok, k), seed=m + k)
    l0 = backend.launch_count()
    Y = backend.gemm(h, X)
    assert backend.launch_count() > l0
    want = oracle.lut_gemm(X[SAMPLED_TOKENS], pay, m, k, threads=oracle.max_threads())
    got = Y[SAMPLED_TOKENS]
    assert rel_l2(got.reshape(-1), want.reshape(-1)) <= TOL
    assert np.mean(got == want) > 0.9
    for i, t in enumerate(SAMPLED_TOKENS):
        assert rel_l2(got[i], want[i]) <= TOL, (name, t)
    backend.free(h)

"""Decode glue kernels against the CPU oracle (through the C ABI's host-slice entry points)."""
import numpy as np
import pytest

from conftest import rel_l2
from prism_engine_b200 import synth

pytestmark = pytest.mark.gpu


def test_rms_norm(backend, oracle):
    for n in (4, 896, 8192):
        x = synth.make_activation(n, seed=n)
        got, want = backend.norm(x, 1e-6), oracle.rms_norm(x, 1e-6)
        assert rel_l2(got, want) < 1e-3 and np.mean(got == want) > 0.98
    assert np.all(np.abs(oracle.f16_vals(backend.norm(np.full(4, 0x3C00, np.uint16), 1e-6)) - 1.0) < 1e-4)


def test_vec_add_silu_exact(backend, oracle):
    a, b = synth.make_activation(4864, seed=1), synth.make_activation(4864, seed=2)
    assert np.array_equal(backend.vec_add(a, b), oracle.vec_add(a, b))
    got, want = backend.silu(a), oracle.silu(a)
    assert np.mean(got == want) > 0.999 and rel_l2(got, want) < 1e-3


@pytest.mark.parametrize("pos", [0, 1, 77, 639])
@pytest.mark.parametrize("base", [10000.0, 1e6])
def test_rope(backend, oracle, pos, base):
    x = synth.make_activation(14 * 64, seed=pos)
    got, want = backend.rope(x, pos, 64, base), oracle.rope(x, pos, 64, base)
    assert rel_l2(got, want) < 1e-3 and np.mean(got == want) > 0.9


@pytest.mark.parametrize("nh,nkv,hd,sl", [(14, 2, 64, 1), (14, 2, 64, 129), (8, 8, 128, 40), (4, 1, 32, 300)])
def test_attention(backend, oracle, nh, nkv, hd, sl):
    q = synth.make_activation(nh * hd, seed=1)
    k = synth.make_activation(sl * nkv * hd, seed=2)
    v = synth.make_activation(sl * nkv * hd, seed=3)
    got, want = backend.attention(q, k, v, sl, nh, nkv, hd), oracle.attention(q, k, v, nh, nkv, hd, sl)
    assert rel_l2(got, want) < 1e-3


def test_attention_short_cache_gives_zeros(backend):
    out = backend.attention(np.zeros(64, np.uint16), np.zeros(10, np.uint16), np.zeros(10, np.uint16), 4, 1, 1, 64)
    assert np.all(out == 0)   # MetalBackend::attention, engine_impl.rs:207-209


def test_argmax_first_max(backend, oracle):
    lg = synth.make_activation(151936, seed=4)
    assert backend.argmax(lg) == oracle.argmax(lg)
    lg[1000] = lg[77] = 0x7BFF          # two equal maxima: the first wins
    assert backend.argmax(lg) == 77 == oracle.argmax(lg)
    assert backend.argmax(np.full(50, 0x7E00, np.uint16)) == 0 == oracle.argmax(np.full(50, 0x7E00, np.uint16))
    assert backend.argmax(np.full(9, 0xFC00, np.uint16)) == 0    # all -inf


def test_softmax(backend):
    x = synth.make_activation(640, seed=9)
    f = x.view(np.float16).astype(np.float64)
    want = np.exp(f - f.max())
    want /= want.sum()
    got = backend.softmax(x).view(np.float16).astype(np.float64)
    assert np.abs(got - want).max() < 1e-3 and abs(got.sum() - 1) < 5e-3

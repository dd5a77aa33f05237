"""GPU quantiser against the CPU restatement of the reference's (bit-identical payloads), through the C ABI.

The oracle's ``fit_palette`` / ``encode_channel`` are pinned on the reference's own tests
(tests/test_oracle_kat.py: palette.rs:371-456); here whole payloads of seeded matrices must be equal
byte for byte, including rows with few distinct values (the seeding's zero-total branch), k < 16,
and the upload -> dequant round trip of the produced payload.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _weights(m, k, seed, kind):
    rng = np.random.default_rng(seed)
    if kind == "normal":
        return (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
    if kind == "few_values":  # fewer distinct values than centroids in some rows
        vals = rng.standard_normal(5).astype(np.float32)
        w = vals[rng.integers(0, 5, size=(m, k))]
        w[0, :] = 0.25  # a constant row
        return w
    if kind == "heavy_tail":
        return (rng.standard_t(2, size=(m, k)) * 0.05).astype(np.float32)
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["normal", "few_values", "heavy_tail"])
@pytest.mark.parametrize("m,k", [(5, 8), (64, 96), (130, 896), (33, 4864)])
def test_payload_is_bit_identical_to_the_cpu_quantiser(backend, oracle, m, k, kind):
    w = _weights(m, k, seed=m * 1000 + k, kind=kind)
    got = backend.palettize(w)
    want = oracle.palettize_to_payload(w, m, k, 16, 50)
    assert got.shape == want.shape
    assert np.array_equal(got[: m * 32], want[: m * 32]), "palettes differ"
    assert np.array_equal(got, want), "index bytes differ"


@pytest.mark.parametrize("k_entries,max_iter", [(4, 50), (16, 3), (1, 50)])
def test_fewer_entries_and_iteration_cap(backend, oracle, k_entries, max_iter):
    w = _weights(48, 256, seed=7, kind="normal")
    got = backend.palettize(w, k=k_entries, max_iter=max_iter)
    want = oracle.palettize_to_payload(w, 48, 256, k_entries, max_iter)
    assert np.array_equal(got, want)


def test_quantise_upload_dequant_round_trip(backend, oracle):
    """The produced payload is what the loader accepts: upload it, dequantise on the device, compare with the
    oracle's dequantisation of the CPU-quantised payload, and bound the quantisation error."""
    m, k = 96, 512
    w = _weights(m, k, seed=3, kind="normal")
    pay = backend.palettize(w)
    h = backend.upload("q.rt", pay, m, k)
    deq = backend.dequant(h).astype(np.uint16)
    want = oracle.dequant(oracle.palettize_to_payload(w, m, k, 16, 50), m, k)
    assert np.array_equal(deq.reshape(-1), np.asarray(want).reshape(-1))
    err = deq.view(np.float16).astype(np.float32).reshape(m, k) - w
    assert float(np.mean(err * err)) < 0.05 * float(np.var(w))  # 16 centroids per row of N(0, 0.02)
    backend.free(h)


def test_bad_shapes_are_refused(backend):
    import prism_engine_b200 as p

    with pytest.raises(p.PrismCudaError):
        backend.palettize(np.zeros((4, 7), dtype=np.float32))  # odd dim_n

"""The fused decode-attention kernel (RoPE q, RoPE k, cache append, attention in one cluster kernel)
against the oracle's rope_inplace + attention_cpu (src/lut/cpu_fallback.rs:84-143), through the C ABI.

Every cluster size (1, 2, 4, 8 CTAs per head), every head size the kernel is instantiated for, grouped
and un-grouped heads, and contexts that leave cluster ranks empty (1, 7), split unevenly (130, 513) or
fill them exactly (512).  The 72B decode benchmark runs cluster 8 x head_dim 128 x GQA 8:1.

Tolerance: 1e-3 relative L2 on the fp16 output (the kernel adds the per-position terms warp by warp and
CTA by CTA, the oracle strictly in position order; device expf / sincosf / powf are not libm's), and
most elements bit-identical.
"""
import numpy as np
import pytest

from conftest import rel_l2
from prism_engine_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _case(backend, oracle, hd, nh, nkv, cluster, ctx_len, rope_k, base, seed):
    kvd = nkv * hd
    max_seq = 1024
    backend.set_option("attn_cluster", cluster)
    backend.kv_init(1, kvd, max_seq)
    rng_seed = seed * 1000 + hd + cluster
    K = synth.make_activation((ctx_len, kvd), seed=rng_seed)
    V = synth.make_activation((ctx_len, kvd), seed=rng_seed + 1)
    q = synth.make_activation(nh * hd, seed=rng_seed + 2)
    # what the cache holds for the earlier positions: K rotated at its own position when the profile asks
    Kc = np.stack([oracle.rope(K[p], p, hd, base) if rope_k else K[p] for p in range(ctx_len)])
    for p in range(ctx_len - 1):
        backend.append_kv(0, Kc[p], V[p], p)
    pos = ctx_len - 1
    got = backend.attention_step_kv(0, q, K[pos], V[pos], pos, nh, nkv, hd, rope_k=rope_k, rope_base=base)
    want = oracle.attention(oracle.rope(q, pos, hd, base), Kc.reshape(-1), V.reshape(-1), nh, nkv, hd, ctx_len)
    err = rel_l2(got, want)
    same = float(np.mean(got == want))
    assert err <= TOL, (hd, nh, nkv, cluster, ctx_len, err)
    assert same > 0.85, (hd, nh, nkv, cluster, ctx_len, same)
    # the kernel also appended this token's (rotated) k and v: a second query over the same cache, through
    # the plain attention entry point, must see them
    again = backend.attention_kv(0, oracle.rope(q, pos, hd, base), ctx_len, nh, nkv, hd)
    assert rel_l2(again, want) <= TOL
    backend.set_option("attn_cluster", 0)


@pytest.mark.parametrize("cluster", [1, 2, 4, 8])
@pytest.mark.parametrize("hd", [32, 64, 128, 256])
def test_fused_attention_clusters_and_head_sizes(backend, oracle, cluster, hd):
    # GQA 8:1 (the 72B shape), contexts: one position, fewer positions than CTAs, ragged, one past a power of two
    for ctx_len in (1, 7, 130, 513):
        _case(backend, oracle, hd, nh=8, nkv=1, cluster=cluster, ctx_len=ctx_len, rope_k=True, base=1e6, seed=ctx_len)


@pytest.mark.parametrize("cluster", [1, 8])
def test_fused_attention_ungrouped_heads_rope_q_only(backend, oracle, cluster):
    # 1:1 heads, the reference CPU profile: base 10000, K cached un-rotated
    for hd, ctx_len in ((64, 40), (128, 512), (128, 513)):
        _case(backend, oracle, hd, nh=4, nkv=4, cluster=cluster, ctx_len=ctx_len, rope_k=False, base=10000.0, seed=3)


def test_fused_attention_72b_head_layout(backend, oracle):
    # 64 query heads over 8 KV heads of 128, the cluster size the engine picks for max_seq >= 512 (8)
    _case(backend, oracle, 128, nh=64, nkv=8, cluster=0, ctx_len=515, rope_k=True, base=1e6, seed=9)


@pytest.mark.parametrize("group", [1, 2, 4])
def test_fused_attention_fewer_heads_per_cluster(backend, oracle, group):
    # the head group split over several clusters: 7 query heads per KV head (the 0.5B layout, which the launcher
    # splits by itself) and 8, with the last cluster of a group only partly filled when 7 is not a multiple
    backend.set_option("attn_group", group)
    try:
        _case(backend, oracle, 64, nh=14, nkv=2, cluster=2, ctx_len=141, rope_k=True, base=1e6, seed=11)
        _case(backend, oracle, 128, nh=16, nkv=2, cluster=4, ctx_len=300, rope_k=True, base=1e6, seed=12)
    finally:
        backend.set_option("attn_group", 0)


def test_kv_entry_points_mirror_the_backend_cache(backend, oracle):
    """append_kv ignores rows outside the cache (as MetalBackend::append_kv does); the C call reports them."""
    import prism_engine_b200 as p

    backend.kv_init(2, 64, 16)
    k = synth.make_activation(64, seed=1)
    backend.append_kv(5, k, k, 0)        # layer out of range: ignored by the mirror
    backend.append_kv(0, k, k, 99)       # token out of range: ignored by the mirror
    with pytest.raises(p.PrismCudaError) as e:
        backend._ck(backend.L.prism_cuda_kv_append(backend.ctx, 5, k.ctypes.data, k.ctypes.data, 0))
    assert e.value.code == -2
    for t in range(3):
        backend.append_kv(1, synth.make_activation(64, seed=10 + t), synth.make_activation(64, seed=20 + t), t)
    Kc = np.concatenate([synth.make_activation(64, seed=10 + t) for t in range(3)])
    Vc = np.concatenate([synth.make_activation(64, seed=20 + t) for t in range(3)])
    q = synth.make_activation(4 * 32, seed=5)
    got = backend.attention_kv(1, q, 3, 4, 2, 32)
    assert rel_l2(got, oracle.attention(q, Kc, Vc, 4, 2, 32, 3)) <= TOL

"""Host-side mirror of the reference's backend surface, over the C ABI.

``CudaBackend`` has the method set of ``MetalBackend``
(src/lut/engine_impl.rs:26-492): ``gemv(key, inp, out)``,
``fused_gate_up(gate_key, up_key, input, output)``, ``attention``,
``norm``, ``rope``, ``softmax``, ``silu``, ``vec_add`` -- same argument
meaning, and an error where the reference returns ``Err(String)`` (here a
``PrismCudaError`` carrying that text).  ``PrismEngine`` mirrors
``PrismEngine::{load, generate}`` (engine_impl.rs:597, 933).  fp16 data is
numpy ``uint16`` bit patterns, as ``&[u16]`` in the reference.

Every call runs on the GPU through ``libprism_cuda.so``; nothing here computes
on the CPU.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, Optional, Tuple

import numpy as np

from . import _lib
from ._lib import ModelConfig, PrismCudaError, check

ROLE = {"q": 0, "k": 1, "v": 2, "o": 3, "gate": 4, "up": 5, "down": 6, "embed": 7, "lm_head": 8}


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _u16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


class CudaBackend:
    """One CUDA context on one B200: the peer of ``MetalBackend``."""

    def __init__(self, tensors: Optional[Dict[str, Tuple[np.ndarray, int, int]]] = None, device: int = 0,
                 bits: int = 4):
        """``tensors``: key -> (payload bytes, dim_m, dim_n), the map ``MetalBackend::new`` receives
        (``HashMap<String, CompiledTensor>``, engine_impl.rs:51-57); each payload is uploaded and re-laid."""
        self.L = _lib.load()
        h = C.c_void_p()
        rc = self.L.prism_cuda_create(device, C.byref(h))
        if rc != 0:
            msg = self.L.prism_cuda_last_error(None)
            raise PrismCudaError(rc, msg.decode() if msg else "")
        self.ctx = h
        self.device = device
        self.handles: Dict[str, int] = {}
        self._engines = weakref.WeakSet()  # engines built on this context: destroyed before it
        for key, (payload, dm, dn) in (tensors or {}).items():
            self.upload(key, payload, dm, dn, bits)

    # -- lifetime -----------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "ctx", None):
            for eng in list(self._engines):
                eng.close()
            self.L.prism_cuda_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _ck(self, rc: int) -> None:
        check(self.ctx, rc)

    # -- options / introspection -----------------------------------------------------------------
    def set_option(self, key: str, value: int) -> None:
        self._ck(self.L.prism_cuda_set_option(self.ctx, key.encode(), value))

    def launch_count(self) -> int:
        return int(self.L.prism_cuda_launch_count(self.ctx))

    def stream(self) -> int:
        return int(self.L.prism_cuda_stream(self.ctx) or 0)

    def synchronize(self) -> None:
        self._ck(self.L.prism_cuda_synchronize(self.ctx))

    # -- weights ---------------------------------------------------------------------------------------
    def upload(self, key: str, payload, dim_m: int, dim_n: int, bits: int = 4, shard=None) -> int:
        payload = np.ascontiguousarray(payload, dtype=np.uint8)
        h = C.c_int32(-1)
        if shard is None:
            rc = self.L.prism_cuda_upload_palettized(self.ctx, key.encode(), _ptr(payload), payload.size, dim_m,
                                                     dim_n, bits, C.byref(h))
        else:
            row0, rows, col0, cols = shard
            rc = self.L.prism_cuda_upload_palettized_shard(self.ctx, key.encode(), _ptr(payload), payload.size,
                                                           dim_m, dim_n, bits, row0, rows, col0, cols, C.byref(h))
        self._ck(rc)
        self.handles[key] = h.value
        return h.value

    def synth(self, key: str, dim_m: int, dim_n: int, bits: int = 4, seed: int = 0, sigma: float = 0.02) -> int:
        h = C.c_int32(-1)
        self._ck(self.L.prism_cuda_synth_palettized(self.ctx, key.encode(), dim_m, dim_n, bits, seed, sigma, C.byref(h)))
        self.handles[key] = h.value
        return h.value

    def find(self, key: str) -> int:
        h = C.c_int32(-1)
        self._ck(self.L.prism_cuda_find_tensor(self.ctx, key.encode(), C.byref(h)))
        return h.value

    def dims(self, handle: int) -> Tuple[int, int, int]:
        m, n, b = C.c_uint32(), C.c_uint32(), C.c_uint32()
        self._ck(self.L.prism_cuda_tensor_dims(self.ctx, handle, C.byref(m), C.byref(n), C.byref(b)))
        return m.value, n.value, b.value

    def free(self, handle: int) -> None:
        self._ck(self.L.prism_cuda_free_tensor(self.ctx, handle))

    def download_payload(self, handle: int) -> np.ndarray:
        m, n, b = self.dims(handle)
        out = np.empty(m * (2 << b) + m * (n * b // 8), np.uint8)
        self._ck(self.L.prism_cuda_download_payload(self.ctx, handle, _ptr(out), out.size))
        return out

    def dequant(self, handle: int) -> np.ndarray:
        m, n, _ = self.dims(handle)
        out = np.empty((m, n), np.uint16)
        self._ck(self.L.prism_cuda_dequant(self.ctx, handle, _ptr(out)))
        return out

    # -- MetalBackend::gemv (engine_impl.rs:155-190) --------------------------------------------------------
    def gemv(self, key, inp, out: Optional[np.ndarray] = None) -> np.ndarray:
        inp = _u16(inp)
        if isinstance(key, str):
            h = self.find(key)
        else:
            h = key
        m, n, _ = self.dims(h)
        if inp.size != n:
            raise PrismCudaError(_lib.E_ARG, f"gemv: input has {inp.size} elements, tensor needs {n}")
        if out is None:
            out = np.empty(m, np.uint16)
        elif out.size != m or out.dtype != np.uint16 or not out.flags.c_contiguous:
            raise PrismCudaError(_lib.E_ARG, f"gemv: output must be contiguous uint16[{m}]")
        self._ck(self.L.prism_cuda_gemv(self.ctx, h, _ptr(inp), _ptr(out)))
        return out

    # -- MetalBackend::fused_gate_up (engine_impl.rs:443-490) ----------------------------------------------------
    def fused_gate_up(self, gate_key, up_key, input, output: Optional[np.ndarray] = None) -> np.ndarray:
        x = _u16(input)
        hg = self.find(gate_key) if isinstance(gate_key, str) else gate_key
        hu = self.find(up_key) if isinstance(up_key, str) else up_key
        m, n, _ = self.dims(hg)
        if x.size != n:
            raise PrismCudaError(_lib.E_ARG, f"fused_gate_up: input has {x.size} elements, tensor needs {n}")
        if output is None:
            output = np.empty(m, np.uint16)
        self._ck(self.L.prism_cuda_fused_gate_up(self.ctx, hg, hu, _ptr(x), _ptr(output)))
        return output

    def mlp(self, gate, up, down, x) -> np.ndarray:
        x = _u16(x)
        hs = [self.find(k) if isinstance(k, str) else k for k in (gate, up, down)]
        m, _, _ = self.dims(hs[2])
        out = np.empty(m, np.uint16)
        self._ck(self.L.prism_cuda_mlp(self.ctx, hs[0], hs[1], hs[2], _ptr(x), _ptr(out)))
        return out

    def gemm(self, key, X) -> np.ndarray:
        X = _u16(X)
        h = self.find(key) if isinstance(key, str) else key
        m, n, _ = self.dims(h)
        if X.ndim != 2 or X.shape[1] != n:
            raise PrismCudaError(_lib.E_ARG, f"gemm: X must be [m_tok, {n}]")
        Y = np.empty((X.shape[0], m), np.uint16)
        self._ck(self.L.prism_cuda_gemm(self.ctx, h, _ptr(X), X.shape[0], _ptr(Y)))
        return Y

    # -- device-pointer variants (ints are raw device addresses, e.g. torch.Tensor.data_ptr()) -------------------
    def gemv_dev(self, handle: int, x_dev: int, y_dev: int) -> None:
        self._ck(self.L.prism_cuda_gemv_dev(self.ctx, handle, x_dev, y_dev))

    def gemv_static_dev(self, handle: int, x_dev: int, y_dev: int) -> None:
        """GEMV that never allocates: split-K scratch comes from a fixed array inside the library
        (for hosts whose own pools already own all of HBM).  Rejects shapes beyond that array."""
        self._ck(self.L.prism_cuda_gemv_static_dev(self.ctx, handle, x_dev, y_dev))

    def fused_gate_up_dev(self, gate: int, up: int, x_dev: int, out_dev: int) -> None:
        self._ck(self.L.prism_cuda_fused_gate_up_dev(self.ctx, gate, up, x_dev, out_dev))

    def mlp_dev(self, gate: int, up: int, down: int, x_dev: int, out_dev: int) -> None:
        self._ck(self.L.prism_cuda_mlp_dev(self.ctx, gate, up, down, x_dev, out_dev))

    def gemm_dev(self, handle: int, X_dev: int, m_tok: int, Y_dev: int) -> None:
        self._ck(self.L.prism_cuda_gemm_dev(self.ctx, handle, X_dev, m_tok, Y_dev))

    # -- MetalBackend::{norm_metal, rope_metal, softmax_metal, silu_metal, vec_add_metal, attention} -----------------
    def norm(self, input, eps: float) -> np.ndarray:
        x = _u16(input)
        out = np.empty_like(x)
        self._ck(self.L.prism_cuda_rms_norm(self.ctx, _ptr(x), _ptr(out), x.size, eps))
        return out

    def rope(self, x, pos: int, hd: int, base: float = 10000.0) -> np.ndarray:
        x = _u16(x).copy()
        self._ck(self.L.prism_cuda_rope(self.ctx, _ptr(x), x.size, pos, hd, base))
        return x

    def softmax(self, input) -> np.ndarray:
        x = _u16(input)
        out = np.empty_like(x)
        self._ck(self.L.prism_cuda_softmax(self.ctx, _ptr(x), _ptr(out), x.size))
        return out

    def silu(self, data) -> np.ndarray:
        x = _u16(data).copy()
        self._ck(self.L.prism_cuda_silu(self.ctx, _ptr(x), x.size))
        return x

    def vec_add(self, a, b) -> np.ndarray:
        a, b = _u16(a).copy(), _u16(b)
        n = min(a.size, b.size)
        self._ck(self.L.prism_cuda_vec_add(self.ctx, _ptr(a), _ptr(b), n))
        return a

    def attention(self, q, k, v, seq_len: int, num_heads: int, kv_heads: int, head_dim: int) -> np.ndarray:
        q, k, v = _u16(q), _u16(k), _u16(v)
        out = np.zeros(num_heads * head_dim, np.uint16)
        kvd = kv_heads * head_dim
        if k.size < seq_len * kvd or v.size < seq_len * kvd:
            return out  # the reference returns zeros on a short cache (engine_impl.rs:207-209)
        self._ck(self.L.prism_cuda_attention(self.ctx, _ptr(q), _ptr(k), _ptr(v), seq_len, num_heads, kv_heads,
                                             head_dim, _ptr(out)))
        return out

    def argmax(self, logits) -> int:
        lg = _u16(logits)
        idx = C.c_uint32()
        self._ck(self.L.prism_cuda_argmax(self.ctx, _ptr(lg), lg.size, C.byref(idx)))
        return idx.value

    def bench_cycle(self, kind: int, handles, reps: int, x_dev: int) -> float:
        """ms for `reps` replays of a graph cycling through the given weight sets with the device activations
        ``x_dev`` (see prism_cuda_bench_cycle)."""
        hs = np.ascontiguousarray(handles, dtype=np.int32).reshape(-1)
        per = kind + 1
        ms = C.c_double()
        self._ck(self.L.prism_cuda_bench_cycle(self.ctx, kind, hs.ctypes.data_as(C.POINTER(C.c_int32)),
                                               hs.size // per, reps, x_dev, C.byref(ms)))
        return ms.value

    def bench_gemm(self, handle: int, X_dev: int, m_tok: int, reps: int) -> float:
        """ms for `reps` prefill GEMMs of the device activations ``X_dev`` [m_tok][dim_n] against one tensor."""
        ms = C.c_double()
        self._ck(self.L.prism_cuda_bench_gemm(self.ctx, handle, X_dev, m_tok, reps, C.byref(ms)))
        return ms.value

    def load_cimage(self, path: str, cache: Optional[str] = None):
        """Uploads every palettized tensor of a reference-format ``.cimage``.  ``cache``: path of the cache
        of the re-laid image ("" = beside the file); returns ``(n, hit)`` then, else ``n``."""
        n = C.c_uint32()
        if cache is None:
            self._ck(self.L.prism_cuda_load_cimage(self.ctx, path.encode(), C.byref(n)))
            return n.value
        hit = C.c_int()
        self._ck(self.L.prism_cuda_load_cimage_cached(self.ctx, path.encode(), cache.encode(), C.byref(n), C.byref(hit)))
        return n.value, bool(hit.value)

    def cimage_plan(self) -> dict:
        """``ExecutionPlan`` of the last container loaded (src/lut/graph.rs:552-589); version 0 = none."""
        pl = _lib.CImagePlan()
        self._ck(self.L.prism_cuda_cimage_plan(self.ctx, C.byref(pl)))
        return {"version": pl.version, "num_layers": pl.num_layers, "n_nodes": pl.n_nodes,
                "n_gemm_nodes": pl.n_gemm_nodes, "kv_cache": {1: "Fp16", 0: "Int8"}.get(pl.kv_fp16),
                "architecture": pl.architecture.decode(), "attention_strategy": pl.attention_strategy.decode(),
                "lm_head_backend": pl.lm_head_backend.decode()}

    # -- MetalBackend::{append_kv, attention} over the backend-held cache (engine_impl.rs:109-119, 256-286) ---
    def kv_init(self, num_layers: int, kv_dim: int, max_seq: int = 4096) -> None:
        self._ck(self.L.prism_cuda_kv_init(self.ctx, num_layers, kv_dim, max_seq))
        self._kv_shape = (num_layers, kv_dim, max_seq)

    def append_kv(self, layer: int, k, v, token_idx: int) -> None:
        """``MetalBackend::append_kv``: a layer or token outside the cache is ignored, as there."""
        k, v = _u16(k), _u16(v)
        nl, kvd, ms = getattr(self, "_kv_shape", (0, 0, 0))
        if layer >= nl or token_idx >= ms or kvd == 0:
            return
        if k.size != kvd or v.size != kvd:
            raise PrismCudaError(_lib.E_ARG, f"append_kv: k and v must have {kvd} elements")
        self._ck(self.L.prism_cuda_kv_append(self.ctx, layer, _ptr(k), _ptr(v), token_idx))

    def attention_kv(self, layer: int, q, seq_len: int, num_heads: int, kv_heads: int, head_dim: int) -> np.ndarray:
        q = _u16(q)
        out = np.zeros(num_heads * head_dim, np.uint16)
        self._ck(self.L.prism_cuda_attention_kv(self.ctx, layer, _ptr(q), seq_len, num_heads, kv_heads, head_dim, _ptr(out)))
        return out

    # -- tensor parallel ------------------------------------------------------------------------------------------
    @staticmethod
    def tp_unique_id() -> bytes:
        L = _lib.load()
        buf = (C.c_uint8 * _lib.NCCL_ID_BYTES)()
        rc = L.prism_cuda_tp_unique_id(buf)
        if rc != 0:
            msg = L.prism_cuda_last_error(None)
            raise PrismCudaError(rc, msg.decode() if msg else "")
        return bytes(buf)

    def tp_init(self, world: int, rank: int, uid: bytes) -> None:
        buf = (C.c_uint8 * _lib.NCCL_ID_BYTES).from_buffer_copy(uid)
        self._ck(self.L.prism_cuda_tp_init(self.ctx, world, rank, buf))

    def palettize(self, weights: np.ndarray, k: int = 16, max_iter: int = 50) -> np.ndarray:
        """``palettize_matrix`` (src/quantization/palette.rs:230-275) + payload assembly
        (src/lut/compiler.rs:50-61) on the GPU: fp32 ``weights[dim_m][dim_n]`` -> the reference payload
        bytes, bit-identical to the CPU quantiser."""
        w = np.ascontiguousarray(weights, dtype=np.float32)
        dm, dn = w.shape
        out = np.empty(dm * 32 + dm * (dn // 2), dtype=np.uint8)
        self._ck(self.L.prism_cuda_palettize(self.ctx, w.ctypes.data_as(C.POINTER(C.c_float)), dm, dn, k, max_iter,
                                             out.ctypes.data_as(C.POINTER(C.c_uint8)), out.size))
        return out

    def tp_peer_ready(self) -> bool:
        """True when the row-parallel partial sums are reduced through peer memory (else NCCL)."""
        return bool(self.L.prism_cuda_tp_peer_ready(self.ctx))

    def attention_step_kv(self, layer: int, q, k, v, token_idx: int, num_heads: int, kv_heads: int, head_dim: int,
                          rope_k: bool = True, rope_base: float = 10000.0) -> np.ndarray:
        """Rope(q), Rope(k), cache append and attention of one decode step in one kernel, on the backend-held cache."""
        q, k, v = _u16(q), _u16(k), _u16(v)
        out = np.zeros(num_heads * head_dim, np.uint16)
        self._ck(self.L.prism_cuda_attention_step_kv(self.ctx, layer, _ptr(q), _ptr(k), _ptr(v), token_idx, num_heads,
                                                     kv_heads, head_dim, int(rope_k), rope_base, _ptr(out)))
        return out

    def tp_peer_reason(self) -> str:
        r = self.L.prism_cuda_tp_peer_reason(self.ctx)
        return r.decode() if r else ""

    def tp_init_loopback(self, world: int, rank: int) -> None:
        """One-GPU diagnostic group whose peers never deliver (see ``prism_cuda_tp_init_loopback``)."""
        self._ck(self.L.prism_cuda_tp_init_loopback(self.ctx, world, rank))

    def tp_all_reduce_resid_dev(self, partial_dev: int, h_dev: int, n: int) -> None:
        self._ck(self.L.prism_cuda_tp_all_reduce_resid_dev(self.ctx, partial_dev, h_dev, n))


def model_config(num_layers, hidden_size, num_heads, num_kv_heads, head_dim, intermediate_size, vocab_size,
                 norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True, bits=4, max_seq=4096, max_batch=1,
                 profile="baseline", kv_page_size=0, kv_pool_pages=0) -> ModelConfig:
    """``profile``: "reference_cpu" keeps every behaviour of the reference's CPU path (RoPE base
    10000 on q only, int8 KV, the DownProj dim test); "baseline" is the configuration the
    benchmarks name (rope_theta from the config on q and k, fp16 KV, DownProj runs)."""
    ref = profile == "reference_cpu"
    if profile not in ("reference_cpu", "baseline"):
        raise ValueError(profile)
    return ModelConfig(num_layers, hidden_size, num_heads, num_kv_heads, head_dim, intermediate_size, vocab_size,
                       norm_eps, rope_theta, int(tie_word_embeddings), bits, max_seq, max_batch,
                       0 if ref else 1, 0 if ref else 1, 1 if ref else 0, 1 if ref else 0, kv_page_size, kv_pool_pages)


QWEN25_0P5B = dict(num_layers=24, hidden_size=896, num_heads=14, num_kv_heads=2, head_dim=64,
                   intermediate_size=4864, vocab_size=151936, norm_eps=1e-6, rope_theta=1e6,
                   tie_word_embeddings=True)
QWEN25_72B = dict(num_layers=80, hidden_size=8192, num_heads=64, num_kv_heads=8, head_dim=128,
                  intermediate_size=29568, vocab_size=152064, norm_eps=1e-6, rope_theta=1e6,
                  tie_word_embeddings=False)
QWEN25_7B = dict(num_layers=28, hidden_size=3584, num_heads=28, num_kv_heads=4, head_dim=128,
                 intermediate_size=18944, vocab_size=152064, norm_eps=1e-6, rope_theta=1e6,
                 tie_word_embeddings=False)


class PrismEngine:
    """Mirror of ``PrismEngine`` (src/lut/engine_impl.rs:503-512) with every op on the device."""

    def __init__(self, backend: CudaBackend, cfg: ModelConfig):
        self.be = backend
        self.cfg = cfg
        self.L = backend.L
        h = C.c_void_p()
        check(backend.ctx, self.L.prism_cuda_engine_create(backend.ctx, C.byref(cfg), C.byref(h)))
        self.h = h
        backend._engines.add(self)

    @classmethod
    def load(cls, backend: CudaBackend, path: str, cfg: ModelConfig, key_prefix: str = "model") -> "PrismEngine":
        """``PrismEngine::load`` (engine_impl.rs:597): read a ``.cimage``, upload, bind."""
        eng = cls(backend, cfg)
        check(backend.ctx, eng.L.prism_cuda_engine_load_cimage(eng.h, path.encode(), key_prefix.encode()))
        return eng

    def close(self) -> None:
        if getattr(self, "h", None):
            self.L.prism_cuda_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc):
        check(self.be.ctx, rc)

    def bind(self, role: str, layer: int, handle: int) -> None:
        self._ck(self.L.prism_cuda_engine_bind(self.h, ROLE[role], layer, handle))

    def bind_by_keys(self, prefix: str = "model") -> None:
        self._ck(self.L.prism_cuda_engine_bind_by_keys(self.h, prefix.encode()))

    def synth_weights(self, seed: int = 0, sigma: float = 0.02) -> None:
        self._ck(self.L.prism_cuda_engine_synth_weights(self.h, seed, sigma))

    def generate(self, prompt, max_new: int, return_logits: bool = False):
        """``PrismEngine::generate`` (engine_impl.rs:933): prompt is [n] or [batch, n] token ids."""
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        single = p.ndim == 1
        if single:
            p = p[None, :]
        batch, n = p.shape
        out = np.empty((batch, max_new), np.uint32)
        lg = np.empty((batch, self.cfg.vocab_size), np.uint16) if return_logits else None
        self._ck(self.L.prism_cuda_engine_generate(self.h, _ptr(p), batch, n, max_new, _ptr(out),
                                                   _ptr(lg) if lg is not None else None))
        if single:
            out = out[0]
            lg = lg[0] if lg is not None else None
        return (out, lg) if return_logits else out

    def reset(self, batch: int = 1) -> None:
        self._ck(self.L.prism_cuda_engine_reset(self.h, batch))

    def step(self, tokens, want_logits: bool = False):
        t = np.ascontiguousarray(np.atleast_1d(tokens), dtype=np.uint32)
        nxt = np.empty(t.size, np.uint32)
        lg = np.empty((t.size, self.cfg.vocab_size), np.uint16) if want_logits else None
        self._ck(self.L.prism_cuda_engine_step(self.h, _ptr(t), _ptr(nxt), _ptr(lg) if lg is not None else None))
        return (nxt, lg) if want_logits else nxt

    def decode(self, tokens_in, n_steps: int, out: Optional[np.ndarray] = None, tokens_ptr: Optional[int] = None,
               out_ptr: Optional[int] = None) -> Optional[np.ndarray]:
        """Runs ``n_steps`` greedy steps on the device.  ``tokens_ptr``/``out_ptr`` pass raw host
        addresses (e.g. pinned torch tensors) instead of numpy arrays."""
        if tokens_ptr is None:
            t = np.ascontiguousarray(np.atleast_1d(tokens_in), dtype=np.uint32)
            tokens_ptr = _ptr(t)
            batch = t.size
            if out is None:
                out = np.empty((batch, n_steps), np.uint32)
            out_ptr = _ptr(out)
        self._ck(self.L.prism_cuda_engine_decode(self.h, tokens_ptr, n_steps, out_ptr))
        return out

    def step_bytes(self) -> int:
        return int(self.L.prism_cuda_engine_step_bytes(self.h))

    def last_ms(self) -> float:
        return float(self.L.prism_cuda_engine_last_ms(self.h))

    def position(self) -> int:
        return int(self.L.prism_cuda_engine_position(self.h))

    def last_device_ms(self) -> float:
        return float(self.L.prism_cuda_engine_last_device_ms(self.h))

    def kernels_per_step(self) -> int:
        return int(self.L.prism_cuda_engine_kernels_per_step(self.h))

    def profile_part(self, part: int, reps: int = 1):
        """(ms, launches) of `reps` passes over one kind of launch of a step: 1 = attention, 2 = TP reductions."""
        ms, ln = C.c_double(), C.c_uint32()
        self._ck(self.L.prism_cuda_engine_profile_part(self.h, part, reps, C.byref(ms), C.byref(ln)))
        return ms.value, ln.value

    def profile_gemv(self, reps: int = 1):
        """(ms, algorithmic bytes, launches) of `reps` passes over the model's GEMV launches only."""
        ms, by, ln = C.c_double(), C.c_uint64(), C.c_uint32()
        self._ck(self.L.prism_cuda_engine_profile_gemv(self.h, reps, C.byref(ms), C.byref(by), C.byref(ln)))
        return ms.value, by.value, ln.value

"""ctypes binding of the CPU oracle (``oracle/prism_oracle.c``).

Test infrastructure only: the test-suite, the smoke check and the benchmark's
CPU-baseline leg import this module; the product package never does.  All
arrays are numpy; fp16 values travel as ``uint16`` bit patterns, exactly as the
reference carries them (``&[u16]`` in src/lut/cpu_fallback.rs).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libprism_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe in ``oracle/Makefile``."""
    src = os.path.join(_HERE, "prism_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "CC=gcc"], stdout=subprocess.DEVNULL)
    return _SO


class Cfg(C.Structure):
    """Mirror of ``po_cfg``."""

    _fields_ = [
        ("num_layers", C.c_uint32), ("hidden", C.c_uint32), ("heads", C.c_uint32),
        ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("inter", C.c_uint32),
        ("vocab", C.c_uint32), ("eps", C.c_float), ("rope_theta", C.c_float),
        ("bits", C.c_uint32), ("tie_embeddings", C.c_uint32),
        ("rope_use_theta", C.c_uint32), ("rope_k", C.c_uint32), ("kv_int8", C.c_uint32),
        ("down_guard", C.c_uint32), ("threads", C.c_int32),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        u16p, u8p, u32p, f32p = (C.POINTER(C.c_uint16), C.POINTER(C.c_uint8),
                                 C.POINTER(C.c_uint32), C.POINTER(C.c_float))
        L.po_f16_to_f32.restype = C.c_float
        L.po_f16_to_f32.argtypes = [C.c_uint16]
        L.po_f32_to_f16.restype = C.c_uint16
        L.po_f32_to_f16.argtypes = [C.c_float]
        L.po_payload_bytes.restype = C.c_uint64
        L.po_payload_bytes.argtypes = [C.c_uint32] * 3
        L.po_lut_gemv.argtypes = [u16p, u8p, C.c_uint32, C.c_uint32, u16p]
        L.po_lut_gemv_bits.argtypes = [u16p, u8p, C.c_uint32, C.c_uint32, C.c_uint32, u16p, C.c_int]
        L.po_lut_gemm.argtypes = [u16p, C.c_uint32, u8p, C.c_uint32, C.c_uint32, C.c_uint32, u16p, C.c_int]
        L.po_embed.argtypes = [C.c_uint32, u8p, C.c_uint32, C.c_uint32, C.c_uint32, u16p]
        L.po_dequant.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, u16p]
        L.po_rms_norm.argtypes = [u16p, C.c_uint32, C.c_float]
        L.po_vec_add.argtypes = [u16p, u16p, C.c_uint32]
        L.po_silu.argtypes = [u16p, C.c_uint32]
        L.po_gelu.argtypes = [u16p, C.c_uint32]
        L.po_mul.argtypes = [u16p, u16p, C.c_uint32]
        L.po_rope.argtypes = [u16p, C.c_uint32, C.c_int64, C.c_uint32, C.c_float]
        L.po_attention.argtypes = [u16p, u16p, u16p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, u16p]
        L.po_argmax.restype = C.c_uint32
        L.po_argmax.argtypes = [u16p, C.c_uint32]
        L.po_top2_margin.restype = C.c_float
        L.po_top2_margin.argtypes = [u16p, C.c_uint32]
        L.po_kv_quant.argtypes = [u16p, C.c_uint32, u8p]
        L.po_kv_dequant.argtypes = [u8p, C.c_uint32, C.c_uint32, u16p]
        L.po_mlp.argtypes = [u8p, u8p, u8p, u16p, C.c_uint32, C.c_uint32, C.c_uint32, u16p, u16p, C.c_int]
        L.po_model_create.restype = C.c_void_p
        L.po_model_create.argtypes = [C.POINTER(Cfg)]
        L.po_model_set_tensor.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, u8p]
        L.po_model_reset.argtypes = [C.c_void_p]
        L.po_model_destroy.argtypes = [C.c_void_p]
        L.po_model_step.restype = u16p
        L.po_model_step.argtypes = [C.c_void_p, C.c_uint32, C.c_int64]
        L.po_model_generate.argtypes = [C.c_void_p, u32p, C.c_uint32, C.c_uint32, u32p, f32p]
        L.po_encode_channel.restype = C.c_float
        L.po_encode_channel.argtypes = [f32p, C.c_uint32, f32p, C.c_uint32, u8p]
        L.po_fit_palette.restype = C.c_uint32
        L.po_fit_palette.argtypes = [f32p, C.c_uint32, C.c_uint32, C.c_uint32, f32p]
        L.po_palettize_to_payload.argtypes = [f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, u8p]
        L.po_max_threads.restype = C.c_int
        L.po_init()
        _lib = L
    return _lib


def _p(a: np.ndarray, ty):
    return a.ctypes.data_as(C.POINTER(ty))


def _u16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def payload_bytes(m: int, k: int, bits: int = 4) -> int:
    return int(lib().po_payload_bytes(m, k, bits))


def lut_gemv(x, payload, dm: int, dn: int, bits: int = 4, threads: int = 1) -> np.ndarray:
    """``lut_gemv_cpu`` (src/lut/cpu_fallback.rs:12-35); bits=2 is the 4-entry generalisation."""
    x, payload = _u16(x), _u8(payload)
    assert payload.size >= payload_bytes(dm, dn, bits) and x.size >= dn
    y = np.empty(dm, np.uint16)
    if bits == 4 and threads <= 1:
        lib().po_lut_gemv(_p(x, C.c_uint16), _p(payload, C.c_uint8), dm, dn, _p(y, C.c_uint16))
    else:
        lib().po_lut_gemv_bits(_p(x, C.c_uint16), _p(payload, C.c_uint8), dm, dn, bits,
                               _p(y, C.c_uint16), threads)
    return y


def lut_gemm(X, payload, dm: int, dn: int, bits: int = 4, threads: int = 1) -> np.ndarray:
    """Prefill semantics: one ``lut_gemv_cpu`` per activation row (engine_impl.rs:1046-1053)."""
    X, payload = _u16(X), _u8(payload)
    m_tok = X.shape[0]
    Y = np.empty((m_tok, dm), np.uint16)
    lib().po_lut_gemm(_p(X, C.c_uint16), m_tok, _p(payload, C.c_uint8), dm, dn, bits,
                      _p(Y, C.c_uint16), threads)
    return Y


def embed(token: int, payload, vocab: int, hd: int, bits: int = 4) -> np.ndarray:
    payload = _u8(payload)
    out = np.empty(hd, np.uint16)
    lib().po_embed(token, _p(payload, C.c_uint8), vocab, hd, bits, _p(out, C.c_uint16))
    return out


def dequant(payload, dm: int, dn: int, bits: int = 4) -> np.ndarray:
    payload = _u8(payload)
    out = np.empty((dm, dn), np.uint16)
    lib().po_dequant(_p(payload, C.c_uint8), dm, dn, bits, _p(out, C.c_uint16))
    return out


def rms_norm(x, eps: float) -> np.ndarray:
    x = _u16(x).copy()
    lib().po_rms_norm(_p(x, C.c_uint16), x.size, eps)
    return x


def vec_add(a, b) -> np.ndarray:
    a, b = _u16(a).copy(), _u16(b)
    lib().po_vec_add(_p(a, C.c_uint16), _p(b, C.c_uint16), a.size)
    return a


def silu(x) -> np.ndarray:
    x = _u16(x).copy()
    lib().po_silu(_p(x, C.c_uint16), x.size)
    return x


def gelu(x) -> np.ndarray:
    x = _u16(x).copy()
    lib().po_gelu(_p(x, C.c_uint16), x.size)
    return x


def mul(g, u) -> np.ndarray:
    g, u = _u16(g).copy(), _u16(u)
    lib().po_mul(_p(g, C.c_uint16), _p(u, C.c_uint16), g.size)
    return g


def rope(x, pos: int, hd: int, base: float = 10000.0) -> np.ndarray:
    x = _u16(x).copy()
    lib().po_rope(_p(x, C.c_uint16), x.size, pos, hd, base)
    return x


def attention(q, kc, vc, nh: int, nkv: int, hd: int, sl: int) -> np.ndarray:
    q, kc, vc = _u16(q), _u16(kc), _u16(vc)
    o = np.empty(nh * hd, np.uint16)
    lib().po_attention(_p(q, C.c_uint16), _p(kc, C.c_uint16), _p(vc, C.c_uint16), nh, nkv, hd, sl,
                       _p(o, C.c_uint16))
    return o


def argmax(logits) -> int:
    logits = _u16(logits)
    return int(lib().po_argmax(_p(logits, C.c_uint16), logits.size))


def top2_margin(logits) -> float:
    logits = _u16(logits)
    return float(lib().po_top2_margin(_p(logits, C.c_uint16), logits.size))


def kv_quant(x) -> np.ndarray:
    x = _u16(x)
    out = np.empty(4 + x.size, np.uint8)
    lib().po_kv_quant(_p(x, C.c_uint16), x.size, _p(out, C.c_uint8))
    return out


def kv_dequant(data, n_tok: int, kv_dim: int) -> np.ndarray:
    data = _u8(data)
    out = np.empty(n_tok * kv_dim, np.uint16)
    lib().po_kv_dequant(_p(data, C.c_uint8), n_tok, kv_dim, _p(out, C.c_uint16))
    return out


def mlp(wg, wu, wd, x, hidden: int, inter: int, bits: int = 4, threads: int = 1):
    """Returns (out[hidden], act[inter]); ``wd=None`` stops after the activation."""
    wg, wu, x = _u8(wg), _u8(wu), _u16(x)
    out = np.zeros(hidden, np.uint16)
    act = np.empty(inter, np.uint16)
    wdp = _p(_u8(wd), C.c_uint8) if wd is not None else None
    lib().po_mlp(_p(wg, C.c_uint8), _p(wu, C.c_uint8), wdp, _p(x, C.c_uint16), hidden, inter, bits,
                 _p(out, C.c_uint16), _p(act, C.c_uint16), threads)
    return out, act


def f16_bits(a) -> np.ndarray:
    """float array -> fp16 bit patterns (numpy's float16 cast is IEEE RNE)."""
    return np.asarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_vals(bits) -> np.ndarray:
    return _u16(bits).view(np.float16).astype(np.float32)


ROLE = {"q": 0, "k": 1, "v": 2, "o": 3, "gate": 4, "up": 5, "down": 6, "embed": 7, "lm_head": 8}


class Model:
    """Oracle twin of ``PrismEngine`` (src/lut/engine_impl.rs:503-512, 933-1459)."""

    def __init__(self, cfg: Cfg):
        self.cfg = cfg
        self._h = lib().po_model_create(C.byref(cfg))
        self._keep = []

    def set_tensor(self, role: str, layer: int, payload) -> None:
        payload = _u8(payload)
        self._keep.append(payload)
        lib().po_model_set_tensor(self._h, ROLE[role], layer, _p(payload, C.c_uint8))

    def step(self, token: int, pos: int) -> np.ndarray:
        ptr = lib().po_model_step(self._h, token, pos)
        return np.ctypeslib.as_array(ptr, shape=(self.cfg.vocab,)).copy()

    def reset(self) -> None:
        lib().po_model_reset(self._h)

    def generate(self, prompt, max_new: int):
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.empty(max_new, np.uint32)
        margins = np.empty(max_new, np.float32)
        lib().po_model_generate(self._h, _p(prompt, C.c_uint32), prompt.size, max_new,
                                _p(out, C.c_uint32), _p(margins, C.c_float))
        return out, margins

    def close(self) -> None:
        if self._h:
            lib().po_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def encode_channel(channel, codebook):
    channel = np.ascontiguousarray(channel, np.float32)
    codebook = np.ascontiguousarray(codebook, np.float32)
    packed = np.empty((channel.size + 1) // 2, np.uint8)
    mse = lib().po_encode_channel(_p(channel, C.c_float), channel.size, _p(codebook, C.c_float),
                                  codebook.size, _p(packed, C.c_uint8))
    return packed, float(mse)


def fit_palette(channel, k: int, max_iter: int) -> np.ndarray:
    channel = np.ascontiguousarray(channel, np.float32)
    out = np.zeros(max(k, 1), np.float32)
    n = lib().po_fit_palette(_p(channel, C.c_float), channel.size, k, max_iter, _p(out, C.c_float))
    return out[:n]


def palettize_to_payload(weights, dm: int, dn: int, k: int = 16, max_iter: int = 50) -> np.ndarray:
    weights = np.ascontiguousarray(weights, np.float32)
    payload = np.zeros(dm * 32 + dm * (dn // 2), np.uint8)
    lib().po_palettize_to_payload(_p(weights, C.c_float), dm, dn, k, max_iter, _p(payload, C.c_uint8))
    return payload


def max_threads() -> int:
    return int(lib().po_max_threads())

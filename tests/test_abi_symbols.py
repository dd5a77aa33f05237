"""The C-ABI library loads and exports every symbol the headers under include/ declare (CPU: no compute calls)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for h in sorted(os.listdir(inc)):
        if not h.endswith(".h"):
            continue
        src = open(os.path.join(inc, h)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names |= set(re.findall(r"\b(prism_cuda_[a-z0-9_]+)\s*\(", src))
    return sorted(names)


@pytest.fixture(scope="module")
def built():
    from prism_engine_b200 import build

    return build.build()


def test_header_symbols_exported(built):
    lib = ctypes.CDLL(built)
    names = _declared()
    assert len(names) >= 45
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_header(built):
    from prism_engine_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared()
    _lib.load()


def test_static_library_built(built):
    assert os.path.exists(os.path.join(os.path.dirname(built), "libprism_cuda.a"))


def test_no_cpu_fallback_without_gpu(built):
    """Without a CUDA device the backend refuses to construct instead of computing on the CPU."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import prism_engine_b200 as p

    with pytest.raises(p.PrismCudaError) as ei:
        p.CudaBackend()
    assert "No CUDA device" in str(ei.value)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "prism_engine_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower().replace("test oracle", ""), os.path.join(dirpath, f)

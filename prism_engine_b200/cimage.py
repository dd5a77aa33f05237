"""The reference's ``.cimage`` weight container (src/quantization/cimage.rs).

File = ``b"TRB_CIMG"`` + u64 LE header length + JSON header; the first 128 KB
are reserved for the header (cimage.rs:24-29, 81-95) and every payload starts
on a 16 KB boundary (cimage.rs:211-222).  Header JSON, as serde_json writes it
(cimage.rs:33-60)::

    {"tensors": {name: {"tensor_type": "Palettized4Bit", "offset": .., "size": ..,
                        "dim_m": .., "dim_n": ..}, ...}, "execution_plan": null | "<json>"}

This module writes and reads that format byte for byte so that synthetic
models travel through the same container the reference's compiler emits.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, Optional

import numpy as np

PAGE_SIZE = 16384
HEADER_PAGES = 8
MAGIC = b"TRB_CIMG"


class CImageWriter:
    """``CImageWriter::{new, append_palettized, append_fp16, append_blob, set_execution_plan, finalize}``."""

    def __init__(self, path: str):
        self.f = open(path, "wb")
        self.f.write(bytes(HEADER_PAGES * PAGE_SIZE))
        self.tensors: Dict[str, dict] = {}
        self.plan: Optional[str] = None

    def _align(self) -> int:
        pos = self.f.tell()
        rem = pos % PAGE_SIZE
        if rem:
            self.f.write(bytes(PAGE_SIZE - rem))
        return self.f.tell()

    def _append(self, name: str, payload, ttype: str, dim_m: int, dim_n: int) -> None:
        data = np.ascontiguousarray(payload, dtype=np.uint8).tobytes()
        off = self._align()
        self.f.write(data)
        self.tensors[name] = {"tensor_type": ttype, "offset": off, "size": len(data), "dim_m": dim_m, "dim_n": dim_n}

    def append_palettized(self, name: str, payload, dim_m: int, dim_n: int) -> None:
        self._append(name, payload, "Palettized4Bit", dim_m, dim_n)

    def append_fp16(self, name: str, payload, dim_m: int, dim_n: int) -> None:
        self._append(name, payload, "StandardFP16", dim_m, dim_n)

    def append_blob(self, name: str, payload) -> None:
        self._append(name, payload, "Blob", 0, 0)

    def set_execution_plan(self, plan_json: str) -> None:
        self.plan = plan_json

    def finalize(self) -> None:
        hdr = json.dumps({"tensors": self.tensors, "execution_plan": self.plan}, separators=(",", ":")).encode()
        if 16 + len(hdr) > HEADER_PAGES * PAGE_SIZE:
            raise ValueError(f"Header ({16 + len(hdr)} B) exceeds reserved {HEADER_PAGES * PAGE_SIZE} B")
        self.f.seek(0)
        self.f.write(MAGIC + struct.pack("<Q", len(hdr)) + hdr)
        self.f.close()


class CImageReader:
    """``CImageReader::{open, tensor, read_blob}`` (cimage.rs:242-303)."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            magic = f.read(8)
            if magic != MAGIC:
                raise ValueError(f"Invalid magic: expected TRB_CIMG, got {magic!r}")
            (n,) = struct.unpack("<Q", f.read(8))
            self.header = json.loads(f.read(n))
        self.tensors = self.header.get("tensors", {})
        self.execution_plan = self.header.get("execution_plan")

    def tensor(self, name: str) -> Optional[dict]:
        return self.tensors.get(name)

    def read_payload(self, name: str) -> np.ndarray:
        rec = self.tensors[name]
        with open(self.path, "rb") as f:
            f.seek(rec["offset"])
            return np.frombuffer(f.read(rec["size"]), np.uint8)

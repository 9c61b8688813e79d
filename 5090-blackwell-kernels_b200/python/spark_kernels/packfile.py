"""On-disk format for quantized weights: quantize and repack once, load the packed tensors directly.

The reference has no such format: every construction of its model re-quantizes the bf16 checkpoint
(python/spark_kernels/engine.py:328-342) and its design notes list a packed-weight format as missing
(docs/design/w4gemm.md:368). A file holds the tensors of ONE quantized projection exactly as the GEMMs
read them (repacked int4 codes, blocked fp4 scales, ...), so loading is a copy to the device.

Layout (little endian):
    bytes 0-7    magic  b"SPKW0001"
    bytes 8-15   u64    length of the JSON header
    then         the header: {"kind": ..., "meta": {...}, "tensors": {name: {"dtype", "shape", "offset", "nbytes", "crc32"}}}
    then         the tensors' raw bytes, each starting on a 256-byte boundary (offsets from the start of the file)
Every tensor carries a CRC-32 that `load_tensors` verifies. `kind` names the Linear class; `meta` its
constructor state that is not a tensor (format name, per-token flag, columns).
"""

from __future__ import annotations

import json
import struct
import zlib

import torch

MAGIC = b"SPKW0001"
ALIGN = 256
_DTYPES = {"int32": torch.int32, "uint8": torch.uint8, "bfloat16": torch.bfloat16, "float32": torch.float32,
           "float8_e4m3fn": torch.float8_e4m3fn}


def _raw(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous().reshape(-1)
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def save_tensors(path: str, kind: str, tensors: dict, meta: dict | None = None) -> None:
    """Write the named tensors (None entries are skipped) of one quantized projection."""
    entries, blobs = {}, []
    for name, t in tensors.items():
        if t is None:
            continue
        dt = str(t.dtype).replace("torch.", "")
        if dt not in _DTYPES:
            raise ValueError(f"packfile: dtype {t.dtype} of {name!r} is not storable")
        raw = _raw(t)
        entries[name] = {"dtype": dt, "shape": list(t.shape), "nbytes": len(raw), "crc32": zlib.crc32(raw)}
        blobs.append((name, raw))
    # offsets depend on the header's own length: lay out with a fixed-size placeholder, then fill in
    for e in entries.values():
        e["offset"] = 0
    header = {"kind": kind, "meta": meta or {}, "tensors": entries}
    size = len(json.dumps(header).encode()) + 32 * len(entries)  # room for the real offsets
    start = -(-(16 + size) // ALIGN) * ALIGN
    off = start
    for name, raw in blobs:
        entries[name]["offset"] = off
        off = -(-(off + len(raw)) // ALIGN) * ALIGN
    hj = json.dumps(header).encode()
    assert 16 + len(hj) <= start
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<Q", len(hj)) + hj)
        for name, raw in blobs:
            f.seek(entries[name]["offset"])
            f.write(raw)
        f.truncate(max(off, f.tell()))


def load_tensors(path: str, device="cpu"):
    """-> (kind, meta, {name: tensor on `device`}); raises ValueError on a bad magic, a truncated file or a
    checksum mismatch."""
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < 16 or data[:8] != MAGIC:
        raise ValueError(f"{path}: not a packed-weight file (bad magic)")
    (hlen,) = struct.unpack("<Q", data[8:16])
    if 16 + hlen > len(data):
        raise ValueError(f"{path}: truncated header")
    header = json.loads(data[16:16 + hlen].decode())
    out = {}
    for name, e in header["tensors"].items():
        raw = data[e["offset"]:e["offset"] + e["nbytes"]]
        if len(raw) != e["nbytes"]:
            raise ValueError(f"{path}: tensor {name!r} is truncated")
        if zlib.crc32(raw) != e["crc32"]:
            raise ValueError(f"{path}: checksum mismatch in tensor {name!r}")
        t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(_DTYPES[e["dtype"]]).reshape(e["shape"]) if e["nbytes"] else \
            torch.empty(e["shape"], dtype=_DTYPES[e["dtype"]])
        out[name] = t.to(device)
    return header["kind"], header["meta"], out


# ---- the Linear classes ---------------------------------------------------------------------------

def save_linear(path: str, lin) -> None:
    """Store an Int4Linear / FP8Linear / MXFP8Linear / FP4Linear (or a W4GateUpWeight) as it is used by its GEMM."""
    from . import ops, quant

    if isinstance(lin, ops.W4GateUpWeight):
        save_tensors(path, "W4GateUpWeight", {"packed": lin.packed, "scales": lin.scales, "zeros": lin.zeros})
    elif isinstance(lin, quant.Int4Linear):
        save_tensors(path, "Int4Linear", {"packed": lin.w4.packed, "scales": lin.w4.scales, "zeros": lin.w4.zeros})
    elif isinstance(lin, quant.FP8Linear):
        save_tensors(path, "FP8Linear", {"wt": lin.wt, "sw": lin.sw}, {"per_token": lin.per_token})
    elif isinstance(lin, quant.MXFP8Linear):
        save_tensors(path, "MXFP8Linear", {"wt": lin.wt, "sfb": lin.sfb})
    elif isinstance(lin, quant.FP4Linear):
        save_tensors(path, "FP4Linear", {"wt": lin.wt, "sfb": lin.sfb, "sw": lin.sw}, {"fmt": lin.fmt, "n": lin.n})
    else:
        raise ValueError(f"packfile: cannot store {type(lin).__name__}")


def load_linear(path: str, device="cuda"):
    """The object `save_linear` stored, ready to call, without re-quantizing anything."""
    from . import ops, quant

    kind, meta, t = load_tensors(path, device)
    if kind == "W4GateUpWeight":
        return ops.W4GateUpWeight(t["packed"], t["scales"], t.get("zeros"))
    if kind == "Int4Linear":
        lin = quant.Int4Linear.__new__(quant.Int4Linear)
        lin.w4, lin.variant = ops.W4Weight(t["packed"], t["scales"], t.get("zeros")), -1
        return lin
    if kind == "FP8Linear":
        lin = quant.FP8Linear.__new__(quant.FP8Linear)
        lin.wt, lin.sw, lin.per_token, lin.variant = t["wt"], t["sw"], bool(meta["per_token"]), -1
        lin.one = torch.ones(1, device=t["wt"].device, dtype=torch.float32)
        return lin
    if kind == "MXFP8Linear":
        lin = quant.MXFP8Linear.__new__(quant.MXFP8Linear)
        lin.wt, lin.sfb, lin.variant = t["wt"], t["sfb"], -1
        return lin
    if kind == "FP4Linear":
        lin = quant.FP4Linear.__new__(quant.FP4Linear)
        lin.wt, lin.sfb, lin.sw, lin.fmt, lin.n = t["wt"], t["sfb"], t.get("sw"), meta["fmt"], meta["n"]
        return lin
    raise ValueError(f"{path}: unknown kind {kind!r}")

"""Mapping between torch / numpy dtypes and the native element-type enum."""
from __future__ import annotations

import struct

import numpy as np
import torch

INT8, UINT8, INT16, UINT16, INT32, UINT32, INT64, UINT64, FLOAT, DOUBLE, BF16, FP16 = range(12)

_TORCH = {
    torch.int8: INT8, torch.uint8: UINT8, torch.int16: INT16, torch.int32: INT32, torch.int64: INT64,
    torch.float32: FLOAT, torch.float64: DOUBLE, torch.bfloat16: BF16, torch.float16: FP16,
}
for _name, _code in (("uint16", UINT16), ("uint32", UINT32), ("uint64", UINT64)):
    if hasattr(torch, _name):
        _TORCH[getattr(torch, _name)] = _code

_SIZES = {INT8: 1, UINT8: 1, INT16: 2, UINT16: 2, INT32: 4, UINT32: 4, INT64: 8, UINT64: 8, FLOAT: 4, DOUBLE: 8,
          BF16: 2, FP16: 2}
_PACK = {INT8: "b", UINT8: "B", INT16: "h", UINT16: "H", INT32: "i", UINT32: "I", INT64: "q", UINT64: "Q",
         FLOAT: "f", DOUBLE: "d"}

# typestr for __cuda_array_interface__ (bf16 has no numpy code: exported as u2 and re-viewed)
TYPESTR = {INT8: "|i1", UINT8: "|u1", INT16: "<i2", UINT16: "<u2", INT32: "<i4", UINT32: "<u4", INT64: "<i8",
           UINT64: "<u8", FLOAT: "<f4", DOUBLE: "<f8", BF16: "<u2", FP16: "<f2"}

SUM, MIN, MAX, PROD, AND, OR, XOR = range(7)
OPS = {"sum": SUM, "min": MIN, "max": MAX, "prod": PROD, "and": AND, "or": OR, "xor": XOR}

CMP_EQ, CMP_NE, CMP_GT, CMP_GE, CMP_LT, CMP_LE = range(6)
CMPS = {"eq": CMP_EQ, "ne": CMP_NE, "gt": CMP_GT, "ge": CMP_GE, "lt": CMP_LT, "le": CMP_LE,
        "==": CMP_EQ, "!=": CMP_NE, ">": CMP_GT, ">=": CMP_GE, "<": CMP_LT, "<=": CMP_LE}

SIGNAL_SET, SIGNAL_ADD = 0, 1

(AMO_FETCH_ADD, AMO_FETCH_INC, AMO_FETCH, AMO_FETCH_CSWAP, AMO_ADD, AMO_INC, AMO_CSWAP, AMO_SET, AMO_SWAP,
 AMO_FETCH_AND, AMO_FETCH_OR, AMO_FETCH_XOR, AMO_AND, AMO_OR, AMO_XOR) = range(15)


def code_of(dtype) -> int:
    if isinstance(dtype, int):
        return dtype
    if isinstance(dtype, torch.dtype):
        return _TORCH[dtype]
    return _TORCH[getattr(torch, np.dtype(dtype).name)]


def size_of(code: int) -> int:
    return _SIZES[code]


def to_bits(code: int, value) -> int:
    """Bit pattern of `value` as element type `code`, zero-extended to 64 bits."""
    if code == BF16:
        return int(torch.tensor(float(value), dtype=torch.bfloat16).view(torch.int16).item()) & 0xFFFF
    if code == FP16:
        return int(torch.tensor(float(value), dtype=torch.float16).view(torch.int16).item()) & 0xFFFF
    fmt = _PACK[code]
    if fmt in "fd":
        raw = struct.pack("<" + fmt, float(value))
    else:
        v = int(value)
        bits = 8 * _SIZES[code]
        raw = (v & ((1 << bits) - 1)).to_bytes(_SIZES[code], "little")
    return int.from_bytes(raw, "little")


def from_bits(code: int, bits: int):
    n = _SIZES[code]
    raw = (bits & ((1 << (8 * n)) - 1)).to_bytes(n, "little")
    if code == BF16:
        return float(torch.tensor(int.from_bytes(raw, "little", signed=False), dtype=torch.int32).to(torch.int16)
                     .view(torch.bfloat16).item())
    if code == FP16:
        return float(np.frombuffer(raw, dtype=np.float16)[0])
    return struct.unpack("<" + _PACK[code], raw)[0]

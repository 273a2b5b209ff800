"""Data-type codes shared with include/rmlk_b200.h (rmlk_dtype), numpy and torch."""
from __future__ import annotations

import numpy as np

F16, F32, F64, I32, I64, UNDEFINED, U8, I8, U16, I16, U32, U64, STRING, BOOL = range(14)

NAMES = {F16: "f16", F32: "f32", F64: "f64", I32: "i32", I64: "i64", U8: "u8", I8: "i8", U16: "u16", I16: "i16",
         U32: "u32", U64: "u64", BOOL: "bool"}

_NP = {F16: np.float16, F32: np.float32, F64: np.float64, I32: np.int32, I64: np.int64, U8: np.uint8, I8: np.int8,
       U16: np.uint16, I16: np.int16, U32: np.uint32, U64: np.uint64, BOOL: np.bool_}
_FROM_NP = {np.dtype(v): k for k, v in _NP.items()}

# ONNX TensorProto.DataType codes, used by the Cast op's `to` attribute
# (reference runtime/src/attributes/cast.rs:6-26 converts the int with DataType::try_from).
ONNX = {1: F32, 2: U8, 3: I8, 4: U16, 5: I16, 6: I32, 7: I64, 9: BOOL, 10: F16, 11: F64, 12: U32, 13: U64}
TO_ONNX = {v: k for k, v in ONNX.items()}


def to_numpy(code: int):
    return np.dtype(_NP[code])


def from_numpy(dt) -> int:
    return _FROM_NP[np.dtype(dt)]


def size(code: int) -> int:
    return to_numpy(code).itemsize


def from_torch(dt) -> int:
    import torch
    return {torch.float16: F16, torch.float32: F32, torch.float64: F64, torch.int32: I32, torch.int64: I64,
            torch.uint8: U8, torch.int8: I8, torch.int16: I16, torch.bool: BOOL, torch.uint16: U16, torch.uint32: U32,
            torch.uint64: U64}[dt]


def to_torch(code: int):
    import torch
    return {F16: torch.float16, F32: torch.float32, F64: torch.float64, I32: torch.int32, I64: torch.int64,
            U8: torch.uint8, I8: torch.int8, I16: torch.int16, BOOL: torch.bool, U16: torch.uint16, U32: torch.uint32,
            U64: torch.uint64}[code]

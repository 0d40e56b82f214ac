"""Enumerations of the public C ABI and the torch / numpy dtype mapping."""
from __future__ import annotations

import enum


class DataType(enum.IntEnum):
    INT8 = 0
    INT16 = 1
    INT32 = 2
    FP16 = 3
    FP32 = 4
    INT64 = 5
    UINT64 = 6
    UINT8 = 7
    UINT16 = 8
    UINT32 = 9
    FP64 = 10
    BFP16 = 11
    INT128 = 12
    HIF8 = 14
    FP8E4M3 = 15
    FP8E5M2 = 16
    FP8E8M0 = 17


class ReduceOp(enum.IntEnum):
    SUM = 0
    PROD = 1
    MAX = 2
    MIN = 3


class Engine(enum.IntEnum):
    DEFAULT = 0
    HOST = 1
    COPY_ENGINE = 2
    SM = 3
    NVLS = 4


class Result(enum.IntEnum):
    SUCCESS = 0
    E_PARA = 1
    E_PTR = 2
    E_MEMORY = 3
    E_INTERNAL = 4
    E_NOT_SUPPORT = 5
    E_NOT_FOUND = 6
    E_UNAVAIL = 7
    E_SYSCALL = 8
    E_TIMEOUT = 9
    E_OPEN_FILE_FAILURE = 10
    E_TCP_TRANSFER = 13
    E_RUNTIME = 15
    E_DRV = 16
    E_REMOTE = 21
    E_SUSPENDING = 22
    E_OPRETRY_FAIL = 23
    E_OOM = 24


_NP = {"int8": DataType.INT8, "int16": DataType.INT16, "int32": DataType.INT32, "float16": DataType.FP16,
       "float32": DataType.FP32, "int64": DataType.INT64, "uint64": DataType.UINT64, "uint8": DataType.UINT8,
       "uint16": DataType.UINT16, "uint32": DataType.UINT32, "float64": DataType.FP64, "bool": DataType.UINT8}


def from_numpy(dt) -> DataType:
    return _NP[str(dt)]


_TORCH = None


def from_torch(dt) -> DataType:
    global _TORCH
    if _TORCH is None:
        _TORCH = _torch_table()
    return _TORCH[dt]


def _torch_table():
    import torch

    table = {torch.int8: DataType.INT8, torch.int16: DataType.INT16, torch.int32: DataType.INT32,
             torch.float16: DataType.FP16, torch.float32: DataType.FP32, torch.int64: DataType.INT64,
             torch.uint8: DataType.UINT8, torch.float64: DataType.FP64, torch.bfloat16: DataType.BFP16,
             torch.bool: DataType.UINT8}
    for name, v in (("uint16", DataType.UINT16), ("uint32", DataType.UINT32), ("uint64", DataType.UINT64),
                    ("float8_e4m3fn", DataType.FP8E4M3), ("float8_e5m2", DataType.FP8E5M2),
                    ("float8_e8m0fnu", DataType.FP8E8M0)):
        if hasattr(torch, name):
            table[getattr(torch, name)] = v
    return {k: int(v) for k, v in table.items()}


def reduce_op_from_torch(op) -> ReduceOp:
    import torch.distributed as dist

    table = {dist.ReduceOp.SUM: ReduceOp.SUM, dist.ReduceOp.PRODUCT: ReduceOp.PROD, dist.ReduceOp.MAX: ReduceOp.MAX,
             dist.ReduceOp.MIN: ReduceOp.MIN}
    return table[op]

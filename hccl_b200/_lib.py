"""ctypes loader for the in-tree native library `hccl_b200/lib/libhccl_b200.so`.

The library is built by `hccl_b200.utils.build.build_native()` (or `__graft_entry__.build()`); it is never installed
into site-packages. Loading fails loudly when the file is missing rather than falling back to anything else.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB = None
# HCCL_B200_LIB selects another build flavor of the same library (e.g. lib/libhccl_b200_debug.so with bounds checks)
LIB_PATH = Path(os.environ.get("HCCL_B200_LIB") or Path(__file__).resolve().parent / "lib" / "libhccl_b200.so")

HCCL_ROOT_INFO_BYTES = 4108


class HcclRootInfo(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * HCCL_ROOT_INFO_BYTES)]


class HcclCommConfig(ctypes.Structure):
    _fields_ = [
        ("size", ctypes.c_uint32), ("magic", ctypes.c_uint32), ("version", ctypes.c_uint32),
        ("hcclBufferSize", ctypes.c_uint32), ("hcclDeterministic", ctypes.c_uint32),
        ("hcclCommName", ctypes.c_char * 128), ("hcclUdi", ctypes.c_char * 128),
        ("hcclOpExpansionMode", ctypes.c_uint32), ("hcclRdmaTrafficClass", ctypes.c_uint32),
        ("hcclRdmaServiceLevel", ctypes.c_uint32), ("hcclWorldRankID", ctypes.c_uint32),
        ("hcclJobID", ctypes.c_uint64), ("hcclExecTimeoutSec", ctypes.c_uint32), ("hcclBackend", ctypes.c_uint32),
        ("reserved", ctypes.c_uint32 * 16),
    ]


class HcclSendRecvItem(ctypes.Structure):
    _fields_ = [("sendRecvType", ctypes.c_int), ("buf", ctypes.c_void_p), ("count", ctypes.c_uint64),
                ("dataType", ctypes.c_int), ("remoteRank", ctypes.c_uint32)]


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m hccl_b200.utils.build` (needs nvcc)")
        _LIB = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        _declare(_LIB)
    return _LIB


def _declare(l: ctypes.CDLL) -> None:
    vp, u32, u64, i32 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int
    P = ctypes.POINTER
    sigs = {
        "HcclGetRootInfo": [P(HcclRootInfo)],
        "HcclCommInitRootInfo": [u32, P(HcclRootInfo), u32, P(vp)],
        "HcclCommInitRootInfoConfig": [u32, P(HcclRootInfo), u32, P(HcclCommConfig), P(vp)],
        "HcclCommInitClusterInfo": [ctypes.c_char_p, u32, P(vp)],
        "HcclCommInitAll": [u32, P(ctypes.c_int32), P(vp)],
        "HcclCreateSubCommConfig": [P(vp), u32, P(u32), u64, u32, P(HcclCommConfig), P(vp)],
        "HcclCommDestroy": [vp],
        "HcclGetRankSize": [vp, P(u32)],
        "HcclGetRankId": [vp, P(u32)],
        "HcclGetCommName": [vp, ctypes.c_char_p],
        "HcclGetHcclBuffer": [vp, P(vp), P(u64)],
        "HcclCommGetStatus": [vp, P(i32)],
        "HcclCommSuspend": [vp], "HcclCommResume": [vp],
        "HcclGetCommAsyncError": [vp, P(i32)],
        "HcclCommSymAlloc": [vp, u64, P(vp)], "HcclCommSymFree": [vp, vp],
        "HcclSymWinGetPeerPointer": [vp, vp, u32, P(vp)],
        "HcclSymGetMulticastPointer": [vp, vp, P(vp)],
        "HcclSimStreamSynchronize": [vp],
        "HcclAllReduce": [vp, vp, u64, i32, i32, vp, vp],
        "HcclBroadcast": [vp, u64, i32, u32, vp, vp],
        "HcclReduceScatter": [vp, vp, u64, i32, i32, vp, vp],
        "HcclReduceScatterV": [vp, vp, vp, vp, u64, i32, i32, vp, vp],
        "HcclScatter": [vp, vp, u64, i32, u32, vp, vp],
        "HcclAllGather": [vp, vp, u64, i32, vp, vp],
        "HcclAllGatherV": [vp, u64, vp, vp, vp, i32, vp, vp],
        "HcclSend": [vp, u64, i32, u32, vp, vp],
        "HcclRecv": [vp, u64, i32, u32, vp, vp],
        "HcclAlltoAllVC": [vp, vp, i32, vp, i32, vp, vp],
        "HcclAlltoAllV": [vp, vp, vp, i32, vp, vp, vp, i32, vp, vp],
        "HcclAlltoAll": [vp, u64, i32, vp, u64, i32, vp, vp],
        "HcclReduce": [vp, vp, u64, i32, i32, u32, vp, vp],
        "HcclBatchSendRecv": [P(HcclSendRecvItem), u32, vp, vp],
        "HcclBarrier": [vp, vp],
    }
    for name, args in sigs.items():
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    l.HcclCommConfigInit.argtypes = [P(HcclCommConfig)]
    l.HcclCommConfigInit.restype = None
    l.HcclGetErrorString.argtypes = [ctypes.c_int]
    l.HcclGetErrorString.restype = ctypes.c_char_p


class HcclError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(f"{what} failed: HcclResult {code} ({lib().HcclGetErrorString(code).decode()})")


def check(code: int, what: str) -> None:
    if code != 0:
        raise HcclError(code, what)

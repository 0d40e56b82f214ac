"""The allocation-free all-reduce entry point, called through its exported C symbol, against the allocating single-GPU
harness that runs the same kernel. Collected last on purpose (file name), and written to pass both alone in a fresh process
and after every other test."""
import ctypes

import pytest
import torch

from hccl_b200.types import ReduceOp, from_torch

pytestmark = pytest.mark.gpu


def _call(lib, sends, recvs, dtype, op=ReduceOp.SUM):
    n = len(sends)
    s = (ctypes.c_void_p * n)(*[t.data_ptr() for t in sends])
    r = (ctypes.c_void_p * n)(*[t.data_ptr() for t in recvs])
    fn = lib.HcclLocalAllReduceNoAlloc
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn(s, r, n, sends[0].numel(), int(from_torch(dtype)), int(op), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_allreduce_matches_allocating_entry_twice():
    from hccl_b200._lib import lib
    from hccl_b200.utils import emu
    l = lib()
    torch.cuda.set_device(0)
    # two calls in a row, with different data, sizes, dtypes and buffer counts: the shared scratch must not leak state
    for call, (n, count, dtype) in enumerate([(4, 30_001, torch.float32), (2, 131_072, torch.bfloat16)]):
        g = torch.Generator(device="cuda").manual_seed(500 + call)
        xs = [(torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype) for _ in range(n)]
        outs = [torch.zeros_like(x) for x in xs]
        assert _call(l, xs, outs, dtype) == 0
        # the status records of that call, copied into host memory this test owns: no wait ran out
        records = (ctypes.c_uint32 * (8 * n))(*([7] * (8 * n)))
        l.HcclLocalAllReduceNoAllocStatus.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p]
        assert l.HcclLocalAllReduceNoAllocStatus(records, n, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
        torch.cuda.synchronize()
        assert all(records[8 * i] == 0 for i in range(n))
        with emu.EmuWorld(n, 512 << 10) as w:
            ref = [torch.zeros_like(x) for x in xs]
            assert w.run(2, "SmAllReduceMesh1DTwoShot", xs, ref, count, dtype, ReduceOp.SUM) == 0
        exact = torch.stack([x.double() for x in xs]).sum(0)
        tol = 1e-5 * n if dtype == torch.float32 else 3e-2 * n
        for o, rf in zip(outs, ref):
            assert torch.equal(o, rf)                     # same kernel, same order: identical bits
            assert torch.allclose(o.double(), exact, atol=tol, rtol=tol)


def test_no_alloc_rejects_what_does_not_fit():
    from hccl_b200._lib import lib
    l = lib()
    torch.cuda.set_device(0)
    big = [torch.zeros((256 << 10) // 4 + 1, device="cuda") for _ in range(2)]
    assert _call(l, big, big, torch.float32) == 1          # HCCL_E_PARA: beyond the fixed scratch
    five = [torch.zeros(16, device="cuda") for _ in range(5)]
    assert _call(l, five, five, torch.float32) == 1

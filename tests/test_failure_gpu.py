"""A device-side wait that runs out reports through the status word and leaves the context usable.

The wait is made to run out by a flag that nothing sets (one GPU, one process, no peer): the kernel gives up after its
cycle limit (about a second), records {code, site, block, last value} and returns."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_runs_out_and_reports():
    from ds41rt_b200.ops import gemm as G, lib
    dev = torch.device("cuda")
    flags = torch.zeros(2, dtype=torch.int32, device=dev)                 # never raised
    flag_ptrs = torch.tensor([flags.data_ptr(), flags.data_ptr() + 4], dtype=torch.int64, device=dev)
    epoch = torch.ones(1, dtype=torch.int32, device=dev)                  # waiters expect >= 1
    slots = torch.zeros(2, 1024, dtype=torch.float32, device=dev)
    out = torch.zeros(1024, dtype=torch.float32, device=dev)
    status = lib.new_status(dev)
    lib.check(lib.kernels().ds41_rs_reduce(lib.ptr(slots), 2, C.c_longlong(1024), lib.ptr(out), 0, C.c_longlong(1024),
                                           lib.ptr(flag_ptrs), lib.ptr(epoch), lib.ptr(status), lib.stream()), "rs_reduce")
    torch.cuda.synchronize()
    code, where, block, detail = lib.read_status(status)
    assert code == 2 and where in (600, 601) and detail == 0              # flag wait timed out, flag still 0
    with pytest.raises(lib.KernelError):
        lib.raise_on_status(status, "reduce")
    # the context is intact: a tensor-core GEMM right after gives the right answer
    x = torch.randn(64, 256, device=dev).bfloat16()
    w = torch.randn(128, 256, device=dev).bfloat16()
    st2 = lib.new_status(dev)
    y = G.matmul_nt(x, w, status=st2)
    torch.cuda.synchronize()
    lib.raise_on_status(st2, "gemm after timeout")
    ref = x.float() @ w.float().t()
    assert float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2

"""Allocation-free entry point: same results as the regular fused hyper-connection step.

Collected last on purpose (file name), so a run that stops at the first failure has already run everything else.
The entry point is for callers that must not allocate device memory when they call the library (a plug-in inside
another runtime's pool, a latency-critical section, a frozen allocator); it keeps its scratch in a fixed array
inside the library.  It is reached here through its exported C symbol, twice in a row, because the array keeps
the previous call's contents and the second call must still be right.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(lib, t, scratch):
    a = lib.HcStepArgs()
    a.streams_in = a.streams_out = lib.ptr(t["streams"])
    a.part_bases = C.cast(t["bases"], C.c_void_p)
    a.post, a.comb, a.pre_in = lib.ptr(t["post"]), lib.ptr(t["comb"]), lib.ptr(t["pre_in"])
    a.fn, a.scale, a.base, a.norm_w = lib.ptr(t["fn"]), lib.ptr(t["scale"]), lib.ptr(t["base"]), lib.ptr(t["norm_w"])
    a.next_pre, a.post_out, a.comb_out, a.xn = (lib.ptr(t["next_pre"]), lib.ptr(t["post_out"]), lib.ptr(t["comb_out"]),
                                                 lib.ptr(t["xn"]))
    a.status = lib.ptr(t["status"])
    if "xq" in t:
        a.xq, a.xq_sf = lib.ptr(t["xq"]), lib.ptr(t["xq_sf"])
    if scratch:
        a.partial, a.xc, a.tickets = lib.ptr(t["partial"]), lib.ptr(t["xc"]), lib.ptr(t["tickets"])
    a.split_stride, a.n_ranks, a.n_splits = t["rows"] * t["H"], 1, 2
    a.rows, a.H, a.iters, a.hc_eps, a.norm_eps = t["rows"], t["H"], 20, 1e-6, 1e-20
    return a


def _tensors(rows, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    sub = r(2, rows, H)
    t = {"rows": rows, "H": H, "sub": sub, "bases": (C.c_void_p * 1)(sub.data_ptr()),
         "streams0": r(rows, 4, H).bfloat16(), "post": r(rows, 4).abs(), "comb": r(rows, 16).abs(),
         "pre_in": r(rows, 4).abs(), "fn": r(24, 4 * H) * 0.02, "scale": torch.tensor([1.0, 0.7, 1.3], device="cuda"),
         "base": r(24) * 0.5, "norm_w": r(H).abs() + 0.5}
    return t


def _outputs(t, quant=False):
    z = lambda *s, dt=torch.float32: torch.zeros(*s, device="cuda", dtype=dt)
    if quant:          # E4M3 rows and their packed scale atoms are written beside the bf16 rows
        t.update(xq=z(t["rows"], t["H"], dt=torch.uint8), xq_sf=z(1, t["H"] // 128, 512, dt=torch.uint8))
    t.update(streams=t["streams0"].clone(), next_pre=z(t["rows"], 4), post_out=z(t["rows"], 4),
             comb_out=z(t["rows"], 16), xn=z(t["rows"], t["H"], dt=torch.bfloat16),
             status=torch.zeros(4, dtype=torch.int32, device="cuda"),
             partial=z(t["H"] // 128, t["rows"], 26), xc=z(t["rows"], t["H"]),
             tickets=torch.zeros(t["rows"], dtype=torch.int32, device="cuda"))
    return t


def test_static_scratch_entry_matches_regular_entry_twice():
    from ds41rt_b200.ops import lib
    k = lib.kernels()
    fn = k.ds41_hc_step_static                     # the exported C symbol
    fn.restype = C.c_int
    # the last two cases sit on the entry point's limits (16 rows, H = 8192); two of them also ask for the quantised row
    for call, (rows, H, seed, quant) in enumerate([(5, 1024, 1, False), (3, 2048, 2, True), (16, 8192, 4, False),
                                                   (16, 8192, 5, True)]):
        t = _outputs(_tensors(rows, H, seed), quant)
        lib.check(k.ds41_hc_step(C.byref(_args(lib, t, True)), lib.stream()), "regular")
        torch.cuda.synchronize()
        names = ("streams", "next_pre", "post_out", "comb_out", "xn") + (("xq", "xq_sf") if quant else ())
        want = {n: t[n].clone() for n in names}
        t = _outputs(t, quant)
        lib.check(fn(C.byref(_args(lib, t, False)), lib.stream()), "static")
        torch.cuda.synchronize()
        assert t["status"].tolist()[0] == 0
        for n in names:                       # the same kernel ran on the same inputs: every output is bit-identical
            assert torch.equal(t[n], want[n]), (call, n)


def test_static_scratch_entry_rejects_sizes_beyond_its_limits():
    from ds41rt_b200.ops import lib
    k = lib.kernels()
    fn = k.ds41_hc_step_static
    fn.restype = C.c_int
    t = _outputs(_tensors(2, 1024, 3))
    a = _args(lib, t, False)
    a.rows = 17
    assert fn(C.byref(a), lib.stream()) == 1        # cudaErrorInvalidValue, nothing launched
    a.rows, a.H = 2, 16384
    assert fn(C.byref(a), lib.stream()) == 1

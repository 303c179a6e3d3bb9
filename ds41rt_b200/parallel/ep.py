"""Expert-parallel routed experts: dispatch -> grouped GEMMs -> combine as peer-memory kernels.

Rank r owns experts [r*E/W, (r+1)*E/W) and holds `tokens` rows of the sequence (sequence-parallel prefill).  One call
of `ExpertParallelMoE.forward` launches, on the current stream and without host synchronisation:

  ep_count -> ep_plan -> ep_dispatch        tokens go straight into the owner's receive buffer (P2P stores), sorted by
                                            expert, every expert group starting on a 128-row boundary
  grouped FC1 (tcgen05, gate+up dual tiles, clamp-SwiGLU x route weight in the epilogue; waits for the peers' dispatch
               flags inside the kernel)
  grouped FC2 (tcgen05; the epilogue stores each result row into the combine buffer of the rank the token came from)
  ep_mark -> ep_combine                     fixed-order sum of the topk returned rows (+ the local shared expert)

The grouped GEMMs read a device-side tile table written by ep_plan, so group sizes never reach the host.
`baseline()` is the same layer with NCCL all_to_all_single and library matmuls, for comparison.
Kernels: csrc/kernels/ep.cu, csrc/kernels/gemm_tc.cu (tile-table mode, out_mode 7).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..ops import gemm as G
from ..ops import lib
from .fabric import Fabric


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class ExpertParallelMoE:
    def __init__(self, fabric: Fabric, w13: torch.Tensor, w2: torch.Tensor, *, topk: int, max_tokens: int,
                 act_limit: float = 10.0, capacity: Optional[int] = None, w13_sf: Optional[torch.Tensor] = None,
                 w2_sf: Optional[torch.Tensor] = None, fp4: bool = False, nvfp4=None,
                 w13_gs: Optional[torch.Tensor] = None, w2_gs: Optional[torch.Tensor] = None,
                 wire: str = "auto", tile_tokens: Optional[int] = None):
        """w13: [E_local, 2*I, H] (gate rows then up rows), w2: [E_local, H, I]; bf16, or e4m3 with UE8M0 scale atoms,
        or (fp4) E2M1 codes two per byte ([.., H/2] / [.., I/2] uint8) with UE8M0 scale atoms, or (nvfp4 = the two
        activation scales) E2M1 codes with E4M3 scale atoms per 16 and one global scale per expert (w13_gs / w2_gs):
        then the received rows and the FC1 output are quantised to NVFP4 too (W4A4).
        wire: what a token row looks like on NVLink.  "fp8" (the default for block-scaled FP8 / FP4 experts): the
        sender quantises the row inside the dispatch kernel (E4M3 + one UE8M0 scale per 128 values, 5280 bytes for 5120
        values - the reference's wire format, docs/dspark-bandwidth-policy.md:19-20) and stores it straight into the
        owner's FC1 operand buffers, so no receive-side wait or quantisation kernel runs; "bf16": rows travel as bf16
        and the owner quantises what it received."""
        self.f = fabric
        self.w13, self.w2, self.w13_sf, self.w2_sf = w13, w2, w13_sf, w2_sf
        self.mx = w13_sf is not None and nvfp4 is None
        self.fp4 = fp4 or nvfp4 is not None
        self.nv = nvfp4
        self.w13_gs, self.w2_gs = w13_gs, w2_gs
        self.e_local, two_i, self.H = w13.shape
        if self.fp4:
            self.H *= 2
        self.I = two_i // 2
        self.topk, self.max_tokens, self.act_limit = topk, max_tokens, act_limit
        assert wire in ("auto", "fp8", "bf16")
        self.wire_fp8 = self.mx and wire != "bf16"
        W, dev = fabric.world, fabric.device
        assert self.H % 128 == 0 and self.I % 128 == 0 and W <= 8
        scaled = self.mx or self.nv is not None
        # FC1 tile width in tokens.  Gate and up accumulators share tensor memory with the scale columns: the block-scaled
        # FP8 kind still takes 128 tokens with a single accumulator set (half the weight bytes per token from L2, which
        # is what bounds it); NVFP4 carries four times the scale columns and stays at 64
        self.bn = 128 if (not scaled or self.mx) else 64
        self.bn2 = 128 if scaled else 256          # FC2
        # `tile_tokens` overrides both for the block-scaled FP8 kind (128 or 192).  With hundreds of experts a pass gives
        # each about 128 rows: 128-token tiles then leave every second expert with a nearly empty second tile that still
        # streams the expert's weights, while a 192-token tile holds the whole expert and multiplies only the columns
        # it has
        if tile_tokens is not None and self.mx and not self.fp4:
            assert tile_tokens in (128, 192)
            self.bn = self.bn2 = tile_tokens
        worst = W * max_tokens * topk
        self.cap = _round_up(min(worst, capacity) if capacity else worst, 128) + 128 * self.e_local
        self.max_tiles = self.cap // self.bn + self.e_local
        H, cap = self.H, self.cap
        # symmetric memory: [counts | send_base | flags | recv_meta | recv_w | recv_x | comb]
        off, lay = 0, {}
        for name, nbytes in (("counts", 4 * W * self.e_local), ("send_base", 4 * W * self.e_local), ("flags", 64),
                             ("recv_meta", 8 * cap), ("recv_w", 4 * cap),
                             ("recv_x", 0 if self.wire_fp8 else 2 * cap * H),
                             ("recv_q", cap * H if self.wire_fp8 else 0),
                             ("recv_sf", cap // 128 * (H // 128) * 512 if self.wire_fp8 else 0),
                             ("comb", 2 * max_tokens * topk * H)):
            lay[name] = off
            off += _round_up(nbytes, 256)
        self.sym = fabric.alloc(off)
        self.lay = lay
        self.recv_x = None if self.wire_fp8 else self.sym.view(torch.bfloat16, (cap, H), lay["recv_x"])
        self.recv_w = self.sym.view(torch.float32, (cap,), lay["recv_w"])
        self.recv_meta = self.sym.view(torch.int32, (cap, 2), lay["recv_meta"])
        self.comb = self.sym.view(torch.bfloat16, (max_tokens * topk, H), lay["comb"])
        self.counts = self.sym.view(torch.int32, (W, self.e_local), lay["counts"])
        self.flag_ptrs = [
            torch.tensor([p + lay["flags"] + 4 * ph for p in self.sym.peer_ptrs], dtype=torch.int64, device=dev)
            for ph in range(4)
        ]
        i32 = dict(dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(1, **i32)
        self.cursor = torch.zeros(W * self.e_local, **i32)
        self.ticket = torch.zeros(1, **i32)
        self.tile_group = torch.zeros(2 * self.max_tiles, **i32)
        self.tile_row0 = torch.zeros(2 * self.max_tiles, **i32)
        self.tile_end = torch.zeros(2 * self.max_tiles, **i32)
        self.n_tiles = torch.zeros(2, **i32)
        self.total_rows = torch.zeros(1, **i32)
        self.status = lib.new_status(dev)
        self.act = torch.zeros(cap, self.I, dtype=torch.bfloat16, device=dev)
        if self.nv is not None:
            u8 = dict(dtype=torch.uint8, device=dev)
            assert H % 256 == 0 and self.I % 256 == 0
            self.xq = torch.zeros(cap, H // 2, **u8)
            self.xq_sf = torch.zeros(cap // 128 * (H // 64) * 512, **u8)
            self.actq = torch.zeros(cap, self.I // 2, **u8)
            self.actq_sf = torch.zeros(cap // 128 * (self.I // 64) * 512, **u8)
        if self.mx:
            u8 = dict(dtype=torch.uint8, device=dev)
            if self.wire_fp8:           # the FC1 operand buffers are the receive buffers: peers write them directly
                self.xq = self.sym.view(torch.uint8, (cap, H), lay["recv_q"])
                self.xq_sf = self.sym.view(torch.uint8, (cap // 128 * (H // 128) * 512,), lay["recv_sf"])
            else:
                self.xq = torch.zeros(cap, H, **u8)
                self.xq_sf = torch.zeros(cap // 128 * (H // 128) * 512, **u8)
            self.actq = torch.zeros(cap, self.I, **u8)
            self.actq_sf = torch.zeros(cap // 128 * (self.I // 128) * 512, **u8)
        self.dispatch_blocks = 4 * 148
        self.marks = None          # list of (name, event) while phase timing is on

    def set_weights(self, w13, w2, w13_sf=None, w2_sf=None, w13_gs=None, w2_gs=None) -> None:
        """Point the layer at another expert stack of the same shape and kind (one instance serves every MoE layer)."""
        assert w13.shape == self.w13.shape and w2.shape == self.w2.shape
        assert (w13_sf is not None) == (self.mx or self.nv is not None)
        self.w13, self.w2, self.w13_sf, self.w2_sf = w13, w2, w13_sf, w2_sf
        self.w13_gs, self.w2_gs = w13_gs, w2_gs

    # ------------------------------------------------------------------ argument blocks
    def _ep_args(self, x, ids, weights, tokens) -> lib.EpArgs:
        f, a = self.f, lib.EpArgs()
        a.world, a.rank, a.e_local, a.topk, a.tokens = f.world, f.rank, self.e_local, self.topk, tokens
        a.H, a.cap, a.bn, a.bn2, a.max_tiles = self.H, self.cap, self.bn, self.bn2, self.max_tiles
        a.x, a.ids, a.weights = lib.ptr(x), lib.ptr(ids), lib.ptr(weights)
        a.epoch, a.cursor, a.ticket = lib.ptr(self.epoch), lib.ptr(self.cursor), lib.ptr(self.ticket)
        for r, base in enumerate(self.sym.peer_ptrs):
            a.counts[r] = base + self.lay["counts"]
            a.send_base[r] = base + self.lay["send_base"]
            a.recv_x[r] = base + self.lay["recv_x"]
            a.recv_meta[r] = base + self.lay["recv_meta"]
            a.recv_w[r] = base + self.lay["recv_w"]
            a.flags[r] = base + self.lay["flags"]
            if self.wire_fp8:
                a.recv_q[r] = base + self.lay["recv_q"]
                a.recv_sf[r] = base + self.lay["recv_sf"]
        a.wire_fp8 = 1 if self.wire_fp8 else 0
        a.tile_group, a.tile_row0, a.tile_end = lib.ptr(self.tile_group), lib.ptr(self.tile_row0), lib.ptr(self.tile_end)
        a.n_tiles, a.total_rows, a.status = lib.ptr(self.n_tiles), lib.ptr(self.total_rows), lib.ptr(self.status)
        return a

    def _grouped(self, A, B, out, M, K, *, lda, ldo, out_mode, wait_phase=None, table=0, **kw) -> None:
        a = lib.GemmArgs()
        a.A, a.B, a.out, a.status = lib.ptr(A), lib.ptr(B), lib.ptr(out), lib.ptr(self.status)
        a.lda, a.ldb, a.ldo = lda, K, ldo
        a.M, a.N, a.K, a.batch, a.a_batches = M, self.cap, K, self.e_local, self.e_local
        a.a_batch_stride = A.stride(0) * (2 if self.fp4 else 1)      # counted in elements
        a.a_format = 1 if (self.fp4 and self.nv is None) else 0
        a.kind, a.out_mode, a.k_splits, a.b_batch_kind = (3 if self.nv is not None else 2 if self.mx else 0), out_mode, 1, 1
        a.bn = self.bn2 if table else self.bn
        t0 = table * self.max_tiles
        a.tile_group, a.tile_row0 = lib.ptr(self.tile_group[t0:]), lib.ptr(self.tile_row0[t0:])
        a.tile_end, a.n_tiles_dev, a.max_tiles = lib.ptr(self.tile_end[t0:]), lib.ptr(self.n_tiles[table:]), self.max_tiles
        a.row_w, a.act_limit = lib.ptr(self.recv_w), self.act_limit
        if wait_phase is not None and self.f.world > 1:
            a.wait_flags, a.wait_epoch, a.wait_world = lib.ptr(self.flag_ptrs[wait_phase]), lib.ptr(self.epoch), self.f.world
        for key, val in kw.items():
            setattr(a, key, lib.ptr(val) if isinstance(val, torch.Tensor) else val)
        if out_mode == 7:
            a.scatter_meta = lib.ptr(self.recv_meta)
            for r, base in enumerate(self.sym.peer_ptrs):
                a.scatter_out[r] = base + self.lay["comb"]
        lib.check(lib.kernels().ds41_gemm_tc(C.byref(a), lib.stream()), "grouped gemm")

    def _mark(self, name: str) -> None:
        if self.marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def phase_times(self, *args, reps: int = 5):
        """Per-phase device times (ms) of forward(*args), averaged over `reps` calls."""
        acc = {}
        for _ in range(reps):
            self.marks = []
            self._mark("start")
            self.forward(*args)
            torch.cuda.synchronize()
            for (_, e0), (name, e1) in zip(self.marks[:-1], self.marks[1:]):
                acc[name] = acc.get(name, 0.0) + e0.elapsed_time(e1) / reps
        self.marks = None
        return acc

    # ------------------------------------------------------------------ the fused layer
    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, out: torch.Tensor,
                extra: Optional[torch.Tensor] = None) -> None:
        """x [T,H] bf16, ids [T,topk] int32 (global expert ids), weights [T,topk] fp32 -> out [T,H] (bf16 or fp32).

        `extra` ([T,H] fp32, e.g. the shared expert's output) is added before the routed rows, in a fixed order."""
        T = x.shape[0]
        assert T <= self.max_tokens and x.dtype == torch.bfloat16 and x.is_contiguous()
        assert ids.dtype == torch.int32 and weights.dtype == torch.float32
        k, st, H, I = lib.kernels(), lib.stream, self.H, self.I
        a = self._ep_args(x, ids, weights, T)
        lib.check(k.ds41_ep_count(C.byref(a), st()), "ep_count")
        lib.check(k.ds41_ep_plan(C.byref(a), st()), "ep_plan")
        self._mark("count+plan")
        lib.check(k.ds41_ep_dispatch(C.byref(a), self.dispatch_blocks, st()), "ep_dispatch")
        self._mark("dispatch")
        if self.nv is not None:
            lib.check(k.ds41_ep_wait(C.byref(a), 2, st()), "ep_wait")
            cap, zero = self.cap, C.c_longlong(0)
            lib.check(k.ds41_act_quant_nvfp4_rows(lib.ptr(self.recv_x), C.c_longlong(H), lib.ptr(self.xq), C.c_longlong(H),
                                                  lib.ptr(self.xq_sf), cap, H, C.c_float(self.nv[0]),
                                                  lib.ptr(self.total_rows), 1, zero, zero, zero, None, st()), "quant")
            self._grouped(self.w13, self.xq, self.act, I, H, lda=H, ldo=I, out_mode=4, up_row_offset=I,
                          sfa=self.w13_sf, sfa_batch_stride=self.w13_sf[0].numel(), sfb=self.xq_sf, alpha=self.nv[0],
                          alpha_batch=self.w13_gs)
            self._mark("wait+quant+fc1")
            lib.check(k.ds41_act_quant_nvfp4_rows(lib.ptr(self.act), C.c_longlong(I), lib.ptr(self.actq), C.c_longlong(I),
                                                  lib.ptr(self.actq_sf), cap, I, C.c_float(self.nv[1]),
                                                  lib.ptr(self.total_rows), 1, zero, zero, zero, None, st()), "quant")
            self._grouped(self.w2, self.actq, self.comb, H, I, lda=I, ldo=H, out_mode=7, table=1, sfa=self.w2_sf,
                          sfa_batch_stride=self.w2_sf[0].numel(), sfb=self.actq_sf, alpha=self.nv[1],
                          alpha_batch=self.w2_gs)
            self._mark("quant+fc2")
        elif self.mx:
            cap = self.cap
            if self.wire_fp8:
                # the rows arrived quantised, in place: FC1 waits for the peers' dispatch flags inside the kernel
                self._grouped(self.w13, self.xq, self.act, I, H, lda=H, ldo=I, out_mode=4, up_row_offset=I,
                              sfa=self.w13_sf, sfa_batch_stride=self.w13_sf[0].numel(), sfb=self.xq_sf, wait_phase=2)
            else:
                lib.check(k.ds41_ep_wait(C.byref(a), 2, st()), "ep_wait")
                lib.check(k.ds41_act_quant_mx_rows(lib.ptr(self.recv_x), C.c_longlong(H), lib.ptr(self.xq),
                                                   C.c_longlong(H), lib.ptr(self.xq_sf), cap, H,
                                                   lib.ptr(self.total_rows), st()), "act_quant")
                self._grouped(self.w13, self.xq, self.act, I, H, lda=H, ldo=I, out_mode=4, up_row_offset=I,
                              sfa=self.w13_sf, sfa_batch_stride=self.w13_sf[0].numel(), sfb=self.xq_sf)
            self._mark("wait+quant+fc1")
            lib.check(k.ds41_act_quant_mx_rows(lib.ptr(self.act), C.c_longlong(I), lib.ptr(self.actq), C.c_longlong(I),
                                               lib.ptr(self.actq_sf), cap, I, lib.ptr(self.total_rows), st()), "act_quant")
            self._grouped(self.w2, self.actq, self.comb, H, I, lda=I, ldo=H, out_mode=7, table=1, sfa=self.w2_sf,
                          sfa_batch_stride=self.w2_sf[0].numel(), sfb=self.actq_sf)
            self._mark("quant+fc2")
        else:
            self._grouped(self.w13, self.recv_x, self.act, I, H, lda=H, ldo=I, out_mode=4, up_row_offset=I,
                          wait_phase=2)
            self._mark("fc1")
            self._grouped(self.w2, self.act, self.comb, H, I, lda=I, ldo=H, out_mode=7, table=1)
            self._mark("fc2")
        lib.check(k.ds41_ep_mark(C.byref(a), 3, st()), "ep_mark")
        lib.check(k.ds41_ep_combine(C.byref(a), lib.ptr(self.comb), lib.ptr(extra),
                                    C.c_longlong(extra.stride(0) if extra is not None else 0), lib.ptr(out),
                                    1 if out.dtype == torch.bfloat16 else 0, st()), "ep_combine")
        self._mark("mark+combine")
        return None

    def check(self):
        lib.raise_on_status(self.status, "expert-parallel layer")

    # ------------------------------------------------------------------ NCCL + library baseline
    def baseline(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w13_ref: torch.Tensor,
                 w2_ref: torch.Tensor, extra: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Same layer with all_to_all_single and torch matmuls (bf16 weights [E_local, 2I, H] / [E_local, H, I])."""
        import torch.distributed as dist
        f, W, EL, I = self.f, self.f.world, self.e_local, self.I
        T, topk = ids.shape
        flat = ids.reshape(-1).long()
        valid = (flat >= 0) & (flat < W * EL)
        order = torch.argsort(torch.where(valid, flat, torch.full_like(flat, W * EL)), stable=True)
        order = order[: int(valid.sum())]
        sorted_ids = flat[order]
        send_counts = torch.bincount(sorted_ids, minlength=W * EL).view(W, EL)
        rows = x[order // topk].contiguous()
        wts = weights.reshape(-1)[order].contiguous()
        if W > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=f.group)
            in_split = send_counts.sum(1).tolist()
            out_split = recv_counts.sum(1).tolist()
            recv = torch.empty(sum(out_split), self.H, dtype=x.dtype, device=x.device)
            recv_wt = torch.empty(sum(out_split), dtype=wts.dtype, device=x.device)
            dist.all_to_all_single(recv, rows, out_split, in_split, group=f.group)
            dist.all_to_all_single(recv_wt, wts, out_split, in_split, group=f.group)
        else:
            recv_counts, recv, recv_wt = send_counts, rows, wts
            in_split = out_split = None
        # received rows are ordered [src][expert]; run expert by expert
        res = torch.empty_like(recv)
        starts = torch.cumsum(recv_counts.reshape(-1), 0) - recv_counts.reshape(-1)
        rc, stl = recv_counts.tolist(), starts.view(W, EL).tolist()
        for e in range(EL):
            idx = torch.cat([torch.arange(stl[s][e], stl[s][e] + rc[s][e], device=x.device) for s in range(W)])
            if idx.numel() == 0:
                continue
            h = recv[idx] @ w13_ref[e].t()
            g = h[:, :I].float().clamp(max=self.act_limit)
            u = h[:, I:].float().clamp(-self.act_limit, self.act_limit)
            a = (torch.nn.functional.silu(g) * u * recv_wt[idx, None]).to(x.dtype)
            res[idx] = a @ w2_ref[e].t()
        if W > 1:
            back = torch.empty(rows.shape[0], self.H, dtype=x.dtype, device=x.device)
            dist.all_to_all_single(back, res, in_split, out_split, group=f.group)
        else:
            back = res
        out = extra.float().clone() if extra is not None else torch.zeros(T, self.H, device=x.device)
        contrib = torch.zeros(T * topk, self.H, dtype=torch.float32, device=x.device)
        contrib[order] = back.float()
        return out + contrib.view(T, topk, self.H).sum(1)

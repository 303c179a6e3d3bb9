"""Choose the physical GPUs of this node for an N-rank launch, from what `nvidia-smi` reports as free.

    python -m ds41rt_b200.utils.select_gpus --gpus 4 --model flash --concurrency 16 --max-context 32768 [--kv-dtype fp8]
    CUDA_VISIBLE_DEVICES=$(python -m ds41rt_b200.utils.select_gpus --gpus 2 --print-devices ...) ./run.sh --gpus 2

The need of one rank is computed, not guessed: the bytes of the tensors that rank reads from the checkpoint layout
(`Catalog.shard_plan`: sliced attention / shared expert / vocabulary rows, its own routed experts), plus the window
rings, the wanted KV page pool for `concurrency` requests at `max_context` (`runtime.memory.plan_pool`), a workspace
allowance and the fixed headroom.  A GPU qualifies with   free + reclaimable >= need   where "reclaimable" is the memory
of processes the caller says will be gone before the launch (`--reclaim-pid`).  Among the qualifying GPUs the ones with
the most free memory win; ties go to the lower index.  Every GPU of an NVSwitch node reaches every peer at full
bandwidth, so topology does not enter the choice.  When the wanted pool does not fit on enough GPUs, the answer says how
many context tokens do fit (`degraded`), or the tool exits 1 with the shortfall per GPU (`--strict`).

Nothing on a GPU is changed: the tool only reads `nvidia-smi --query-gpu` / `--query-compute-apps` (`--nvidia-smi` names
another executable with the same output, which is how the CPU test drives it).
Counterpart of the reference's launcher helper that picks one or two cards by projected memory
(scripts/select-release-gpus.py: inventory, reclaimable processes, fixed + per-group bytes).
"""
from __future__ import annotations

import argparse
import json
import math
import subprocess
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

MIB = 1 << 20
WORKSPACE_BYTES = 6 << 30          # step buffers, graphs, library workspaces and the CUDA context of one rank
DTYPE_BYTES = {"BF16": 2, "F32": 4, "F8_E4M3": 1, "F8_E8M0": 1, "I8": 1, "U8": 1, "F16": 2, "I32": 4, "I64": 8}


class SelectionError(ValueError):
    pass


@dataclass(frozen=True)
class Gpu:
    index: int
    uuid: str
    name: str
    total_mib: int
    free_mib: int
    reclaim_mib: int = 0

    @property
    def usable_bytes(self) -> int:
        return min(self.total_mib, self.free_mib + self.reclaim_mib) * MIB


def _run(cmd: Sequence[str]) -> str:
    try:
        return subprocess.run(list(cmd), check=True, text=True, capture_output=True).stdout
    except (OSError, subprocess.CalledProcessError) as e:
        tail = (getattr(e, "stderr", "") or "").strip()
        raise SelectionError(f"GPU query failed: {' '.join(cmd)}" + (f": {tail}" if tail else "")) from e


def inventory(tool: str = "nvidia-smi", reclaim_pids: Sequence[int] = ()) -> List[Gpu]:
    """The node's GPUs as `nvidia-smi` sees them (one query for the GPUs, one for the compute processes)."""
    reclaim: Dict[str, int] = {}
    if reclaim_pids:
        want = set(int(p) for p in reclaim_pids)
        for line in _run([tool, "--query-compute-apps=gpu_uuid,pid,used_memory", "--format=csv,noheader,nounits"]).splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) == 3 and f[1].isdigit() and f[2].isdigit() and int(f[1]) in want:
                reclaim[f[0]] = reclaim.get(f[0], 0) + int(f[2])
    gpus = []
    for line in _run([tool, "--query-gpu=index,uuid,name,memory.total,memory.free", "--format=csv,noheader,nounits"]).splitlines():
        if not line.strip():
            continue
        f = [x.strip() for x in line.split(",")]
        if len(f) != 5 or not (f[0].isdigit() and f[3].isdigit() and f[4].isdigit()):
            raise SelectionError(f"unreadable nvidia-smi row: {line!r}")
        gpus.append(Gpu(int(f[0]), f[1], f[2], int(f[3]), int(f[4]), reclaim.get(f[1], 0)))
    if not gpus:
        raise SelectionError("nvidia-smi reported no GPUs")
    if len({g.uuid for g in gpus}) != len(gpus) or len({g.index for g in gpus}) != len(gpus):
        raise SelectionError("nvidia-smi reported a GPU twice")
    return gpus


def rank_weight_bytes(cfg, variant: str, world: int) -> int:
    """Largest device-resident checkpoint share of any rank (Engram tables stay on the host and are not counted)."""
    from ..loader.catalog import Catalog, expected_tensors
    cat = object.__new__(Catalog)
    cat.cfg, cat.expected = cfg, expected_tensors(cfg, variant)
    worst = 0
    for r in range(world):
        total = 0
        for name, (rows, cols) in cat.shard_plan(r, world).items():
            if ".engram.embed" in name:
                continue
            dt, shape = cat.expected[name][0], list(cat.expected[name][1])
            if rows is not None and shape:
                shape[0] = rows[1] - rows[0]
            if cols is not None and len(shape) > 1:
                shape[1] = cols[1] - cols[0]
            total += math.prod(shape) * DTYPE_BYTES.get(dt, 1)
        worst = max(worst, total)
    return worst


@dataclass
class Need:
    weight_bytes: int
    ring_bytes: int
    pool_bytes: int
    workspace_bytes: int
    headroom_bytes: int
    pages_wanted: int
    bytes_per_page: int
    page_tokens: int

    @property
    def fixed_bytes(self) -> int:
        return self.weight_bytes + self.ring_bytes + self.workspace_bytes + self.headroom_bytes

    @property
    def total_bytes(self) -> int:
        return self.fixed_bytes + self.pool_bytes


def rank_need(cfg, variant: str, world: int, concurrency: int, max_context: int, kv_dtype: str = "bf16",
              retained: int = 40, workspace_bytes: int = WORKSPACE_BYTES) -> Need:
    """Bytes one rank wants on its GPU.  The KV pool is per rank in full: every rank keeps the whole latent cache."""
    from ..runtime import memory as M
    plan = M.plan_pool(cfg, n_layers=cfg.n_layers, slots=concurrency, max_context=max_context, free_bytes=1 << 62,
                       kv_dtype=kv_dtype, retained=retained)
    return Need(rank_weight_bytes(cfg, variant, world), plan.ring_bytes, plan.pages_wanted * plan.bytes_per_page,
                workspace_bytes, M.HEADROOM_BYTES, plan.pages_wanted, plan.bytes_per_page, plan.page_tokens)


def choose(gpus: Sequence[Gpu], n: int, need: Need, strict: bool = False, pinned: Sequence[str] = ()) -> dict:
    """Pick `n` of `gpus`.  `pinned` (UUIDs or indices as text) must be part of the answer.  Returns the selection
    document; raises SelectionError when fewer than `n` GPUs can hold even the fixed part (or, with `strict`, the whole)."""
    if n <= 0 or n > len(gpus):
        raise SelectionError(f"{n} GPUs wanted, {len(gpus)} present")
    pins = []
    for p in pinned:
        hit = [g for g in gpus if g.uuid == p or str(g.index) == str(p)]
        if not hit:
            raise SelectionError(f"pinned GPU {p} is not on this node")
        if hit[0] not in pins:
            pins.append(hit[0])
    if len(pins) > n:
        raise SelectionError(f"{len(pins)} GPUs pinned for a {n}-GPU launch")
    rest = sorted((g for g in gpus if g not in pins), key=lambda g: (-g.usable_bytes, g.index))
    picked = pins + rest[:n - len(pins)]
    floor = min(g.usable_bytes for g in picked)
    short = {g.index: need.total_bytes - g.usable_bytes for g in picked if g.usable_bytes < need.total_bytes}
    too_small = [g.index for g in picked if g.usable_bytes < need.fixed_bytes + need.bytes_per_page]
    if too_small:
        raise SelectionError("no room for the weights on GPU(s) " + ", ".join(map(str, too_small)) +
                             f": {need.fixed_bytes / 2 ** 30:.1f} GiB fixed, "
                             f"{min(g.usable_bytes for g in picked) / 2 ** 30:.1f} GiB usable")
    if short and strict:
        raise SelectionError("the wanted KV pool does not fit: short by " +
                             ", ".join(f"{b / 2 ** 30:.1f} GiB on GPU {i}" for i, b in sorted(short.items())))
    pages = need.pages_wanted
    if short and need.bytes_per_page:
        pages = min(pages, (floor - need.fixed_bytes) // need.bytes_per_page)
    picked_sorted = sorted(picked, key=lambda g: g.index)
    return {"gpus": n, "devices": [g.index for g in picked_sorted], "uuids": [g.uuid for g in picked_sorted],
            "cuda_visible_devices": ",".join(str(g.index) for g in picked_sorted),
            "need_gib": round(need.total_bytes / 2 ** 30, 2), "fixed_gib": round(need.fixed_bytes / 2 ** 30, 2),
            "weights_gib": round(need.weight_bytes / 2 ** 30, 2), "pool_gib": round(need.pool_bytes / 2 ** 30, 2),
            "least_usable_gib": round(floor / 2 ** 30, 2), "degraded": bool(short), "pages": int(pages),
            "pages_wanted": need.pages_wanted, "pool_tokens": int(pages) * need.page_tokens,
            "reclaimed_mib": {g.index: g.reclaim_mib for g in picked_sorted if g.reclaim_mib}}


def main(argv: Optional[List[str]] = None) -> int:
    from ..config import ModelConfig
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, required=True, choices=[1, 2, 4, 8])
    ap.add_argument("--model", default="flash", choices=["flash", "small", "tiny"])
    ap.add_argument("--layers", type=int, default=0, help="layer count of a truncated flash model (0 = full)")
    ap.add_argument("--config", default="", help="official config.json instead of --model")
    ap.add_argument("--variant", default="mxfp4", choices=["mxfp4", "nvfp4"])
    ap.add_argument("--concurrency", type=int, default=4)
    ap.add_argument("--max-context", type=int, default=8192)
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp4"])
    ap.add_argument("--retained", type=int, default=40)
    ap.add_argument("--workspace-gb", type=float, default=WORKSPACE_BYTES / 2 ** 30)
    ap.add_argument("--pin", action="append", default=[], help="GPU index or UUID that must be part of the answer")
    ap.add_argument("--reclaim-pid", action="append", type=int, default=[],
                    help="process whose GPU memory will be free again before the launch (e.g. the server being replaced)")
    ap.add_argument("--strict", action="store_true", help="fail instead of shrinking the KV pool")
    ap.add_argument("--print-devices", action="store_true", help="print only the CUDA_VISIBLE_DEVICES value")
    ap.add_argument("--nvidia-smi", default="nvidia-smi")
    args = ap.parse_args(argv)
    if args.config:
        with open(args.config) as f:
            cfg = ModelConfig.from_official_json(json.load(f))
    elif args.model == "flash":
        cfg = ModelConfig.flash(args.layers) if args.layers else ModelConfig.flash()
    else:
        cfg = getattr(ModelConfig, args.model)()
    try:
        need = rank_need(cfg, args.variant, args.gpus, args.concurrency, args.max_context, args.kv_dtype,
                         args.retained, int(args.workspace_gb * 2 ** 30))
        out = choose(inventory(args.nvidia_smi, args.reclaim_pid), args.gpus, need, args.strict, args.pin)
    except SelectionError as e:
        print(json.dumps({"error": str(e)}), file=sys.stderr)
        return 1
    print(out["cuda_visible_devices"] if args.print_devices else json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

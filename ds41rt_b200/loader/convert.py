"""Offline checkpoint conversion: official layout (FP4 + UE8M0/32 routed experts) -> NVFP4 variant, shard by shard.

    python -m ds41rt_b200.loader.convert SRC_DIR DST_DIR [--model flash] [--layers N] [--link-unchanged]

Every routed-expert matrix `X.weight` (I8, two E2M1 codes per byte) + `X.scale` (UE8M0 per 32) becomes

    X.weight          U8      [n, k/2]   E2M1 codes, even element in the low nibble
    X.weight_scale    F8_E4M3 [n, k/16]  block scales
    X.weight_scale_2  F32     []         tensor scale = amax / (6 * 448)
    X.input_scale     F32     []         1.0 (activations are quantised dynamically)

by decoding the matrix to fp32 (one matrix at a time, 47 MB at Flash size) and re-quantising it with the weight-only
round-to-nearest-even NVFP4 recipe (`ops.quant_ref.quant_nvfp4`).  Every other tensor is copied byte for byte with its
container dtype.  A source shard maps to one output shard of the same file name; a shard whose tensors hold no expert
weights can be hard-linked instead of rewritten (`--link-unchanged`).  Each finished shard leaves a receipt
`<shard>.done.json` (source size + mtime + tensor count), so an interrupted run continues with the next shard; the index
is written last, and the result is validated by opening it as a `Catalog(variant="nvfp4")`.
Counterpart of the reference's offline conversion pipeline (quantization/write_export.py, export_layout.py,
validate_export.py; the NVFP4 expert contract is rust/crates/ds41rt-loader/src/v41_nvfp4.rs).
"""
from __future__ import annotations

import argparse
import json
import os
import time
from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..ops import quant_ref as Q
from .catalog import Catalog, expected_tensors
from .safetensors_io import write_safetensors


def _is_expert_weight(name: str) -> bool:
    return ".ffn.experts." in name and name.endswith(".weight")


def _is_expert_scale(name: str) -> bool:
    return ".ffn.experts." in name and name.endswith(".scale")


def convert_expert(packed: torch.Tensor, e8: torch.Tensor):
    """(I8/U8 [n, k/2], UE8M0 [n, k/32]) -> (U8 [n, k/2], F8_E4M3 [n, k/16], F32 [])."""
    vals = Q.dequant_mxfp4(packed.view(torch.uint8), e8.view(torch.uint8), 32)
    q, bs, gs = Q.quant_nvfp4(vals)
    return q.view(torch.uint8), bs, gs.reshape(()).float()


def _receipt(src_path: str, n_tensors: int) -> dict:
    st = os.stat(src_path)
    return {"source_bytes": st.st_size, "source_mtime_ns": st.st_mtime_ns, "tensors": n_tensors}


def convert_checkpoint(src: str, dst: str, cfg: ModelConfig, with_vision: bool = True, with_engram: bool = True,
                       link_unchanged: bool = False, stop_after_shards: Optional[int] = None, log=None) -> dict:
    """Convert the checkpoint in `src` (variant mxfp4) into `dst` (variant nvfp4).  Returns a summary; `complete` is
    False when `stop_after_shards` ended the run early (used by the resume test and for time-boxed runs)."""
    cat = Catalog(src, cfg, "mxfp4", with_vision, with_engram)
    want_out = expected_tensors(cfg, "nvfp4", with_vision, with_engram)
    os.makedirs(dst, exist_ok=True)
    weight_map: Dict[str, str] = {}
    done_now = skipped = experts = linked = 0
    t0 = time.time()
    complete = True
    for shard, f in cat.files.items():
        names = f.names()
        out_names = []
        for n in names:
            if _is_expert_scale(n):
                continue
            if _is_expert_weight(n):
                base = n[:-len(".weight")]
                out_names += [n, base + ".weight_scale", base + ".weight_scale_2", base + ".input_scale"]
            else:
                out_names.append(n)
        for n in out_names:
            weight_map[n] = shard
        out_path, receipt_path = os.path.join(dst, shard), os.path.join(dst, shard + ".done.json")
        receipt = _receipt(f.path, len(out_names))
        if os.path.exists(receipt_path) and os.path.exists(out_path):
            with open(receipt_path) as r:
                if json.load(r) == receipt:
                    skipped += 1
                    continue
        if stop_after_shards is not None and done_now >= stop_after_shards:
            complete = False
            continue
        has_expert = any(_is_expert_weight(n) for n in names)
        if link_unchanged and not has_expert:
            if os.path.exists(out_path):
                os.remove(out_path)
            try:
                os.link(f.path, out_path)
            except OSError:                                  # another file system: fall through to a rewrite
                pass
            else:
                linked += 1
        if not (link_unchanged and not has_expert and os.path.exists(out_path)):
            tensors, dts = {}, {}
            for n in names:
                if _is_expert_scale(n):
                    continue
                if _is_expert_weight(n):
                    base = n[:-len(".weight")]
                    q, bs, gs = convert_expert(cat.read(n), cat.read(base + ".scale"))
                    tensors[n], dts[n] = q, "U8"
                    tensors[base + ".weight_scale"], dts[base + ".weight_scale"] = bs, "F8_E4M3"
                    tensors[base + ".weight_scale_2"], dts[base + ".weight_scale_2"] = gs, "F32"
                    tensors[base + ".input_scale"], dts[base + ".input_scale"] = torch.tensor(1.0), "F32"
                    experts += 1
                else:
                    tensors[n], dts[n] = f.read(n), f.entries[n].dtype
            tmp = out_path + ".tmp"
            write_safetensors(tmp, tensors, dts)
            os.replace(tmp, out_path)
        with open(receipt_path + ".tmp", "w") as r:
            json.dump(receipt, r)
        os.replace(receipt_path + ".tmp", receipt_path)
        done_now += 1
        if log:
            log(f"{shard}: {len(out_names)} tensors ({done_now + skipped}/{len(cat.files)})")
    summary = {"complete": complete, "shards": len(cat.files), "written": done_now, "already_done": skipped,
               "linked": linked, "expert_matrices": experts, "seconds": round(time.time() - t0, 3)}
    if not complete:
        return summary
    missing = [n for n in want_out if n not in weight_map]
    if missing:
        raise RuntimeError(f"conversion would miss {len(missing)} tensors, e.g. {missing[:3]}")
    tmp = os.path.join(dst, "model.safetensors.index.json.tmp")
    with open(tmp, "w") as w:
        json.dump({"metadata": {"variant": "nvfp4", "converted_from": os.path.basename(os.path.abspath(src))},
                   "weight_map": weight_map}, w)
    os.replace(tmp, os.path.join(dst, "model.safetensors.index.json"))
    Catalog(dst, cfg, "nvfp4", with_vision, with_engram)     # the strict catalog is the validator
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--model", default="flash", choices=["flash", "small", "tiny"])
    ap.add_argument("--layers", type=int, default=0, help="layer count of a truncated flash checkpoint (0 = full)")
    ap.add_argument("--no-vision", action="store_true")
    ap.add_argument("--no-engram", action="store_true")
    ap.add_argument("--link-unchanged", action="store_true", help="hard-link shards without expert weights")
    args = ap.parse_args(argv)
    cfg = (ModelConfig.flash(args.layers) if args.layers else ModelConfig.flash()) if args.model == "flash" \
        else getattr(ModelConfig, args.model)()
    out = convert_checkpoint(args.src, args.dst, cfg, not args.no_vision, not args.no_engram, args.link_unchanged,
                             log=lambda m: print(m, flush=True))
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

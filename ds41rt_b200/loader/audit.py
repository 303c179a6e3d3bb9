"""Audit a checkpoint directory from its shard headers: structure, index agreement and identity, no weights loaded.

    python -m ds41rt_b200.loader.audit DIR [--payload-hashes] [--model flash --variant mxfp4 [--layers N]]

Per shard: the header parses, every tensor's extent matches its dtype and shape, the payloads tile the data section
without gap or overlap (`SafetensorsFile` refuses anything else), and the shard is the one the index names for each of
its tensors.  Across shards: no tensor twice, none of the index missing, shard names are plain file names.  The report
carries what identifies the checkpoint without reading 160 GB: sha256 of the index, of every shard header and of all
headers together, byte counts per dtype, and the sha256 of the side files (configuration, tokenizer).  `--payload-hashes`
additionally streams every shard once for a sha256 of its whole file.  With `--model` the tensor set is also compared
with the strict catalog of that model and variant (names, dtypes, shapes).
Counterpart of the reference's header-level checkpoint inventory (scripts/audit-ds41-checkpoint.py).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
from typing import Optional

from .safetensors_io import SafetensorsError, SafetensorsFile

ASSETS = ("config.json", "tokenizer.json", "tokenizer_config.json", "generation_config.json")


class AuditError(ValueError):
    pass


def _sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(8 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def audit(directory: str, payload_hashes: bool = False, cfg=None, variant: str = "mxfp4", with_vision: bool = True,
          with_engram: bool = True) -> dict:
    index_path = os.path.join(directory, "model.safetensors.index.json")
    try:
        raw = open(index_path, "rb").read()
        weight_map = json.loads(raw)["weight_map"]
    except (OSError, ValueError, KeyError) as e:
        raise AuditError(f"{index_path}: {e}")
    if not isinstance(weight_map, dict) or not weight_map:
        raise AuditError("the index has no weight_map")
    all_headers = hashlib.sha256()
    seen, shards, by_dtype = set(), [], {}
    for name in sorted(set(weight_map.values())):
        if os.path.basename(name) != name or name in ("", ".", ".."):
            raise AuditError(f"index names shard {name!r}: must be a plain file name")
        path = os.path.join(directory, name)
        try:
            f = SafetensorsFile(path)
        except (OSError, SafetensorsError) as e:
            raise AuditError(str(e))
        with open(path, "rb") as fh:
            head = fh.read(f.data_start)
        all_headers.update(name.encode() + b"\0" + head)
        for tensor in f.names():
            if tensor in seen:
                raise AuditError(f"{tensor}: stored in two shards")
            if weight_map.get(tensor) != name:
                raise AuditError(f"{tensor}: stored in {name}, the index says {weight_map.get(tensor)!r}")
            seen.add(tensor)
            e = f.entries[tensor]
            by_dtype[e.dtype] = by_dtype.get(e.dtype, 0) + e.nbytes
        entry = {"name": name, "bytes": os.path.getsize(path), "tensors": len(f.names()),
                 "header_sha256": hashlib.sha256(head[8:]).hexdigest()}
        if payload_hashes:
            entry["file_sha256"] = _sha256_file(path)
        shards.append(entry)
    missing = sorted(set(weight_map) - seen)
    if missing:
        raise AuditError(f"{len(missing)} tensors of the index are in no shard, e.g. {missing[:3]}")
    out = {"directory": os.path.abspath(directory), "tensors": len(seen), "shards": shards,
           "shard_bytes": sum(s["bytes"] for s in shards), "bytes_by_dtype": dict(sorted(by_dtype.items())),
           "index_sha256": hashlib.sha256(raw).hexdigest(), "headers_sha256": all_headers.hexdigest(),
           "assets_sha256": {a: _sha256_file(os.path.join(directory, a)) for a in ASSETS
                             if os.path.isfile(os.path.join(directory, a))},
           "payload_hashes": bool(payload_hashes)}
    if cfg is not None:
        from .catalog import Catalog
        try:
            Catalog(directory, cfg, variant, with_vision, with_engram)
            out["catalog"] = {"model": cfg.name, "variant": variant, "ok": True}
        except Exception as e:
            out["catalog"] = {"model": cfg.name, "variant": variant, "ok": False, "error": str(e)[:300]}
    return out


def main(argv: Optional[list] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("directory")
    ap.add_argument("--payload-hashes", action="store_true", help="also stream every shard once for a sha256 of the file")
    ap.add_argument("--model", default="", choices=["", "flash", "small", "tiny"], help="compare with this model's catalog")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--variant", default="mxfp4", choices=["mxfp4", "nvfp4"])
    ap.add_argument("--no-vision", action="store_true")
    ap.add_argument("--no-engram", action="store_true")
    args = ap.parse_args(argv)
    cfg = None
    if args.model:
        from ..config import ModelConfig
        cfg = (ModelConfig.flash(args.layers) if args.layers else ModelConfig.flash()) if args.model == "flash" \
            else getattr(ModelConfig, args.model)()
    try:
        out = audit(args.directory, args.payload_hashes, cfg, args.variant, not args.no_vision, not args.no_engram)
    except AuditError as e:
        print(json.dumps({"ok": False, "error": str(e)}))
        return 1
    out["ok"] = out.get("catalog", {}).get("ok", True)
    print(json.dumps(out, indent=1))
    return 0 if out["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())

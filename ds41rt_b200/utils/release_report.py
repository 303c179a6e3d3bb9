"""Render a results report from raw bench records: every cell is recomputed from the records or left empty.

    python -m ds41rt_b200.utils.release_report RECORDS... [--output REPORT.md] [--json REPORT.json] [--tolerance 0.05]

RECORDS are files that hold the JSON lines `bench.py` printed (logs with other text around them are fine; both arms may
share a file - a line with `"impl": "reference"` belongs to the reference arm).  Records are grouped by workload (metric,
stable part of `config`, dtype) and GPU count.  Every group goes through the record gate (`validate_bench.check_set`:
contract keys, value recomputed from ms_per_step, warm-up, clock reasons, end-to-end copies, spread across repeats); a
group that fails is shown as "-" with the gate's reasons under the table, never with a number, and nothing is carried
over from an earlier report.  What is rendered:

* results      one row per workload and GPU count: median value, ms per step, end-to-end value, repeats and spread,
               ratio to the published baseline (only where the record is allowed to quote one), the reference arm's
               value measured beside it and the ratio to it, or why that arm has no number;
* scaling      for a workload measured at several GPU counts with the same model: speed-up over the smallest count
               and efficiency (speed-up / GPU ratio), recomputed here from the per-count medians;
* clocks       median SM clock under load, its maximum and the active reasons per group;
* provenance   sha256 of every record file, the source digests the records carry (`bench.py` writes them under
               `source`; a group measured from more than one tree is called out), and the identity of the tree that
               renders the report (source digest, git commit, compilers; `source_manifest.identity`).

Counterpart of the reference's release renderers and provenance scripts (scripts/render-ds41-v7-headline.py: cells from
raw records, "-" instead of estimates, disclosure notes; scripts/summarize-ds41-upstream-release.py;
scripts/sparkinfer-release-provenance.py).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import statistics
import sys
from pathlib import Path
from typing import Dict, List, Optional, Tuple

from . import validate_bench as V

N_DEPENDENT = ("parallelism", "weights_gb_per_gpu", "kv_gb_per_gpu", "global_batch", "tokens_per_step")


def load(paths: List[Path]) -> Tuple[List[dict], Dict[str, str]]:
    """All JSON records of the files (a record is a line that parses to an object with `metric` or `impl`), each tagged
    with `_file`; plus the sha256 of every file."""
    recs, shas = [], {}
    for p in paths:
        raw = p.read_bytes()
        shas[str(p)] = hashlib.sha256(raw).hexdigest()
        for line in raw.decode("utf-8", "replace").splitlines():
            line = line.strip()
            if not line.startswith("{"):
                continue
            try:
                r = json.loads(line)
            except ValueError:
                continue
            if isinstance(r, dict) and ("metric" in r or r.get("impl") == "reference"):
                r["_file"] = p.name
                recs.append(r)
    return recs, shas


def _key(r: dict) -> Tuple[str, str, str]:
    cfg = V.stable_config(r.get("config") or {})
    return (str(r.get("metric")), json.dumps(cfg, sort_keys=True), str(r.get("dtype")))


def group(recs: List[dict]) -> Dict[Tuple, Dict[int, Dict[str, List[dict]]]]:
    """workload key -> n_gpus -> {"ours": [...], "reference": [...]}.  A reference record is filed under the workload of
    our arm with the same metric and GPU count (its config may name its own parallelism); an `unavailable` line, which
    carries no metric, is filed under every workload of its file."""
    out: Dict[Tuple, Dict[int, Dict[str, List[dict]]]] = {}
    ours = [r for r in recs if r.get("impl") != "reference"]
    for r in ours:
        out.setdefault(_key(r), {}).setdefault(int(r.get("n_gpus", 0)), {"ours": [], "reference": []})["ours"].append(r)
    for r in recs:
        if r.get("impl") != "reference":
            continue
        for key, by_n in out.items():
            for n, arms in by_n.items():
                same_file = any(o["_file"] == r["_file"] for o in arms["ours"])
                if "unavailable" in r:
                    if same_file or len(out) == 1:
                        arms["reference"].append(r)
                elif r.get("metric") == key[0] and int(r.get("n_gpus", 0)) == n:
                    arms["reference"].append(r)
    return out


def _num(v: Optional[float]) -> str:
    if v is None:
        return "-"
    return f"{v:,.0f}" if abs(v) >= 1000 else f"{v:,.1f}" if abs(v) >= 100 else f"{v:,.2f}"


def _ratio(a: Optional[float], b: Optional[float]) -> str:
    return "-" if a is None or not b else f"{a / b:.2f}x"


def _strip(r: dict) -> dict:
    return {k: v for k, v in r.items() if not k.startswith("_")}


def summarise(recs: List[dict], tolerance: float = 0.05) -> List[dict]:
    """One entry per workload and GPU count, in order of first appearance."""
    rows = []
    for key, by_n in group(recs).items():
        for n in sorted(by_n):
            arms = by_n[n]
            gate = V.check_set([_strip(r) for r in arms["ours"]], tolerance)
            head = arms["ours"][0]
            cfg = head.get("config") or {}
            row = {"metric": key[0], "model": cfg.get("model"), "parallelism": cfg.get("parallelism"), "n_gpus": n,
                   "unit": head.get("unit"), "higher_is_better": head.get("higher_is_better", True),
                   "scaling": head.get("scaling"), "layers": cfg.get("layers"), "records": len(arms["ours"]),
                   "ok": gate["ok"], "errors": gate["errors"], "warnings": gate["warnings"],
                   "files": sorted({r["_file"] for r in arms["ours"]}), "_key": key,
                   "value": None, "ms_per_step": None, "e2e": None, "spread": None, "vs_baseline": None,
                   "clocks": None, "reference": None, "reference_note": None,
                   "sources": sorted({json.dumps(r["source"], sort_keys=True) for r in arms["ours"]
                                      if isinstance(r.get("source"), dict)})}
            if len(row["sources"]) > 1:
                row["warnings"] = row["warnings"] + ["records of this group were measured from different source trees"]
            if gate["ok"]:
                good = arms["ours"]
                row.update(value=gate["median"], spread=gate["spread"], e2e=gate["e2e_median"],
                           ms_per_step=statistics.median(r["ms_per_step"] for r in good))
                vb = [r["vs_baseline"] for r in good if r.get("vs_baseline") is not None]
                row["vs_baseline"] = statistics.median(vb) if len(vb) == len(good) else None
                sm = [r["clocks"].get("sm_mhz") for r in good if isinstance(r["clocks"].get("sm_mhz"), (int, float))]
                row["clocks"] = {"sm_mhz": statistics.median(sm) if sm else None,
                                 "sm_max_mhz": good[0]["clocks"].get("sm_max_mhz"),
                                 "reasons": sorted({x for r in good for x in (r["clocks"].get("reasons") or [])})}
            ref = arms["reference"]
            measured = [r for r in ref if "unavailable" not in r]
            if measured:
                rgate = V.check_set([_strip(r) for r in measured], tolerance)
                if rgate["ok"]:
                    row["reference"] = rgate["median"]
                else:
                    row["reference_note"] = "reference arm rejected: " + "; ".join(rgate["errors"][:3])
            elif ref:
                row["reference_note"] = "reference arm unavailable: " + str(ref[0]["unavailable"])
            rows.append(row)
    return rows


def scaling_rows(rows: List[dict]) -> List[dict]:
    """Speed-up and efficiency between GPU counts of one workload family: same metric text up to the layer count, same
    model, same configuration apart from what the GPU count itself changes."""
    fam: Dict[str, List[dict]] = {}
    for r in rows:
        if not r["ok"]:
            continue
        cfg = json.loads(r["_key"][1])
        for k in N_DEPENDENT:
            cfg.pop(k, None)
        fam.setdefault(json.dumps([r["metric"], cfg, r["_key"][2]], sort_keys=True), []).append(r)
    out = []
    for members in fam.values():
        members = sorted(members, key=lambda r: r["n_gpus"])
        if len({m["n_gpus"] for m in members}) < 2:
            continue
        base = members[0]
        for m in members:
            g = m["n_gpus"] / base["n_gpus"]
            speed = (m["value"] / base["value"]) if m["higher_is_better"] else (base["value"] / m["value"])
            out.append({"metric": m["metric"], "model": m["model"], "n_gpus": m["n_gpus"], "base_gpus": base["n_gpus"],
                        "value": m["value"], "speedup": speed, "efficiency": speed / g, "scaling": m["scaling"]})
    return out


def render(rows: List[dict], shas: Dict[str, str], identity: Optional[dict] = None) -> str:
    L = ["# Results", "",
         "Every number below is the median of the listed records, recomputed from them; a cell is `-` when its records "
         "are missing or did not pass the record gate (reasons under the table).  Nothing is estimated or carried over.",
         "", "| workload | model | GPUs | value | unit | ms / step | end to end | repeats (spread) | vs published baseline "
         "| reference arm | vs reference arm |", "|---|---|---:|---:|---|---:|---:|---:|---:|---:|---:|"]
    notes = []
    for r in rows:
        rep = f"{r['records']}" + (f" ({100 * r['spread']:.1f} %)" if r["spread"] is not None and r["records"] > 1 else "")
        L.append("| " + " | ".join([
            r["metric"], str(r["model"] or "-"), str(r["n_gpus"]), _num(r["value"]), str(r["unit"] or "-"),
            _num(r["ms_per_step"]), _num(r["e2e"]), rep,
            "-" if r["vs_baseline"] is None else f"{r['vs_baseline']:.2f}x", _num(r["reference"]),
            _ratio(r["value"], r["reference"]) if r["higher_is_better"] else _ratio(r["reference"], r["value"])]) + " |")
        tag = f"{r['metric']} at {r['n_gpus']} GPU(s)"
        if not r["ok"]:
            notes.append(f"* {tag}: not quoted - " + "; ".join(r["errors"][:4]))
        elif r["vs_baseline"] is None and r["layers"] is not None:
            notes.append(f"* {tag}: no ratio to the published baseline (the record does not quote one; "
                         f"{r['layers']} layers measured)")
        if r["reference_note"]:
            notes.append(f"* {tag}: {r['reference_note']}")
    if notes:
        L += [""] + notes
    sc = scaling_rows(rows)
    if sc:
        L += ["", "## Scaling", "", "Speed-up over the smallest measured GPU count of the same workload and model; "
              "efficiency = speed-up / (GPU ratio).", "",
              "| workload | model | GPUs | value | speed-up | efficiency |", "|---|---|---:|---:|---:|---:|"]
        for s in sc:
            L.append(f"| {s['metric']} | {s['model'] or '-'} | {s['n_gpus']} | {_num(s['value'])} | "
                     f"{s['speedup']:.2f}x over {s['base_gpus']} | {100 * s['efficiency']:.0f} % |")
    ck = [r for r in rows if r["clocks"]]
    if ck:
        L += ["", "## Clocks during the timed regions", "", "| workload | GPUs | median SM MHz | max SM MHz | reasons |",
              "|---|---:|---:|---:|---|"]
        for r in ck:
            c = r["clocks"]
            L.append(f"| {r['metric']} | {r['n_gpus']} | {_num(c['sm_mhz'])} | {_num(c['sm_max_mhz'])} | "
                     f"{', '.join(c['reasons']) or 'none'} |")
    L += ["", "## Provenance", "", "| record file | sha256 |", "|---|---|"]
    L += [f"| {Path(p).name} | `{h}` |" for p, h in sorted(shas.items())]
    srcs = sorted({s for r in rows for s in r.get("sources", [])})
    if srcs:
        L += ["", "Source digests carried by the records (whole tree / kernel sources / host runtime / headers / package):", ""]
        for s in srcs:
            d = json.loads(s)
            used = sorted({f"{r['metric']} at {r['n_gpus']} GPU(s)" for r in rows if s in r.get("sources", [])})
            L.append(f"* `{d.get('tree')}` / `{d.get('kernels')}` / `{d.get('core')}` / `{d.get('headers')}` / "
                     f"`{d.get('python')}`: " + "; ".join(used))
        mixed = [f"{r['metric']} at {r['n_gpus']} GPU(s)" for r in rows if len(r.get("sources", [])) > 1]
        if mixed:
            L += ["", "Measured from more than one source tree: " + "; ".join(mixed) + "."]
    if identity:
        git = identity.get("git") or {}
        L += ["", f"Rendered from source tree `{identity.get('tree')}` ({identity.get('files')} files)"
              + (f", git commit `{git.get('commit')}`" + (" with uncommitted changes" if git.get("dirty") else "")
                 if git else "") + f"; nvcc: {identity.get('nvcc')}; host compiler: {identity.get('cxx')}; "
              f"torch {identity.get('torch')}.  The records themselves name no tree: the digest identifies the renderer's "
              "checkout, which is the measured one only when the records were produced from it."]
    return "\n".join(L) + "\n"


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("records", nargs="+", type=Path)
    ap.add_argument("--output", type=Path, default=None, help="Markdown report (default: standard output)")
    ap.add_argument("--json", type=Path, default=None, help="the same content as one JSON document")
    ap.add_argument("--tolerance", type=float, default=0.05)
    ap.add_argument("--no-identity", action="store_true", help="leave the source-tree identity out")
    args = ap.parse_args(argv)
    recs, shas = load(args.records)
    if not recs:
        print("no bench records in the given files", file=sys.stderr)
        return 1
    rows = summarise(recs, args.tolerance)
    ident = None
    if not args.no_identity:
        from . import source_manifest
        from .. import build
        ident = source_manifest.identity(build.ROOT)
    text = render(rows, shas, ident)
    if args.output:
        args.output.write_text(text)
    else:
        sys.stdout.write(text)
    if args.json:
        pub = [{k: v for k, v in r.items() if not k.startswith("_")} for r in rows]
        args.json.write_text(json.dumps({"rows": pub, "scaling": scaling_rows(rows), "records": shas,
                                         "identity": ident}, indent=1))
    return 0 if all(r["ok"] for r in rows) else 2


if __name__ == "__main__":
    raise SystemExit(main())

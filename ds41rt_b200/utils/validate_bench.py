"""Gate for benchmark records: refuse to quote a number unless its record is complete and self-consistent.

    python bench.py ... > run1.json ; python bench.py ... > run2.json
    python -m ds41rt_b200.utils.validate_bench run1.json run2.json [--tolerance 0.05] [--expect-gpus 1]

Reads the JSON line(s) `bench.py` printed (one record per file, or several lines in one file), checks each record and
the set as a whole, and prints one JSON line {"ok", "errors", "warnings", "median", ...}; exit status 1 when a hard check
fails.  CPU only: nothing is launched or contacted.  Hard checks per record:

* shape       every key of the record contract is present with the right type; `value` and `ms_per_step` are positive;
* arithmetic  value == tokens_per_step x 1000 / ms_per_step within 0.5 % when the config names `tokens_per_step`;
              the end-to-end value is present, differs from the device-timed one and is not faster than it by > 2 %;
* hygiene     warmup >= 3; the clock record has samples, no thermal or hardware slowdown reason, and a median SM clock
              within 25 % of the maximum unless `sw_power_cap` explains it; `gpu_launches` > 0;
              end-to-end copies are declared (bytes per step > 0 both ways);
* honesty     `vs_baseline` is null when the model is truncated (layers < layers_full_model) and equals
              value / baseline within 1 % otherwise; dtype and data are named; a reference-arm record is either a full
              record or an `unavailable` line.
Across records: same metric, unit, config and GPU count; the spread (max - min) / median of `value` within
`--tolerance`; the reported median is recomputed here from the records.
Counterpart of the reference's publication gate for its campaigns (scripts/validate-sampling-campaign.py: completeness,
identity, recomputed medians).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from typing import List, Tuple

REQUIRED = {"metric": str, "value": (int, float), "unit": str, "n_gpus": int, "steps": int, "warmup": int,
            "ms_per_step": (int, float), "higher_is_better": bool, "scaling": str, "dtype": str, "data": str,
            "config": dict, "clocks": dict, "e2e": dict, "gpu_launches": int}
BAD_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")
VOLATILE_CONFIG = ("setup_s", "context_at_end")             # differ between two runs of one configuration (set-up time;
                                                            # where the context stood after a time-boxed repeat count)


def stable_config(cfg: dict) -> dict:
    """The part of a record's `config` that identifies the workload (run-to-run timings of the set-up removed)."""
    return {k: v for k, v in cfg.items() if k not in VOLATILE_CONFIG}


def check_record(r: dict) -> Tuple[List[str], List[str]]:
    """(errors, warnings) of one bench record."""
    err, warn = [], []
    if r.get("impl") == "reference" and "unavailable" in r:
        if not isinstance(r["unavailable"], str) or not r["unavailable"].strip():
            err.append("reference arm: empty `unavailable` reason")
        return err, warn
    for k, t in REQUIRED.items():
        if k not in r:
            err.append(f"missing key `{k}`")
        elif not isinstance(r[k], t) or isinstance(r[k], bool) != (t is bool):
            err.append(f"`{k}` has type {type(r[k]).__name__}")
    if "vs_baseline" not in r:
        err.append("missing key `vs_baseline`")
    if err:
        return err, warn
    if not r["value"] > 0 or not r["ms_per_step"] > 0 or r["steps"] <= 0:
        err.append("value, ms_per_step and steps must be positive")
        return err, warn
    if r["warmup"] < 3:
        err.append(f"warmup {r['warmup']} < 3")
    if r["scaling"] not in ("weak", "strong"):
        err.append(f"scaling `{r['scaling']}`")
    cfg = r["config"]
    tps = cfg.get("tokens_per_step")
    if isinstance(tps, (int, float)) and tps > 0:
        want = tps * 1000.0 / r["ms_per_step"]
        if abs(want - r["value"]) > 0.005 * want:
            err.append(f"value {r['value']} != tokens_per_step x 1000 / ms_per_step = {want:.1f}")
    else:
        warn.append("config names no tokens_per_step: value not recomputed")
    # clocks
    ck = r["clocks"]
    reasons = ck.get("reasons") or []
    for b in BAD_REASONS:
        if b in reasons:
            err.append(f"clock record shows {b}")
    if not ck.get("samples"):
        err.append("clock record has no samples from the timed region")
    sm, top = ck.get("sm_mhz"), ck.get("sm_max_mhz")
    if isinstance(sm, (int, float)) and isinstance(top, (int, float)) and top > 0 and sm < 0.75 * top:
        (warn if "sw_power_cap" in reasons else err).append(
            f"median SM clock {sm} MHz is below 75 % of {top} MHz" + ("" if "sw_power_cap" in reasons
                                                                        else " with no reason active (clock lock?)"))
    if "sw_power_cap" in reasons:
        warn.append("sw_power_cap active (kept; normal under a dense load)")
    if r["gpu_launches"] <= 0:
        err.append("gpu_launches must be > 0")
    # end to end
    e = r["e2e"]
    if not isinstance(e.get("value"), (int, float)) or not e["value"] > 0:
        err.append("e2e.value missing")
    else:
        if e["value"] == r["value"]:
            err.append("e2e.value repeats the device-timed value")
        better = e["value"] > r["value"] if r["higher_is_better"] else e["value"] < r["value"]
        if better and abs(e["value"] - r["value"]) > 0.02 * r["value"]:
            err.append(f"e2e.value {e['value']} beats the device-timed {r['value']} by more than 2 %")
        if not (e.get("h2d_bytes_per_step", 0) > 0 and e.get("d2h_bytes_per_step", 0) > 0):
            err.append("e2e copies not declared (h2d / d2h bytes per step)")
    # baseline ratio
    layers, full = cfg.get("layers"), cfg.get("layers_full_model")
    truncated = isinstance(layers, int) and isinstance(full, int) and layers < full
    vb = r["vs_baseline"]
    if truncated and vb is not None:
        err.append(f"vs_baseline {vb} quoted for {layers} of {full} layers")
    base = (r.get("baseline") or {}).get("value")
    if not truncated and vb is not None and isinstance(base, (int, float)) and base > 0:
        if abs(vb - r["value"] / base) > 0.01 * r["value"] / base:
            err.append(f"vs_baseline {vb} != value / baseline = {r['value'] / base:.3f}")
    if truncated and str(layers) not in r["metric"]:
        warn.append("metric string does not name the layer count of the truncated model")
    if "synthetic" not in r["data"] and "random" not in r["data"]:
        warn.append(f"data `{r['data']}`")
    return err, warn


def check_set(records: List[dict], tolerance: float = 0.05, expect_gpus: int = 0) -> dict:
    errors, warnings = [], []
    full = []
    for i, r in enumerate(records):
        e, w = check_record(r)
        errors += [f"record {i}: {m}" for m in e]
        warnings += [f"record {i}: {m}" for m in w]
        if "unavailable" not in r and not e:
            full.append(r)
    out = {"records": len(records), "measured": len(full)}
    if full:
        head = full[0]
        for i, r in enumerate(full[1:], 1):
            for k in ("metric", "unit", "n_gpus", "dtype", "higher_is_better"):
                if r[k] != head[k]:
                    errors.append(f"record {i}: `{k}` differs from record 0")
            a, b = stable_config(r["config"]), stable_config(head["config"])
            if a != b:
                keys = sorted(k for k in set(a) | set(b) if a.get(k) != b.get(k))
                errors.append(f"record {i}: `config` differs from record 0 in {', '.join(keys)}")
        if expect_gpus and head["n_gpus"] != expect_gpus:
            errors.append(f"n_gpus {head['n_gpus']} != expected {expect_gpus}")
        vals = [r["value"] for r in full]
        med = statistics.median(vals)
        spread = (max(vals) - min(vals)) / med if med > 0 else 0.0
        if len(vals) > 1 and spread > tolerance:
            errors.append(f"spread {spread:.3f} over {len(vals)} records exceeds {tolerance}")
        out.update({"metric": head["metric"], "unit": head["unit"], "n_gpus": head["n_gpus"], "median": med,
                    "min": min(vals), "max": max(vals), "spread": round(spread, 4),
                    "e2e_median": statistics.median([r["e2e"]["value"] for r in full])})
    elif not errors:
        errors.append("no measured record")
    out.update({"ok": not errors, "errors": errors, "warnings": warnings})
    return out


def load_records(paths: List[str]) -> List[dict]:
    recs = []
    for p in paths:
        with (sys.stdin if p == "-" else open(p)) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{"):
                    try:
                        recs.append(json.loads(line))
                    except ValueError:
                        recs.append({"_unparsed": line[:80]})
    return recs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("files", nargs="+", help="files holding bench.py JSON lines ('-' = standard input)")
    ap.add_argument("--tolerance", type=float, default=0.05)
    ap.add_argument("--expect-gpus", type=int, default=0)
    args = ap.parse_args(argv)
    out = check_set(load_records(args.files), args.tolerance, args.expect_gpus)
    print(json.dumps(out))
    return 0 if out["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())

"""The benchmark-record gate: a good record passes, every broken rule is named."""
import copy
import json

from ds41rt_b200.utils.validate_bench import check_record, check_set, main

GOOD = {"metric": "decode tok/s C1 (dSpark drafter, fixed acceptance 3/4, 10 of 40 layers)", "value": 900.0,
        "unit": "tok/s", "n_gpus": 1, "steps": 20, "warmup": 5, "ms_per_step": 4.4444, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "baseline": {"value": 146.12, "layers": 40},
        "dtype": "bf16 dense / fp8-e4m3 experts", "data": "synthetic",
        "config": {"model": "flash-L10", "layers": 10, "layers_full_model": 40, "tokens_per_step": 4},
        "clocks": {"sm_mhz": 1965.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 21},
        "e2e": {"value": 888.2, "unit": "tok/s", "h2d_bytes_per_step": 68, "d2h_bytes_per_step": 48},
        "gpu_launches": 97240, "impl": "ours"}


def _broken(**changes):
    r = copy.deepcopy(GOOD)
    for k, v in changes.items():
        if "." in k:
            a, b = k.split(".")
            r[a][b] = v
        elif v is KeyError:
            r.pop(k)
        else:
            r[k] = v
    return check_record(r)[0]


def test_a_complete_record_passes_and_notes_the_power_cap():
    err, warn = check_record(GOOD)
    assert err == [] and any("sw_power_cap" in w for w in warn)
    out = check_set([GOOD, dict(GOOD, value=905.0, ms_per_step=4.4199)])
    assert out["ok"] and out["median"] == 902.5 and out["measured"] == 2


def test_each_rule_is_enforced():
    assert any("warmup" in e for e in _broken(warmup=2))
    assert any("tokens_per_step" in e for e in _broken(value=1200.0))
    assert any("hw_thermal_slowdown" in e for e in _broken(**{"clocks.reasons": ["hw_thermal_slowdown"]}))
    assert any("no samples" in e for e in _broken(**{"clocks.samples": 0}))
    assert any("clock lock" in e for e in _broken(**{"clocks.sm_mhz": 900.0, "clocks.reasons": []}))
    assert _broken(**{"clocks.sm_mhz": 1300.0}) == []                   # explained by the power cap: a warning only
    assert any("gpu_launches" in e for e in _broken(gpu_launches=0))
    assert any("repeats the device-timed" in e for e in _broken(**{"e2e.value": 900.0}))
    assert any("beats the device-timed" in e for e in _broken(**{"e2e.value": 960.0}))
    assert any("copies not declared" in e for e in _broken(**{"e2e.h2d_bytes_per_step": 0}))
    assert any("10 of 40 layers" in e for e in _broken(vs_baseline=6.2))
    assert any("missing key `clocks`" in e for e in _broken(clocks=KeyError))
    assert any("type bool" in e for e in _broken(steps=True))
    full = copy.deepcopy(GOOD)
    full["config"].update(layers=40)
    full["vs_baseline"] = 3.0
    assert any("value / baseline" in e for e in check_record(full)[0])
    full["vs_baseline"] = round(900.0 / 146.12, 3)
    assert check_record(full)[0] == []


def test_sets_must_agree_and_stay_within_the_spread(tmp_path, capsys):
    other = dict(GOOD, n_gpus=2)
    out = check_set([GOOD, other])
    assert not out["ok"] and any("n_gpus" in e for e in out["errors"])
    wide = dict(GOOD, value=800.0, ms_per_step=5.0, e2e=dict(GOOD["e2e"], value=790.0))
    assert any("spread" in e for e in check_set([GOOD, wide])["errors"])
    ref = {"impl": "reference", "unavailable": "the reference's daemon is Rust and cannot be built here"}
    assert check_set([ref, GOOD])["ok"] and not check_set([ref])["ok"]
    p = tmp_path / "run.json"
    p.write_text("NCCL version 2.28\n" + json.dumps(GOOD) + "\n")
    assert main([str(p), "--expect-gpus", "1"]) == 0
    assert json.loads(capsys.readouterr().out)["median"] == 900.0
    assert main([str(p), "--expect-gpus", "8"]) == 1

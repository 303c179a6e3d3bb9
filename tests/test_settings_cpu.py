"""Settings tiers, the KV pool plan and the operator commands (no GPU)."""
import argparse
import json
import re
import subprocess
import sys

import pytest

from ds41rt_b200 import settings as S
from ds41rt_b200.config import ModelConfig
from ds41rt_b200.runtime.memory import plan_pool


def _parser():
    p = argparse.ArgumentParser()
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp4"])
    p.add_argument("--speculative", action="store_true")
    p.add_argument("--engram-table", action="append", default=[])
    p.add_argument("--max-context", type=int, default=8192)
    return p


def test_file_environment_and_flags_override_in_that_order():
    text = "# comment\nPORT=9000\nKV_DTYPE='fp8'\nSPECULATIVE=true\nexport MAX_CONTEXT=65536  # inline\nENGRAM_TABLE=a.bin, b.bin\n"
    f = S.parse_settings_text(text)
    assert f == {"PORT": "9000", "KV_DTYPE": "fp8", "SPECULATIVE": "true", "MAX_CONTEXT": "65536",
                 "ENGRAM_TABLE": "a.bin, b.bin"}
    args = S.apply_tiers(_parser(), ["--port", "7000"], f, env={"DS41RT_KV_DTYPE": "fp4"})
    assert (args.port, args.kv_dtype, args.speculative, args.max_context) == (7000, "fp4", True, 65536)
    assert args.engram_table == ["a.bin", "b.bin"]
    assert args._origin == {"port": "flag", "kv_dtype": "env", "speculative": "file", "engram_table": "file",
                            "max_context": "file"}
    assert any(line.startswith("port=7000") for line in S.describe(args))


def test_typos_and_bad_values_are_errors():
    with pytest.raises(S.SettingsError):
        S.apply_tiers(_parser(), [], {"PROT": "1"}, env={})
    with pytest.raises(S.SettingsError):
        S.apply_tiers(_parser(), [], {"KV_DTYPE": "fp16"}, env={})
    with pytest.raises(S.SettingsError):
        S.apply_tiers(_parser(), [], {}, env={"DS41RT_PORT": "eighty"})
    with pytest.raises(S.SettingsError):
        S.parse_settings_text("lowercase=1")
    with pytest.raises(S.SettingsError):
        S.parse_settings_text("JUSTAKEY")


def test_pool_plan_wants_full_contexts_and_yields_to_memory():
    cfg = ModelConfig.flash(40)
    plan = plan_pool(cfg, n_layers=40, slots=16, max_context=1 << 20, free_bytes=60 << 30, kv_dtype="fp4")
    # four sources (three of ratio 2, one of ratio 1): 2.5 rows per token position, 288-byte KV row + bf16 index key
    assert plan.bytes_per_page == (3 * 32 + 64) * (288 + 2 * cfg.index_dim)
    assert plan.pages_wanted == (1 << 20) // 64 * 18 + 16 + 80 and plan.pages == plan.pages_wanted
    tight = plan_pool(cfg, n_layers=40, slots=16, max_context=1 << 20, free_bytes=12 << 30, kv_dtype="fp4")
    assert tight.limited_by_memory and 0 < tight.pages < plan.pages
    assert tight.pool_bytes <= tight.budget_bytes
    none = plan_pool(cfg, n_layers=40, slots=16, max_context=1 << 20, free_bytes=1 << 30, kv_dtype="fp4")
    assert none.pages == 0


def _cli(*argv):
    r = subprocess.run([sys.executable, "-m", "ds41rt_b200", *argv], capture_output=True, text=True, timeout=300)
    return r.returncode, r.stdout


def test_operator_commands():
    rc, out = _cli("doctor", "--lenient")
    rep = json.loads(out)
    assert rc == 0 and rep["libraries"]["libds41_core.so"] and rep["core_loads"] is True
    rc, out = _cli("inspect-model", "--model", "tiny")
    rep = json.loads(out)
    assert rc == 0 and rep["tensors"] > 50 and "experts" in rep["gb_by_class"]
    rc, out = _cli("tokenize", "--model", "tiny", "--text", "tool call {}")
    rep = json.loads(out)
    assert rc == 0 and rep["tokens"] == len(rep["ids"]) and rep["round_trip"]
    rc, out = _cli("plan-memory", "--model", "small", "--free-gb", "8")
    assert rc == 0 and json.loads(out)["pages"] > 0


def test_load_tensors_reads_an_exported_checkpoint(tmp_path):
    import torch
    from ds41rt_b200.loader.official import export_official
    from ds41rt_b200.models.weights import init_weights
    cfg = ModelConfig.tiny()
    export_official(cfg, init_weights(cfg, seed=0), str(tmp_path))
    rc, out = _cli("load-tensors", "--model", "tiny", "--checkpoint", str(tmp_path), "--pattern", "layers.0.attn.*")
    rep = json.loads(out)
    assert rc == 0 and rep["tensors_read"] > 3 and rep["bytes"] > 0
    rc, out = _cli("inspect-model", "--model", "tiny", "--checkpoint", str(tmp_path))
    assert rc == 0 and json.loads(out)["checkpoint"]["validated_tensors"] > 50


def test_load_plan_transport_report_and_scheduler_smoke(tmp_path):
    rc, out = _cli("make-loadplan", "--model", "tiny", "--world", "2")
    rep = json.loads(out)
    assert rc == 0 and [r["rank"] for r in rep["ranks"]] == [0, 1]
    assert rep["ranks"][0]["experts"] == [0, 7] and rep["ranks"][1]["experts"] == [8, 15]
    assert rep["ranks"][0]["device_gb"] == rep["ranks"][1]["device_gb"] > 0 and rep["ranks"][0]["sliced_tensors"] > 0
    rc, out = _cli("make-loadplan", "--model", "tiny", "--world", "2", "--rank", "1", "--list")
    plan = json.loads(out)["ranks"][0]["plan"]
    assert rc == 0 and plan["head.weight"]["rows"] == [2048, 4096] and "layers.0.ffn.experts.3.w1.weight" not in plan
    rc, out = _cli("transport-capabilities")
    rep = json.loads(out)
    assert rc == 0 and "peer_access" in rep and "transport" in rep
    rc, out = _cli("scheduler-smoke")
    rep = json.loads(out)
    assert rc == 0 and rep["ok"] and rep["plain"]["text"] == "scheduler smoke ok" and rep["admission"]["refused"] == 1
    # the tools under the same entry point
    good = {"impl": "reference", "unavailable": "not installed"}
    p = tmp_path / "r.json"
    p.write_text(json.dumps(good))
    rc, out = _cli("validate-bench", str(p))
    assert rc == 1 and "no measured record" in out


def test_stop_script_ends_the_recorded_process_group(tmp_path):
    """stop.sh signals exactly the process group that run.sh recorded, and clears the record."""
    import os
    import shutil
    import time
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    shutil.copy(os.path.join(root, "stop.sh"), tmp_path / "stop.sh")
    child = subprocess.Popen(["setsid", "sleep", "120"])
    (tmp_path / "ds41rt.pid").write_text(str(child.pid))
    r = subprocess.run(["bash", str(tmp_path / "stop.sh"), "--grace", "5"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "stopped process group" in r.stdout
    deadline = time.time() + 10
    while child.poll() is None and time.time() < deadline:
        time.sleep(0.05)
    assert child.poll() is not None and not (tmp_path / "ds41rt.pid").exists()
    r = subprocess.run(["bash", str(tmp_path / "stop.sh")], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "not running" in r.stdout
    r = subprocess.run(["bash", os.path.join(root, "run.sh"), "--gpus", "3"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 64


def test_native_selftest_of_the_host_runtime_passes():
    rc, out = _cli("selftest")
    done = re.search(r"ok (\d+) checks", out)
    assert rc == 0 and done and int(done.group(1)) >= 74 and "FAILED" not in out

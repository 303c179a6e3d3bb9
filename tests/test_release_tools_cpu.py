"""Launcher and release helpers that run without a GPU: GPU selection from an `nvidia-smi` stand-in, the source
manifest and build identity, and the report renderer over bench records."""
import copy
import json
import os
import stat
import subprocess
import sys
from pathlib import Path

import pytest

from ds41rt_b200 import build
from ds41rt_b200.config import ModelConfig
from ds41rt_b200.utils import release_report as R
from ds41rt_b200.utils import select_gpus as G
from ds41rt_b200.utils import source_manifest as M

ROOT = Path(__file__).resolve().parent.parent


# ---------------------------------------------------------------------------------------------- GPU selection
def fake_smi(tmp_path, gpus, apps=()):
    """An executable that answers the two queries `select_gpus` makes, like nvidia-smi with csv,noheader,nounits."""
    p = tmp_path / "fake-nvidia-smi"
    g = "".join(f"{i}, GPU-{i:04d}, NVIDIA B200, {total}, {free}\\n" for i, (total, free) in enumerate(gpus))
    a = "".join(f"GPU-{i:04d}, {pid}, {mib}\\n" for i, pid, mib in apps)
    p.write_text("#!/bin/sh\ncase \"$1\" in\n  --query-gpu=*) printf '" + g + "' ;;\n  --query-compute-apps=*) printf '"
                 + a + "' ;;\n  *) echo unsupported >&2; exit 3 ;;\nesac\n")
    p.chmod(p.stat().st_mode | stat.S_IXUSR)
    return str(p)


def test_rank_need_follows_the_shard_plan_and_the_pool_plan():
    cfg = ModelConfig.tiny()
    one = G.rank_need(cfg, "mxfp4", 1, concurrency=2, max_context=512)
    two = G.rank_need(cfg, "mxfp4", 2, concurrency=2, max_context=512)
    assert 0 < two.weight_bytes < one.weight_bytes            # experts and sliced matrices split, the rest replicated
    assert two.weight_bytes > one.weight_bytes // 2
    assert one.pool_bytes == one.pages_wanted * one.bytes_per_page and one.pool_bytes == two.pool_bytes
    more = G.rank_need(cfg, "mxfp4", 1, concurrency=4, max_context=2048)
    assert more.pool_bytes > one.pool_bytes and more.ring_bytes == 2 * one.ring_bytes
    assert one.total_bytes == one.fixed_bytes + one.pool_bytes


def test_most_free_gpus_win_and_reclaimable_memory_counts(tmp_path):
    need = G.Need(weight_bytes=80 << 30, ring_bytes=1 << 30, pool_bytes=10 << 30, workspace_bytes=6 << 30,
                  headroom_bytes=2 << 30, pages_wanted=10240, bytes_per_page=1 << 20, page_tokens=64)
    smi = fake_smi(tmp_path, [(183359, 150000), (183359, 40000), (183359, 183000), (183359, 120000)],
                   apps=[(1, 4242, 140000), (1, 77, 1000)])
    gpus = G.inventory(smi)
    assert [g.index for g in gpus] == [0, 1, 2, 3] and gpus[1].reclaim_mib == 0
    pick = G.choose(gpus, 2, need)
    assert pick["devices"] == [0, 2] and pick["cuda_visible_devices"] == "0,2" and not pick["degraded"]
    assert pick["pages"] == 10240 and pick["pool_tokens"] == 10240 * 64
    # GPU 1 is mostly held by the server that is being replaced: with its memory counted it beats GPU 3
    gpus = G.inventory(smi, reclaim_pids=[4242])
    assert gpus[1].reclaim_mib == 140000 and gpus[1].usable_bytes == 180000 * G.MIB
    pick = G.choose(gpus, 3, need)
    assert pick["devices"] == [0, 1, 2] and pick["reclaimed_mib"] == {1: 140000}
    # a pinned GPU is always part of the answer, by index or by UUID
    assert G.choose(gpus, 2, need, pinned=["3"])["devices"] == [2, 3]
    assert G.choose(gpus, 1, need, pinned=["GPU-0003"])["devices"] == [3]
    with pytest.raises(G.SelectionError, match="not on this node"):
        G.choose(gpus, 1, need, pinned=["GPU-nope"])
    with pytest.raises(G.SelectionError, match="4 present"):
        G.choose(gpus, 8, need)


def test_pool_shrinks_to_what_fits_or_fails_when_strict(tmp_path):
    need = G.Need(weight_bytes=80 << 30, ring_bytes=1 << 30, pool_bytes=40 << 30, workspace_bytes=6 << 30,
                  headroom_bytes=2 << 30, pages_wanted=40960, bytes_per_page=1 << 20, page_tokens=64)
    gpus = G.inventory(fake_smi(tmp_path, [(183359, 100 * 1024), (183359, 183000)]))
    pick = G.choose(gpus, 2, need)
    assert pick["degraded"] and pick["pages"] == (100 - 89) * 1024 and pick["pages_wanted"] == 40960
    with pytest.raises(G.SelectionError, match="short by 29.0 GiB on GPU 0"):
        G.choose(gpus, 2, need, strict=True)
    with pytest.raises(G.SelectionError, match="no room for the weights on GPU.s. 0"):
        G.choose(G.inventory(fake_smi(tmp_path, [(183359, 50 * 1024), (183359, 183000)])), 2, need)
    assert G.choose(gpus, 1, need)["devices"] == [1]


def test_unreadable_inventory_is_an_error_not_a_guess(tmp_path):
    bad = tmp_path / "bad-smi"
    bad.write_text("#!/bin/sh\necho '0, GPU-a, NVIDIA B200, [N/A], 100'\n")
    bad.chmod(0o755)
    with pytest.raises(G.SelectionError, match="unreadable"):
        G.inventory(str(bad))
    with pytest.raises(G.SelectionError, match="GPU query failed"):
        G.inventory(str(tmp_path / "absent"))
    empty = tmp_path / "empty-smi"
    empty.write_text("#!/bin/sh\nexit 0\n")
    empty.chmod(0o755)
    with pytest.raises(G.SelectionError, match="no GPUs"):
        G.inventory(str(empty))


def test_select_gpus_command_line(tmp_path):
    smi = fake_smi(tmp_path, [(183359, 1000), (183359, 183000), (183359, 182000)])
    cmd = [sys.executable, "-m", "ds41rt_b200", "select-gpus", "--gpus", "2", "--model", "tiny", "--nvidia-smi", smi,
           "--workspace-gb", "1"]
    out = subprocess.run(cmd + ["--print-devices"], capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0 and out.stdout.strip() == "1,2", out.stderr
    doc = json.loads(subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT).stdout)
    assert doc["uuids"] == ["GPU-0001", "GPU-0002"] and doc["gpus"] == 2
    out = subprocess.run(cmd[:5] + ["1", "--model", "tiny", "--nvidia-smi", smi, "--pin", "0"], capture_output=True,
                         text=True, cwd=ROOT)
    assert out.returncode == 1 and "no room for the weights" in out.stderr


# ---------------------------------------------------------------------------------------------- manifest / identity
def tree(tmp_path):
    root = tmp_path / "tree"
    (root / "csrc" / "kernels").mkdir(parents=True)
    (root / "pkg" / "__pycache__").mkdir(parents=True)
    (root / "_work").mkdir()
    (root / "csrc" / "kernels" / "a.cu").write_text("__global__ void k() {}\n")
    (root / "pkg" / "m.py").write_text("x = 1\n")
    (root / "pkg" / "__pycache__" / "m.cpython-312.pyc").write_bytes(b"\0")
    (root / "pkg" / "lib.so").write_bytes(b"\x7fELF")
    (root / "_work" / "probe.py").write_text("print(1)\n")
    (root / "README.md").write_text("hello\n")
    (root / "server.log").write_text("noise\n")
    (root / ".gitignore").write_text("# working files\n/_work/\n*.log\n")
    return root


def test_manifest_lists_sources_only_and_verifies(tmp_path):
    root = tree(tmp_path)
    n, digest = M.write(root, root / "SOURCE-MANIFEST.sha256")
    lines = (root / "SOURCE-MANIFEST.sha256").read_text().splitlines()
    assert n == 4 and [l.split("  ")[1] for l in lines] == ["./.gitignore", "./README.md", "./csrc/kernels/a.cu",
                                                            "./pkg/m.py"]
    rep = M.verify(root, root / "SOURCE-MANIFEST.sha256")
    assert rep["ok"] and rep["tree"] == digest and rep["files"] == 4
    # the format is the one `sha256sum -c` reads
    chk = subprocess.run(["sha256sum", "-c", "--quiet", "SOURCE-MANIFEST.sha256"], cwd=root, capture_output=True)
    assert chk.returncode == 0
    # same content elsewhere -> same digest; built files and working folders do not enter it
    (root / "pkg" / "other.o").write_bytes(b"obj")
    assert M.tree_digest(M.digests(root, "SOURCE-MANIFEST.sha256")) == digest


def test_manifest_covers_exactly_what_the_repository_tracks():
    """What the tree's .gitignore leaves out is left out here too: the inventory of this checkout is git's file list."""
    if not (ROOT / ".git").exists():
        pytest.skip("not a git checkout")
    def git(*a):
        r = subprocess.run(["git", "-C", str(ROOT), *a], capture_output=True, text=True)
        if r.returncode != 0:
            pytest.skip(f"git {a[0]} does not work here: {r.stderr.strip()[:80]}")
        return set(r.stdout.split("\n")) - {""}
    tracked, untracked = git("ls-files"), git("ls-files", "--others", "--exclude-standard")
    if not tracked:
        pytest.skip("git lists no tracked files here")
    tracked = {f for f in tracked if (ROOT / f).exists()}                       # deleted but not yet committed
    assert {k[2:] for k in M.inventory(ROOT)} == (tracked | untracked)
    with pytest.raises(M.ManifestError, match="negated"):
        import tempfile
        with tempfile.TemporaryDirectory() as d:
            (Path(d) / ".gitignore").write_text("*.log\n!keep.log\n")
            M.inventory(Path(d))


def test_manifest_reports_changed_missing_and_unlisted_files(tmp_path):
    root = tree(tmp_path)
    man = tmp_path / "m.sha256"
    M.write(root, man)
    (root / "pkg" / "m.py").write_text("x = 2\n")
    (root / "README.md").unlink()
    (root / "csrc" / "kernels" / "b.cu").write_text("// new\n")
    rep = M.verify(root, man)
    assert not rep["ok"] and rep["changed"] == ["./pkg/m.py"] and rep["missing"] == ["./README.md"]
    assert rep["unlisted"] == ["./csrc/kernels/b.cu"]
    out = subprocess.run([sys.executable, "-m", "ds41rt_b200.utils.source_manifest", "verify", "--root", str(root),
                          str(man)], capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 1 and json.loads(out.stdout)["changed"] == ["./pkg/m.py"]


def test_manifest_refuses_what_it_cannot_vouch_for(tmp_path):
    root = tree(tmp_path)
    outside = tmp_path / "outside.txt"
    outside.write_text("x")
    os.symlink(outside, root / "pkg" / "leak.py")
    with pytest.raises(M.ManifestError, match="leaves the tree"):
        M.inventory(root)
    (root / "pkg" / "leak.py").unlink()
    os.symlink(root / "pkg" / "m.py", root / "pkg" / "alias.py")           # stays inside: hashed by content
    d = M.digests(root)
    assert d["./pkg/alias.py"] == d["./pkg/m.py"]
    os.symlink(root / "csrc", root / "csrc2")
    with pytest.raises(M.ManifestError, match="directory symlink"):
        M.inventory(root)
    h = "0" * 64
    for text, why in ((f"{h} ./a\n", "line 1"), (f"{h}  ./a\n{h}  ./a\n", "twice"), (f"{h}  ./../etc/passwd\n", "leaves"),
                      ("", "empty")):
        with pytest.raises(M.ManifestError, match=why):
            M.parse(text)


def test_identity_names_the_tree_the_toolchain_and_the_state_of_the_libraries():
    doc = M.identity(ROOT)
    assert len(doc["tree"]) == 64 and doc["files"] > 100
    assert "arch=compute_100a,code=sm_100a" in doc["kernels"]["flags"] and str(ROOT) not in json.dumps(doc["kernels"])
    assert doc["kernels"]["sources"] != doc["core"]["sources"] and doc["kernels"]["headers"] == doc["core"]["headers"]
    assert doc["libraries"]["libds41_core.so"]["current"] is True           # conftest built it from these sources
    assert doc["libraries"]["libds41_core.so"]["stale"] == []


def test_library_status_sees_an_edited_source(tmp_path, monkeypatch):
    """A source edited after the build leaves no object under its new digest: the library is reported stale without
    compiling anything.  (A copy of one source is edited; the real tree is not touched.)"""
    before = build.library_status()["libds41_core.so"]
    assert before["current"] is True and before["sources"] >= 10
    src = sorted((build.CSRC / "core").glob("*.cc"))[0]
    fake = tmp_path / "core"
    fake.mkdir()
    for s in (build.CSRC / "core").glob("*.cc"):
        (fake / s.name).write_bytes(s.read_bytes() + (b"\n// edited\n" if s.name == src.name else b""))
    cxx = build._core_recipe()[1]
    monkeypatch.setattr(build, "_core_recipe", lambda: (sorted(fake.glob("*.cc")), cxx))
    after = build.library_status()["libds41_core.so"]
    assert after["current"] is False and after["stale"] == [src.name]
    # two sources with one stem (a .cu kernel file and a .cc host file) keep separate objects
    names = [p.name for p in build.OBJDIR.glob("*.o")]
    assert any(n.startswith("engram.cc.") for n in names)


# ---------------------------------------------------------------------------------------------- report renderer
def record(n=1, value=900.0, layers=40, impl="ours", **cfg):
    ms = 4 * 1000.0 / value
    r = {"metric": "decode tok/s C1", "value": value, "unit": "tok/s", "n_gpus": n, "steps": 20, "warmup": 5,
         "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
         "vs_baseline": round(value / 146.12, 3) if layers == 40 else None, "baseline": {"value": 146.12},
         "dtype": "bf16", "data": "synthetic",
         "config": {"model": "flash", "layers": layers, "layers_full_model": 40, "tokens_per_step": 4,
                    "parallelism": f"tp{n}+ep{n}", "setup_s": 1.0 + n, "context_at_end": 5000 + n, **cfg},
         "clocks": {"sm_mhz": 1900.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 12},
         "e2e": {"value": value * 0.98, "unit": "tok/s", "h2d_bytes_per_step": 68, "d2h_bytes_per_step": 48},
         "gpu_launches": 1000, "impl": impl}
    return r


def write_lines(path, recs, noise=True):
    path.write_text(("W1201 torch.distributed.run: some banner {not json}\n" if noise else "") +
                    "".join(json.dumps(r) + "\n" for r in recs))
    return path


def test_report_recomputes_medians_scaling_and_ratios(tmp_path):
    f1 = write_lines(tmp_path / "n1.log", [record(1, 400.0), record(1, 404.0), record(1, 396.0),
                                           record(1, 100.0, impl="reference")])
    f8 = write_lines(tmp_path / "n8.log", [record(8, 800.0), {"impl": "reference", "unavailable": "needs RTX workers"}])
    recs, shas = R.load([f1, f8])
    assert len(recs) == 6 and len(shas) == 2
    rows = R.summarise(recs)
    assert [(r["n_gpus"], r["records"], r["ok"]) for r in rows] == [(1, 3, True), (8, 1, True)]
    assert rows[0]["value"] == 400.0 and abs(rows[0]["spread"] - 0.02) < 1e-9 and rows[0]["reference"] == 100.0
    assert abs(rows[0]["vs_baseline"] - 400.0 / 146.12) < 1e-3 and rows[0]["e2e"] == 392.0
    assert rows[1]["reference"] is None and "needs RTX workers" in rows[1]["reference_note"]
    sc = R.scaling_rows(rows)
    assert [(s["n_gpus"], round(s["speedup"], 3), round(s["efficiency"], 3)) for s in sc] == [(1, 1.0, 1.0), (8, 2.0, 0.25)]
    text = R.render(rows, shas, {"tree": "t" * 64, "files": 3, "git": {"commit": "abc", "dirty": True}, "nvcc": "12.9",
                                 "cxx": "g++ 13", "torch": "2.11"})
    assert "| 400.0 | tok/s |" in text and "| 100.0 | 4.00x |" in text and "2.00x over 1 | 25 %" in text
    assert "reference arm unavailable: needs RTX workers" in text and "with uncommitted changes" in text
    assert "n1.log" in text and shas[str(f1)] in text and "sw_power_cap" in text
    assert "Source digests" not in text                                          # these records carry none


def test_report_names_the_source_digests_the_records_carry(tmp_path):
    a, b, c = record(1, 400.0), record(1, 401.0), record(8, 800.0)
    src = {"tree": "t1", "kernels": "k1", "core": "c1", "headers": "h1", "python": "p1"}
    a["source"], b["source"], c["source"] = src, dict(src, kernels="k2", tree="t2"), src
    rows = R.summarise(R.load([write_lines(tmp_path / "r.log", [a, b, c])])[0])
    assert len(rows[0]["sources"]) == 2 and len(rows[1]["sources"]) == 1
    assert any("different source trees" in w for w in rows[0]["warnings"])
    text = R.render(rows, {})
    assert "`t1` / `k1` / `c1` / `h1` / `p1`" in text and "`t2` / `k2`" in text
    assert "Measured from more than one source tree: decode tok/s C1 at 1 GPU(s)." in text
    # bench.py's own helper: digests of this checkout, stable between two calls
    sys.path.insert(0, str(ROOT))
    try:
        import bench
        got = bench._provenance()
    finally:
        sys.path.remove(str(ROOT))
    assert got == bench._provenance() and set(got) == {"tree", "kernels", "core", "headers", "python"}
    assert got["kernels"] == M.identity(ROOT)["kernels"]["sources"][:16]


def test_report_leaves_a_cell_empty_when_the_gate_rejects_its_records(tmp_path):
    hot = record(2, 700.0)
    hot["clocks"]["reasons"] = ["hw_thermal_slowdown"]
    wide = [record(4, 500.0), record(4, 700.0)]                                 # 33 % apart: no median is quoted
    short = record(1, 950.0, layers=10)
    short["vs_baseline"] = 6.5                                                  # a truncated model may not quote one
    f = write_lines(tmp_path / "all.log", [hot] + wide + [short, record(8, 810.0)])
    out_md, out_json = tmp_path / "report.md", tmp_path / "report.json"
    rc = R.main([str(f), "--output", str(out_md), "--json", str(out_json), "--no-identity"])
    assert rc == 2
    doc = json.loads(out_json.read_text())
    by_n = {(r["n_gpus"], r["layers"]): r for r in doc["rows"]}
    assert by_n[(2, 40)]["value"] is None and any("hw_thermal_slowdown" in e for e in by_n[(2, 40)]["errors"])
    assert by_n[(4, 40)]["value"] is None and any("spread" in e for e in by_n[(4, 40)]["errors"])
    assert by_n[(1, 10)]["value"] is None and any("10 of 40 layers" in e for e in by_n[(1, 10)]["errors"])
    assert by_n[(8, 40)]["value"] == 810.0
    text = out_md.read_text()
    assert "| 2 | - | tok/s | - | - |" in text and "not quoted - record 0: clock record shows hw_thermal_slowdown" in text
    assert doc["scaling"] == []                                                 # one usable GPU count: nothing to compare
    assert all("_key" not in r for r in doc["rows"])


def test_two_runs_of_one_configuration_are_one_group(tmp_path):
    a, b = record(1, 400.0), record(1, 402.0)
    b["config"]["setup_s"], b["config"]["context_at_end"] = 9.9, 7777          # differ run to run; not the workload
    c = copy.deepcopy(b)
    c["config"]["experts"] = "nvfp4"                                            # another workload
    rows = R.summarise(R.load([write_lines(tmp_path / "r.log", [a, b, c], noise=False)])[0])
    assert [(r["records"], r["ok"]) for r in rows] == [(2, True), (1, True)]
    assert R.main([str(tmp_path / "nothing-here.log")] if (tmp_path / "nothing-here.log").write_text("x\n") else []) == 1

"""Source manifest and build identity: say exactly which tree a number or a binary came from.

    python -m ds41rt_b200.utils.source_manifest write   [--root DIR] [--output SOURCE-MANIFEST.sha256]
    python -m ds41rt_b200.utils.source_manifest verify  [--root DIR] MANIFEST
    python -m ds41rt_b200.utils.source_manifest identity [--root DIR]

`write` lists every build-relevant file under the root as `<sha256>  ./<path>` (sorted, the format `sha256sum -c`
reads).  Left out: version control, caches, built artefacts (`*.so`, `*.o`, the object cache) and whatever the tree's
own `.gitignore` leaves out of the repository (working folders, the launcher's pid and log files, fetched outputs).
`verify` recomputes the inventory and fails on any file that is missing, changed, or present but not listed, on a
malformed or duplicate line and on a path that leaves the root; a symlink is followed only when it stays inside the root and names a regular file.  `identity` prints one JSON
document: the digest of the whole inventory, the digests of the kernel and host-runtime source sets together with the
compile commands that turn them into the two libraries, the compiler versions, the git commit when there is one, and
whether the built libraries match the sources (`build.library_status`).  Two trees with the same `tree` digest build the
same libraries with the same toolchain; bench records can carry the digest to tie a number to its sources.
Counterpart of the reference's frozen-tree verification and cache identity
(scripts/verify-release-source-manifest.py, scripts/kernel-cache-identity.py, scripts/release-digests.sh).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import re
import stat
import subprocess
import sys
from pathlib import Path, PurePosixPath
from typing import Dict, List, Optional, Tuple

LINE = re.compile(r"^([0-9a-f]{64})  (\./.+)$")
# always left out, whatever the tree says: version control, interpreter and tool caches, built objects
SKIP_DIRS = frozenset({".git", "__pycache__", ".pytest_cache", ".hypothesis", ".mypy_cache", ".ruff_cache", "obj"})
SKIP_SUFFIXES = (".pyc", ".pyo", ".so", ".o", ".a", ".cubin", ".fatbin", ".tmp")


class Ignore:
    """The tree's own `.gitignore`, read for the pattern forms it uses: `name/` and `name` (anywhere), `/name` and
    `dir/sub/` (from the root), `*.ext` and other single-star names; `#` comments.  Negations (`!`) are not supported
    and raise, so that a manifest is never silently wider or narrower than the repository."""

    def __init__(self, root: Path):
        self.anywhere, self.rooted, self.globs = set(), set(), []
        f = root / ".gitignore"
        if not f.is_file():
            return
        for raw in f.read_text().splitlines():
            pat = raw.strip()
            if not pat or pat.startswith("#"):
                continue
            if pat.startswith("!"):
                raise ManifestError(f".gitignore: negated pattern {pat!r} is not supported")
            body = pat.rstrip("/")
            if "*" in body or "?" in body or "[" in body:
                self.globs.append(body.lstrip("/"))
            elif "/" in body:
                self.rooted.add(body.lstrip("/"))
            else:
                self.anywhere.add(body)

    def match(self, rel: PurePosixPath) -> bool:
        import fnmatch
        if rel.name in self.anywhere or rel.as_posix() in self.rooted:
            return True
        return any(fnmatch.fnmatch(rel.name, g) or fnmatch.fnmatch(rel.as_posix(), g) for g in self.globs)


class ManifestError(RuntimeError):
    pass


def file_sha256(path: Path) -> str:
    h = hashlib.sha256()
    with path.open("rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _skip_dir(rel: PurePosixPath, ignore: Ignore) -> bool:
    return rel.name in SKIP_DIRS or ignore.match(rel)


def _skip_file(rel: PurePosixPath, ignore: Ignore) -> bool:
    return rel.name.endswith(SKIP_SUFFIXES) or ignore.match(rel)


def inventory(root: Path, manifest_name: Optional[str] = None) -> Dict[str, Path]:
    """`./relative/path` -> file to hash, for every build-relevant file under `root`."""
    root = root.resolve()
    ignore = Ignore(root)
    found: Dict[str, Path] = {}
    bad: List[str] = []
    for cur, dirs, files in os.walk(root, topdown=True, followlinks=False):
        rel_root = Path(cur).relative_to(root)
        keep = []
        for d in sorted(dirs):
            rel = PurePosixPath(*(rel_root / d).parts)
            if _skip_dir(rel, ignore):
                continue
            if (Path(cur) / d).is_symlink():
                bad.append(f"./{rel.as_posix()} (directory symlink)")
                continue
            keep.append(d)
        dirs[:] = keep
        for name in sorted(files):
            rel = PurePosixPath(*(rel_root / name).parts)
            if _skip_file(rel, ignore) or (manifest_name and rel.as_posix() == manifest_name):
                continue
            path = Path(cur) / name
            mode = path.lstat().st_mode
            shown = f"./{rel.as_posix()}"
            if stat.S_ISLNK(mode):
                try:
                    target = path.resolve(strict=True)
                    target.relative_to(root)
                except (OSError, ValueError):
                    bad.append(f"{shown} (symlink leaves the tree or is broken)")
                    continue
                if not target.is_file():
                    bad.append(f"{shown} (symlink to something that is not a file)")
                    continue
                found[shown] = target
            elif stat.S_ISREG(mode):
                found[shown] = path
            else:
                bad.append(f"{shown} (not a regular file)")
    if bad:
        raise ManifestError("unsupported entries: " + "; ".join(bad[:8]))
    return found


def digests(root: Path, manifest_name: Optional[str] = None) -> Dict[str, str]:
    return {k: file_sha256(p) for k, p in sorted(inventory(root, manifest_name).items())}


def render(d: Dict[str, str]) -> str:
    return "".join(f"{h}  {k}\n" for k, h in sorted(d.items()))


def tree_digest(d: Dict[str, str]) -> str:
    return hashlib.sha256(render(d).encode()).hexdigest()


def write(root: Path, output: Path) -> Tuple[int, str]:
    root = root.resolve()
    name = None
    try:
        name = output.resolve().relative_to(root).as_posix()
    except ValueError:
        pass
    d = digests(root, name)
    tmp = output.with_name(output.name + ".tmp")
    tmp.write_text(render(d))
    os.replace(tmp, output)
    return len(d), tree_digest(d)


def parse(text: str) -> Dict[str, str]:
    out: Dict[str, str] = {}
    for i, line in enumerate(text.splitlines(), 1):
        m = LINE.match(line)
        if not m:
            raise ManifestError(f"line {i}: not `<sha256>  ./<path>`")
        h, k = m.groups()
        parts = PurePosixPath(k).parts
        if ".." in parts or k.startswith(".//") or PurePosixPath(k[2:]).is_absolute():
            raise ManifestError(f"line {i}: path leaves the tree: {k}")
        if k in out:
            raise ManifestError(f"line {i}: {k} listed twice")
        out[k] = h
    if not out:
        raise ManifestError("empty manifest")
    return out


def verify(root: Path, manifest: Path) -> dict:
    """{"ok", "files", "tree", "missing", "unlisted", "changed"}; raises ManifestError for a manifest that cannot be read."""
    root = root.resolve()
    want = parse(manifest.read_text())
    name = None
    try:
        name = manifest.resolve().relative_to(root).as_posix()
    except ValueError:
        pass
    have_paths = inventory(root, name)
    missing = sorted(k for k in want if k not in have_paths)
    unlisted = sorted(k for k in have_paths if k not in want)
    changed = sorted(k for k, h in want.items() if k in have_paths and file_sha256(have_paths[k]) != h)
    return {"ok": not (missing or unlisted or changed), "files": len(want), "tree": tree_digest(want),
            "missing": missing, "unlisted": unlisted, "changed": changed}


def _version(cmd: List[str]) -> Optional[str]:
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=30).stdout.strip().splitlines()
        return out[-1 if "nvcc" in cmd[0] else 0] if out else None
    except (OSError, subprocess.SubprocessError):
        return None


def _git(root: Path) -> Optional[dict]:
    try:
        head = subprocess.run(["git", "-C", str(root), "rev-parse", "HEAD"], capture_output=True, text=True, timeout=30)
        if head.returncode != 0:
            return None
        dirty = subprocess.run(["git", "-C", str(root), "status", "--porcelain"], capture_output=True, text=True,
                               timeout=60).stdout.strip()
        return {"commit": head.stdout.strip(), "dirty": bool(dirty)}
    except (OSError, subprocess.SubprocessError):
        return None


def identity(root: Path) -> dict:
    from .. import build
    root = root.resolve()
    d = digests(root)
    sub = lambda prefix: tree_digest({k: h for k, h in d.items() if k.startswith(prefix)})
    inc = sub("./csrc/include/")
    doc = {"schema": 1, "files": len(d), "tree": tree_digest(d),
           "kernels": {"sources": sub("./csrc/kernels/"), "headers": inc, "flags": build.NVCC_FLAGS_PORTABLE},
           "core": {"sources": sub("./csrc/core/"), "headers": inc, "flags": build.CXX_FLAGS_PORTABLE},
           "python": sub("./ds41rt_b200/"), "git": _git(root)}
    try:
        doc["nvcc"] = _version([build._nvcc(), "--version"])
    except RuntimeError:
        doc["nvcc"] = None
    doc["cxx"] = _version(["g++", "--version"])
    try:
        import torch
        doc["torch"] = torch.__version__
    except Exception:                                        # pragma: no cover - torch is part of the image
        doc["torch"] = None
    doc["libraries"] = build.library_status() if root == build.ROOT else None
    return doc


def main(argv: Optional[List[str]] = None) -> int:
    from .. import build
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    w = sub.add_parser("write")
    w.add_argument("--root", type=Path, default=build.ROOT)
    w.add_argument("--output", type=Path, default=None)
    v = sub.add_parser("verify")
    v.add_argument("--root", type=Path, default=build.ROOT)
    v.add_argument("manifest", type=Path)
    i = sub.add_parser("identity")
    i.add_argument("--root", type=Path, default=build.ROOT)
    args = ap.parse_args(argv)
    try:
        if args.cmd == "write":
            out = args.output or args.root / "SOURCE-MANIFEST.sha256"
            n, tree = write(args.root, out)
            print(json.dumps({"written": str(out), "files": n, "tree": tree}))
            return 0
        if args.cmd == "verify":
            rep = verify(args.root, args.manifest)
            print(json.dumps(rep))
            return 0 if rep["ok"] else 1
        print(json.dumps(identity(args.root), indent=1))
        return 0
    except (ManifestError, OSError) as e:
        print(json.dumps({"ok": False, "error": str(e)}), file=sys.stderr)
        return 1


if __name__ == "__main__":
    raise SystemExit(main())

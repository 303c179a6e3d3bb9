"""Three tiers of settings for the launcher: a KEY=VALUE file, the environment, the command line.

Precedence (lowest first): built-in default < settings file < environment (`DS41RT_<KEY>`) < explicit command-line
flag.  The file format is the reference's shell-style config (ds41rt.config:1-120 of the reference): one KEY=VALUE per
line, `#` comments, optional quotes, keys in upper case with underscores; `--settings path` names it, else
`./ds41rt.config` is read when present.  Keys map onto the flags of `python -m ds41rt_b200 serve` by lower-casing
(`MAX_CONTEXT=65536` is `--max-context 65536`); example overlays live under examples/configs/.
Reference: rust/crates/ds41rt-daemon/src/cli.rs:603-735 (flags with environment fallbacks), run.sh:15-100 (overrides).
"""
from __future__ import annotations

import argparse
import os
from typing import Dict, List, Optional, Sequence

ENV_PREFIX = "DS41RT_"
DEFAULT_FILE = "ds41rt.config"


class SettingsError(ValueError):
    pass


def parse_settings_text(text: str, origin: str = "<settings>") -> Dict[str, str]:
    out: Dict[str, str] = {}
    for n, raw in enumerate(text.splitlines(), 1):
        line = raw.strip()
        if not line or line.startswith("#"):
            continue
        if line.startswith("export "):
            line = line[7:].lstrip()
        if "=" not in line:
            raise SettingsError(f"{origin}:{n}: expected KEY=VALUE")
        key, val = line.split("=", 1)
        key, val = key.strip(), val.strip()
        if not key.replace("_", "").isalnum() or key != key.upper():
            raise SettingsError(f"{origin}:{n}: bad key {key!r} (upper case, digits and underscores)")
        if len(val) >= 2 and val[0] == val[-1] and val[0] in "\"'":
            val = val[1:-1]
        elif " #" in val:
            val = val.split(" #", 1)[0].rstrip()
        out[key] = val
    return out


def load_settings_file(path: Optional[str]) -> Dict[str, str]:
    if path is None:
        if not os.path.exists(DEFAULT_FILE):
            return {}
        path = DEFAULT_FILE
    with open(path) as f:
        return parse_settings_text(f.read(), path)


def _coerce(action: argparse.Action, val: str, where: str):
    if isinstance(action, (argparse._StoreTrueAction, argparse._StoreFalseAction)):
        low = val.strip().lower()
        if low in ("1", "true", "yes", "on"):
            return True
        if low in ("0", "false", "no", "off", ""):
            return False
        raise SettingsError(f"{where}: expected a boolean, got {val!r}")
    if isinstance(action, argparse._AppendAction):
        return [v for v in (x.strip() for x in val.split(",")) if v]
    conv = action.type or str
    try:
        out = conv(val)
    except Exception:
        raise SettingsError(f"{where}: cannot read {val!r} as {getattr(conv, '__name__', conv)}")
    if action.choices is not None and out not in action.choices:
        raise SettingsError(f"{where}: {val!r} is not one of {sorted(action.choices)}")
    return out


def apply_tiers(parser: argparse.ArgumentParser, argv: Sequence[str], file_values: Dict[str, str],
                env: Optional[Dict[str, str]] = None) -> argparse.Namespace:
    """Parse `argv` with `parser`, then fill every option the command line did not name from the environment, else
    from the settings file.  Unknown keys in the file are an error (a typo must not pass silently)."""
    env = os.environ if env is None else env
    args = parser.parse_args(list(argv))
    by_key = {}
    for a in parser._actions:
        if a.dest in ("help",) or not a.option_strings:
            continue
        by_key[a.dest.upper()] = a
    named = set()
    for tok in argv:
        if tok.startswith("--"):
            named.add(tok[2:].split("=", 1)[0].replace("-", "_").upper())
    unknown = [k for k in file_values if k not in by_key]
    if unknown:
        raise SettingsError(f"settings file: unknown keys {sorted(unknown)} (known: {sorted(by_key)})")
    origin = {}
    for key, action in by_key.items():
        if key in named:
            origin[action.dest] = "flag"
            continue
        if ENV_PREFIX + key in env:
            setattr(args, action.dest, _coerce(action, env[ENV_PREFIX + key], f"${ENV_PREFIX}{key}"))
            origin[action.dest] = "env"
        elif key in file_values:
            setattr(args, action.dest, _coerce(action, file_values[key], f"settings file {key}"))
            origin[action.dest] = "file"
        else:
            origin[action.dest] = "default"
    args._origin = origin
    return args


def describe(args: argparse.Namespace) -> List[str]:
    """One line per option with the tier its value came from (for `doctor` and start-up logs)."""
    origin = getattr(args, "_origin", {})
    return [f"{k}={getattr(args, k)!r} ({origin[k]})" for k in sorted(origin)]

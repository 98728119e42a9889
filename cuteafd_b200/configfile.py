"""Operator configuration: a KEY=VALUE file (+ `--set K=V` overrides) that becomes the argv of a command.

    MODEL=/models/Qwen3-235B-A22B-NVFP4        ->  serve --model /models/Qwen3-235B-A22B-NVFP4
    LISTEN=0.0.0.0:8000                             --listen 0.0.0.0:8000
    HOST_CACHE_GIB=64                               --host-cache-gib 64
    ENABLE_BENCH=true                               --enable-bench

Rules: one `KEY=VALUE` per line, `#` comments, blank lines ignored, optional quotes around the value, `${OTHER_KEY}`
and `${ENV:NAME}` expand.  `COMMAND` picks the sub-command (default `serve`).  Keys map to flags by lower-casing and
turning `_` into `-`; booleans (`true/on/yes/1`) emit the bare flag, (`false/off/no/0`) emit nothing.  A key that is
not a flag of the command is an error that names the closest flag; retired spellings are rejected with their
replacement named, never silently accepted.

Reference: cuteafd.config:1-107 + run.sh:33-49 (KEY=VALUE file with --set overrides), run.sh:90-96 and
cli.rs:1075-1079 (deprecated spellings rejected with the replacement named).
"""
from __future__ import annotations

import difflib
import os
import re

RETIRED = {"SNAPSHOT": "MODEL", "KV_POOL_TOKENS": "POOL_TOKENS", "SPECULATOR": "DRAFT", "HOST_CACHE_BYTES": "HOST_CACHE_GIB",
           "PREFILL_CHUNK": "PREFILL_BATCH_TOKENS", "API_KEYS": "API_KEY_FILE"}
TRUE, FALSE = {"true", "on", "yes", "1"}, {"false", "off", "no", "0"}
_VAR = re.compile(r"\$\{(ENV:)?([A-Za-z_][A-Za-z0-9_]*)\}")


class ConfigError(ValueError):
    pass


def parse_text(text: str, where: str = "<config>") -> dict:
    out: dict = {}
    for n, line in enumerate(text.splitlines(), 1):
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        if "=" not in line:
            raise ConfigError(f"{where}:{n}: expected KEY=VALUE, got {line!r}")
        k, v = line.split("=", 1)
        k, v = k.strip(), v.strip()
        if not re.fullmatch(r"[A-Z][A-Z0-9_]*", k):
            raise ConfigError(f"{where}:{n}: key {k!r} must be UPPER_SNAKE_CASE")
        if len(v) >= 2 and v[0] == v[-1] and v[0] in "\"'":
            v = v[1:-1]
        elif " #" in v:
            v = v.split(" #", 1)[0].rstrip()
        if k in RETIRED:
            raise ConfigError(f"{where}:{n}: {k} was retired; use {RETIRED[k]}")
        out[k] = v
    return out


def apply_overrides(cfg: dict, sets: list[str]) -> dict:
    cfg = dict(cfg)
    for s in sets or []:
        if "=" not in s:
            raise ConfigError(f"--set wants K=V, got {s!r}")
        k, v = s.split("=", 1)
        k = k.strip().upper().replace("-", "_")
        if k in RETIRED:
            raise ConfigError(f"--set {k}: retired; use {RETIRED[k]}")
        cfg[k] = v.strip()
    return cfg


def expand(cfg: dict, env=None) -> dict:
    env = os.environ if env is None else env

    def sub(v: str, depth: int = 0) -> str:
        if depth > 8:
            raise ConfigError(f"reference loop while expanding {v!r}")

        def rep(m):
            if m.group(1):
                if m.group(2) not in env:
                    raise ConfigError(f"environment variable {m.group(2)} is not set")
                return env[m.group(2)]
            if m.group(2) not in cfg:
                raise ConfigError(f"${{{m.group(2)}}} is not defined in the configuration")
            return sub(cfg[m.group(2)], depth + 1)
        return _VAR.sub(rep, v)
    return {k: sub(v) for k, v in cfg.items()}


def flags_of(parser) -> dict:
    """flag spelling ('--host-cache-gib') -> argparse action, for one sub-command parser."""
    return {o: a for a in parser._actions for o in a.option_strings if o.startswith("--")}


def to_argv(cfg: dict, subparsers: dict) -> list[str]:
    """`subparsers`: command name -> its argparse parser.  Returns [command, flags...]."""
    cfg = expand(cfg)
    cmd = cfg.pop("COMMAND", "serve")
    if cmd not in subparsers:
        raise ConfigError(f"COMMAND={cmd}: no such command (have: {', '.join(sorted(subparsers))})")
    flags = flags_of(subparsers[cmd])
    argv = [cmd]
    for k, v in cfg.items():
        flag = "--" + k.lower().replace("_", "-")
        act = flags.get(flag)
        if act is None:
            near = difflib.get_close_matches(flag, list(flags), n=1)
            raise ConfigError(f"{k}: `{cmd}` has no flag {flag}" + (f" (did you mean {near[0][2:].upper().replace('-', '_')}?)" if near else ""))
        if act.nargs == 0:                                   # store_true style
            if v.lower() in TRUE:
                argv.append(flag)
            elif v.lower() not in FALSE:
                raise ConfigError(f"{k}: expected a boolean, got {v!r}")
        else:
            if act.choices and v not in act.choices:
                raise ConfigError(f"{k}={v}: expected one of {', '.join(map(str, act.choices))}")
            argv += [flag, v]
    return argv


def load(path: str, sets: list[str] | None = None) -> dict:
    with open(path) as f:
        return apply_overrides(parse_text(f.read(), path), sets or [])

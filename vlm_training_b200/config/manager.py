"""TOML + command-line configuration loader.

Precedence is dataclass defaults < TOML file (``--config path``) < dotted
command-line overrides (``--data.seq_len 8192`` or ``--data.seq_len=8192``),
the same precedence the reference gets from tomllib + tyro
(reference: train/config_manager.py:13-70).  Unknown TOML keys and unknown
command-line options are errors.  The override parser is implemented here,
without a CLI library, so the trainer has no import-time dependency besides
the standard library.
"""
from __future__ import annotations

import dataclasses
import tomllib
import typing
from typing import Any, Sequence

from .schema import Config


def _fill(cls, values: dict, path: str):
    if not isinstance(values, dict):
        raise ValueError(f"[{path}] must be a table, got {type(values).__name__}")
    known = {f.name: f for f in dataclasses.fields(cls)}
    hints = typing.get_type_hints(cls)
    kwargs = {}
    for key, val in values.items():
        if key not in known:
            raise ValueError(f"unknown configuration key '{path + '.' if path else ''}{key}'")
        tp = hints[key]
        if dataclasses.is_dataclass(tp):
            kwargs[key] = _fill(tp, val, f"{path + '.' if path else ''}{key}")
        else:
            kwargs[key] = _coerce(val, tp, f"{path}.{key}")
    return cls(**kwargs)


def _coerce(val: Any, tp, where: str):
    if tp is bool:
        if isinstance(val, bool):
            return val
        if isinstance(val, str):
            low = val.strip().lower()
            if low in ("1", "true", "yes", "on"):
                return True
            if low in ("0", "false", "no", "off"):
                return False
        raise ValueError(f"{where}: expected a boolean, got {val!r}")
    if tp is int:
        if isinstance(val, bool):
            raise ValueError(f"{where}: expected an integer, got {val!r}")
        if isinstance(val, float) and val.is_integer():
            return int(val)
        return int(val)
    if tp is float:
        return float(val)
    if tp is str:
        return str(val)
    return val


class ConfigManager:
    """``ConfigManager(Config).parse_args(argv)`` → populated ``Config``."""

    def __init__(self, config_cls=Config):
        self.config_cls = config_cls

    # -- TOML ---------------------------------------------------------------
    @staticmethod
    def _find_config_path(argv: Sequence[str]) -> str | None:
        for i, tok in enumerate(argv):
            if tok == "--config":
                if i + 1 >= len(argv):
                    raise ValueError("--config needs a path")
                return argv[i + 1]
            if tok.startswith("--config="):
                return tok.split("=", 1)[1]
        return None

    def from_toml(self, path: str):
        with open(path, "rb") as fh:
            raw = tomllib.load(fh)
        cfg = _fill(self.config_cls, raw, "")
        if hasattr(cfg, "config"):
            cfg.config = path
        return cfg

    # -- CLI ----------------------------------------------------------------
    def _apply_override(self, cfg, dotted: str, raw: str | None):
        node = cfg
        parts = dotted.replace("-", "_").split(".")
        hints = None
        for i, part in enumerate(parts):
            if not dataclasses.is_dataclass(node) or part not in {f.name for f in dataclasses.fields(node)}:
                raise ValueError(f"unknown option --{dotted}")
            hints = typing.get_type_hints(type(node))
            if i < len(parts) - 1:
                node = getattr(node, part)
        leaf = parts[-1]
        tp = hints[leaf]
        if dataclasses.is_dataclass(tp):
            raise ValueError(f"--{dotted} names a section, not a field")
        if raw is None:
            if tp is not bool:
                raise ValueError(f"--{dotted} needs a value")
            raw = "true"
        setattr(node, leaf, _coerce(raw, tp, dotted))

    def parse_args(self, argv: Sequence[str] | None = None):
        argv = list(argv or [])
        path = self._find_config_path(argv)
        cfg = self.from_toml(path) if path else self.config_cls()
        i = 0
        while i < len(argv):
            tok = argv[i]
            if not tok.startswith("--"):
                raise ValueError(f"unexpected argument {tok!r}")
            body = tok[2:]
            if "=" in body:
                key, val = body.split("=", 1)
                i += 1
            else:
                key = body
                nxt = argv[i + 1] if i + 1 < len(argv) else None
                if nxt is not None and not nxt.startswith("--"):
                    val, i = nxt, i + 2
                else:
                    val, i = None, i + 1
            if key.startswith("no-") or key.startswith("no_"):
                # --no-training.compile style negation
                self._apply_override(cfg, key[3:], "false")
                continue
            if key == "config":
                continue
            self._apply_override(cfg, key, val)
        return cfg


def to_flat_dict(cfg) -> dict:
    """Nested dataclass → flat ``section.key`` dict (for run logging)."""
    out = {}

    def rec(node, prefix):
        for f in dataclasses.fields(node):
            v = getattr(node, f.name)
            if dataclasses.is_dataclass(v):
                rec(v, f"{prefix}{f.name}.")
            else:
                out[f"{prefix}{f.name}"] = v

    rec(cfg, "")
    return out

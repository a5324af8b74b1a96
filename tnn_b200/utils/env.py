"""``.env`` files and typed environment lookups.

Same rules as the reference's ``EnvLoader`` (include/utils/env.hpp:13-136): one ``KEY=value`` per line, blank lines
and lines starting with ``#`` ignored, lines without ``=`` ignored, key and value trimmed, an unquoted value ends at
the first ``#``, one pair of matching single or double quotes around the value is removed, keys containing blanks
or ``=`` are skipped; every accepted pair is exported to the process environment (overwriting). ``get`` looks in
the loaded file first, then in the process environment, and converts to the type of the default.

Variables the framework reads: ``DEVICE_TYPE`` (``CPU`` / ``CUDA`` default device of the examples and the CLI,
examples/gpt2_inference.cpp:31), ``AUGMENTATION`` / ``tunx_AUGMENTATION`` (turn the image augmentation pipeline on,
src/data_loading/data_loading.cpp:98), and the ``TNNB_*`` switches documented where they are used.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

_TRUE = {"1", "true", "yes", "on"}


class EnvLoader:
    def __init__(self, file_path: str = "./.env", quiet: bool = True):
        self.vars: Dict[str, str] = {}
        self.loaded = self.load_env_file(file_path, quiet)

    def load_env_file(self, file_path: str = "./.env", quiet: bool = True) -> bool:
        try:
            f = open(file_path, "r")
        except OSError:
            if not quiet:
                print(f"Warning: Could not open .env file: {file_path}")
            return False
        with f:
            for line in f:
                line = line.strip(" \t\r\n")
                if not line or line[0] == "#" or "=" not in line:
                    continue
                key, value = line.split("=", 1)
                key, value = key.strip(" \t\r\n"), value.strip(" \t\r\n")
                if value and value[0] not in "\"'" and "#" in value:
                    value = value[:value.index("#")].strip(" \t\r\n")
                if len(value) >= 2 and value[0] == value[-1] and value[0] in "\"'":
                    value = value[1:-1]
                if not key or any(c in key for c in "= \t"):
                    continue
                self.vars[key] = value
                os.environ[key] = value
        return True

    def get(self, name: str, default: Any = None) -> Any:
        raw: Optional[str] = self.vars.get(name, os.environ.get(name))
        if raw is None:
            return default
        return from_str(raw, type(default) if default is not None else str)


def from_str(text: str, kind: type = str) -> Any:
    """String to bool / int / float / str (the reference's ``from_str<T>``, include/utils/misc.hpp:12-53)."""
    if kind is bool:
        return text.strip().lower() in _TRUE
    if kind is int:
        return int(text.strip(), 0)
    if kind is float:
        return float(text)
    return text


def get_env(name: str, default: Any = None) -> Any:
    raw = os.environ.get(name)
    if raw is None:
        return default
    return from_str(raw, type(default) if default is not None else str)


def default_device_type() -> str:
    """``DEVICE_TYPE`` from the environment (``CPU`` or ``CUDA``), else CUDA when a GPU is present."""
    import torch

    v = os.environ.get("DEVICE_TYPE", "").strip().upper()
    if v in ("CPU", "CUDA", "GPU"):
        return "CUDA" if v in ("CUDA", "GPU") else "CPU"
    return "CUDA" if torch.cuda.is_available() else "CPU"


def augmentation_enabled() -> bool:
    return get_env("AUGMENTATION", False) or get_env("tunx_AUGMENTATION", False)

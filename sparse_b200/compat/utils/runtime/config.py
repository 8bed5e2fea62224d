"""`utils.runtime.config` of the reference (utils/runtime/config.py:11-229): the
environment helpers, and the ERS configuration reader that `scripts/perf.py`
imports.  ERS (expert replica scheduling across nodes) is outside the MoE-layer
path built here: the reader returns a disabled configuration and refuses an
environment that switches ERS on."""
from __future__ import annotations

import os
from dataclasses import dataclass


def env_value(name: str, default: str = "") -> str:
    return str(os.environ.get(name, default))


def env_flag(name: str, default: str = "0") -> bool:
    return env_value(name, default).strip().lower() in ("1", "true", "yes", "on")


@dataclass(frozen=True)
class ERSRuntimeConfig:
    enabled: bool = False


def ers_config_from_env() -> ERSRuntimeConfig:
    if env_flag("SPARSE_ERS_ENABLE", "0"):
        raise NotImplementedError("SPARSE_ERS_ENABLE=1: ERS is not part of the B200 MoE-layer path")
    return ERSRuntimeConfig(enabled=False)

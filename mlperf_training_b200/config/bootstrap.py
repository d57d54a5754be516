"""Bind configuration values to environment variables before the modules that read them are imported.

Kernels and runtime switches of this package read a few ``B200_*`` environment variables at import
time (library path, verbosity, NVLS use).  A configuration file therefore has to reach the
environment *first*.  ``apply_env_bootstrap`` does what the reference's bootstrap does for its
~170 gin bindings (generative_recommenders/dlrm_v4/train/_env_bootstrap.py:82-260):

* a value already present in the environment wins over the configuration, and the override is
  logged;
* booleans are written as ``1`` / ``0`` (``0`` is always a kill switch);
* a *group* of switches that only make sense together (an "arm") is either fully on or reported:
  a partial arm is detected and returned so the caller can refuse to start.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field


@dataclass
class BootstrapReport:
    bound: dict = field(default_factory=dict)          # variable -> value written
    kept: dict = field(default_factory=dict)           # variable -> pre-set value that won
    partial_arms: dict = field(default_factory=dict)   # arm -> {"on": [...], "off": [...]}

    def lines(self) -> list[str]:
        out = [f"[bootstrap] {k}={v}" for k, v in sorted(self.bound.items())]
        out += [f"[bootstrap] {k} kept from the environment ({v!r} overrides the configuration)" for k, v in sorted(self.kept.items())]
        out += [f"[bootstrap] partial arm '{a}': on={d['on']} off={d['off']}" for a, d in sorted(self.partial_arms.items())]
        return out


def _as_env(v) -> str:
    if isinstance(v, bool):
        return "1" if v else "0"
    return str(v)


def apply_env_bootstrap(bindings: dict, values: dict, arms: dict | None = None, environ=None) -> BootstrapReport:
    """``bindings``: configuration key -> environment variable.  ``values``: configuration key ->
    value (missing keys are skipped).  ``arms``: arm name -> list of configuration keys that must
    be all-on or all-off."""
    env = os.environ if environ is None else environ
    rep = BootstrapReport()
    for key, var in bindings.items():
        if key not in values or values[key] is None:
            continue
        want = _as_env(values[key])
        if var in env and env[var] != "":
            if env[var] != want:
                rep.kept[var] = env[var]
            continue
        env[var] = want
        rep.bound[var] = want
    for arm, keys in (arms or {}).items():
        state = {k: env.get(bindings[k], "0") not in ("", "0", "false", "False") for k in keys if k in bindings}
        on, off = [k for k, v in state.items() if v], [k for k, v in state.items() if not v]
        if on and off:
            rep.partial_arms[arm] = {"on": on, "off": off}
    return rep


# configuration keys of this package that are read from the environment by lower layers
DEFAULT_BINDINGS = {
    "quiet": "B200_QUIET", "verbose": "B200_VERBOSE", "nvls": "NCCL_NVLS_ENABLE", "pg_timeout_s": "PG_TIMEOUT_S",
    "alloc_conf": "PYTORCH_CUDA_ALLOC_CONF", "fprop_switch_step": "FLUX_FPROP_SWITCH_STEP", "healing_iter": "HEALING_ITER",
}

"""Configuration system: three stacked mechanisms, environment always wins.

1. ``config_<SYSTEM>.sh`` files: plain ``export KEY=VALUE`` lines.  ``load_shell_defaults`` turns
   them into *defaults* - a variable already present in the environment keeps its value - exactly as
   the reference's launcher does (small_llm_pretraining/primus/run_with_docker.sh:32-44).
2. Experiment YAML with ``${VAR:default}`` substitution, typed casting, ``modules.<name>.overrides``
   layering over a packaged base and ``key=value`` command-line overrides
   (small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:1-15,29-37;
   llama2_sft/primus/run_and_time.sh:15-17).
3. ``env_int / env_str / env_float / env_bool / env_path / env_str_map`` helpers that bind a knob
   to an environment variable with a default - the role of the gin macros of the recommender
   workload (generative_recommenders/dlrm_v4/utils.py:1537-1632, gin ``@x/env_int()``).

Convention kept from the reference: features default off in code and on in config, ``=0`` is always
a kill switch.
"""
from __future__ import annotations

import copy
import os
import re
import shlex
from pathlib import Path
from typing import Any, Mapping

import yaml

_VAR = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)(?::([^}]*))?\}")
_EXPORT = re.compile(r"^\s*(?:export\s+)?([A-Za-z_][A-Za-z0-9_]*)=(.*)$")


# --------------------------------------------------------------------------------------
# typed env helpers
# --------------------------------------------------------------------------------------
def env_str(name: str, default: str = "", env: Mapping[str, str] | None = None) -> str:
    env = os.environ if env is None else env
    return env.get(name, default)


def env_int(name: str, default: int = 0, env: Mapping[str, str] | None = None) -> int:
    v = env_str(name, "", env)
    return int(v) if v.strip() != "" else default


def env_float(name: str, default: float = 0.0, env: Mapping[str, str] | None = None) -> float:
    v = env_str(name, "", env)
    return float(v) if v.strip() != "" else default


def env_bool(name: str, default: bool = False, env: Mapping[str, str] | None = None) -> bool:
    v = env_str(name, "", env).strip().lower()
    if v == "":
        return default
    return v not in ("0", "false", "no", "off", "none")


def env_path(name: str, default: str = "", env: Mapping[str, str] | None = None) -> Path:
    return Path(env_str(name, default, env)).expanduser()


def env_str_map(name: str, default: str = "", env: Mapping[str, str] | None = None) -> dict[str, str]:
    """``"a:1,b:2"`` -> ``{"a": "1", "b": "2"}``."""
    out = {}
    for item in env_str(name, default, env).split(","):
        if ":" in item:
            k, v = item.split(":", 1)
            out[k.strip()] = v.strip()
    return out


# --------------------------------------------------------------------------------------
# shell config files
# --------------------------------------------------------------------------------------
def parse_shell_exports(text: str, env: Mapping[str, str] | None = None) -> dict[str, str]:
    """``export K=V`` / ``K=V`` lines of a ``config_*.sh`` file, in order, with ``$VAR`` /
    ``${VAR}`` / ``${VAR:-default}`` references resolved against earlier lines and ``env``.
    Lines that are not simple assignments (``source``, conditionals, functions) are skipped."""
    known: dict[str, str] = dict(env or {})
    out: dict[str, str] = {}
    ref = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)(?::-([^}]*))?\}|\$([A-Za-z_][A-Za-z0-9_]*)")

    def expand(val: str) -> str:
        def sub(m):
            name = m.group(1) or m.group(3)
            if name in known and known[name] != "":
                return known[name]
            return m.group(2) if m.group(2) is not None else known.get(name, "")
        return ref.sub(sub, val)

    for raw in text.splitlines():
        line = raw.split(" #", 1)[0] if not raw.lstrip().startswith("#") else ""
        m = _EXPORT.match(line)
        if not m:
            continue
        key, val = m.group(1), m.group(2).strip()
        try:
            parts = shlex.split(val, posix=True)
            val = parts[0] if len(parts) == 1 else (" ".join(parts) if parts else "")
        except ValueError:
            pass
        val = expand(val)
        out[key] = val
        if key not in (env or {}):   # a pre-set variable keeps its value for later references too
            known[key] = val
    return out


def load_shell_defaults(path: str | os.PathLike, env: dict[str, str] | None = None) -> dict[str, str]:
    """Apply a ``config_*.sh`` file to ``env`` (default ``os.environ``) as defaults: variables that
    are already set win.  Returns the values that were applied."""
    target = os.environ if env is None else env
    values = parse_shell_exports(Path(path).read_text(), target)
    applied = {}
    for k, v in values.items():
        if k not in target:
            target[k] = v
            applied[k] = v
    return applied


# --------------------------------------------------------------------------------------
# YAML experiments
# --------------------------------------------------------------------------------------
def _cast(s: str) -> Any:
    t = s.strip()
    low = t.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("null", "none", "~", ""):
        return None if low != "" else ""
    try:
        return int(t)
    except ValueError:
        pass
    try:
        return float(t)
    except ValueError:
        pass
    if (t.startswith("[") and t.endswith("]")) or (t.startswith("{") and t.endswith("}")):
        try:
            return yaml.safe_load(t)
        except yaml.YAMLError:
            return t
    return t


def substitute(node: Any, env: Mapping[str, str] | None = None) -> Any:
    """Resolve ``${VAR:default}`` in every string of a YAML tree.  A string that is exactly one
    reference is cast to bool / int / float / list; a reference without default whose variable is
    unset raises ``KeyError``."""
    env = os.environ if env is None else env
    if isinstance(node, dict):
        return {k: substitute(v, env) for k, v in node.items()}
    if isinstance(node, list):
        return [substitute(v, env) for v in node]
    if not isinstance(node, str):
        return node

    def repl(m):
        name, default = m.group(1), m.group(2)
        if name in env:
            return env[name]
        if default is None:
            raise KeyError(f"config references ${{{name}}} which is not set and has no default")
        return default

    whole = _VAR.fullmatch(node.strip())
    out = _VAR.sub(repl, node)
    return _cast(out) if whole else out


def deep_merge(base: dict, over: Mapping) -> dict:
    out = copy.deepcopy(base)
    for k, v in over.items():
        if isinstance(v, Mapping) and isinstance(out.get(k), dict):
            out[k] = deep_merge(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


def set_by_path(cfg: dict, dotted: str, value: Any) -> None:
    cur = cfg
    keys = dotted.split(".")
    for k in keys[:-1]:
        cur = cur.setdefault(k, {})
    cur[keys[-1]] = value


def get_by_path(cfg: Mapping, dotted: str, default: Any = None) -> Any:
    cur: Any = cfg
    for k in dotted.split("."):
        if not isinstance(cur, Mapping) or k not in cur:
            return default
        cur = cur[k]
    return cur


def apply_cli_overrides(cfg: dict, overrides: list[str]) -> dict:
    """``["a.b=3", "x=true"]`` -> values set by dotted path (typed like YAML scalars)."""
    for item in overrides:
        if "=" not in item:
            raise ValueError(f"override '{item}' is not key=value")
        k, v = item.split("=", 1)
        set_by_path(cfg, k.strip(), _cast(v))
    return cfg


def load_experiment(path: str | os.PathLike, env: Mapping[str, str] | None = None,
                    overrides: list[str] | None = None, base_dir: str | os.PathLike | None = None) -> dict:
    """Load an experiment YAML.

    Layout (the reference's Primus experiment file): top-level metadata plus
    ``modules.<trainer>.{framework, config, model, overrides}``.  ``config`` and ``model`` name base
    YAML files (looked up next to the experiment, then in ``base_dir``); the module's resolved
    settings are ``base config <- model preset <- overrides``, returned under
    ``modules.<trainer>.resolved``."""
    path = Path(path)
    raw = yaml.safe_load(path.read_text()) or {}
    cfg = substitute(raw, env)
    search = [path.parent] + ([Path(base_dir)] if base_dir else []) + [Path(__file__).parent / "presets"]

    def find(name: str) -> dict:
        for d in search:
            for cand in (d / name, d / "models" / name):
                if cand.exists():
                    return substitute(yaml.safe_load(cand.read_text()) or {}, env)
        return {}

    for name, mod in (cfg.get("modules") or {}).items():
        if not isinstance(mod, dict):
            continue
        resolved: dict = {}
        if isinstance(mod.get("config"), str):
            resolved = deep_merge(resolved, find(mod["config"]))
        if isinstance(mod.get("model"), str):
            resolved = deep_merge(resolved, {"model": find(mod["model"])})
        resolved = deep_merge(resolved, mod.get("overrides") or {})
        mod["resolved"] = resolved
    if overrides:
        apply_cli_overrides(cfg, overrides)
    return cfg


def warn_unknown_keys(exp: dict, run_fn, what: str) -> list:
    """Warn about top-level keys of ``exp`` that ``run_fn`` never looks up (``exp.get("key")`` / ``exp["key"]`` in its
    source): a misspelt key otherwise falls back to its default without a word.  Returns the unknown keys."""
    import inspect
    import re
    import warnings
    src = inspect.getsource(run_fn)
    known = set(re.findall(r'exp\.get\(\s*"(\w+)"', src)) | set(re.findall(r'exp\["(\w+)"\]', src))
    unknown = sorted(k for k in exp if k not in known)
    if unknown:
        warnings.warn(f"{what}: keys without a meaning here are ignored: {unknown}", stacklevel=3)
    return unknown


"""Quiet-stdout mode for timed runs: only ``:::MLLOG`` lines (plus anything matching the allow
patterns) reach the real stdout; everything else is dropped or teed to a side file.

Import-and-call-first module, as the reference's ``_log_suppression``
(small_llm_pretraining/primus/src/_log_suppression.py:33-186): it sets the quiet environment
variables of the libraries underneath, raises Python logger levels, and re-plumbs file descriptor 1
through a pipe with a reader thread that filters lines; file descriptor 2 goes to /dev/null (or the
side file).  ``restore()`` undoes the plumbing (used by tests).
"""
from __future__ import annotations

import logging
import os
import re
import sys
import threading

_ALWAYS = re.compile(r":::MLLOG|^RESULT,|STARTING TIMING RUN|ENDING TIMING RUN")
_state: dict = {}

QUIET_ENV = {
    "NCCL_DEBUG": "WARN", "TORCH_CPP_LOG_LEVEL": "ERROR", "TORCH_DISTRIBUTED_DEBUG": "OFF",
    "PYTHONWARNINGS": "ignore", "TOKENIZERS_PARALLELISM": "false",
}


def install(allow: list[str] | None = None, side_file: str | None = None, verbose_env: str = "B200_VERBOSE") -> bool:
    """Start filtering.  Returns False (and does nothing) when ``$B200_VERBOSE`` is truthy."""
    if os.environ.get(verbose_env, "0") not in ("", "0", "false"):
        return False
    if _state:
        return True
    for k, v in QUIET_ENV.items():
        os.environ.setdefault(k, v)
    logging.getLogger().setLevel(logging.ERROR)
    patterns = [_ALWAYS] + [re.compile(p) for p in (allow or [])]
    sys.stdout.flush()
    sys.stderr.flush()
    real_out = os.dup(1)
    real_err = os.dup(2)
    r, w = os.pipe()
    os.dup2(w, 1)
    os.close(w)
    side = open(side_file, "ab") if side_file else None
    devnull = os.open(os.devnull, os.O_WRONLY)
    os.dup2(side.fileno() if side else devnull, 2)

    def pump():
        with os.fdopen(r, "rb", buffering=0) as src:
            buf = b""
            while True:
                chunk = src.read(65536)
                if not chunk:
                    break
                buf += chunk
                *lines, buf = buf.split(b"\n")
                for ln in lines:
                    text = ln.decode(errors="replace")
                    if any(p.search(text) for p in patterns):
                        os.write(real_out, ln + b"\n")
                    elif side:
                        side.write(ln + b"\n")
            if buf:
                text = buf.decode(errors="replace")
                if any(p.search(text) for p in patterns):
                    os.write(real_out, buf + b"\n")

    t = threading.Thread(target=pump, daemon=True, name="log-filter")
    t.start()
    _state.update(real_out=real_out, real_err=real_err, thread=t, side=side, devnull=devnull)
    return True


def restore() -> None:
    if not _state:
        return
    sys.stdout.flush()
    sys.stderr.flush()
    os.dup2(_state["real_out"], 1)   # closes the pipe's write end held by fd 1 -> reader sees EOF
    os.dup2(_state["real_err"], 2)
    _state["thread"].join(timeout=5)
    os.close(_state["real_out"])
    os.close(_state["real_err"])
    os.close(_state["devnull"])
    if _state["side"]:
        _state["side"].close()
    _state.clear()

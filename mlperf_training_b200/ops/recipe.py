"""Linear-layer precision recipes and their schedule over a run.

The reference trains with micro-scaled low-precision linears and changes the recipe during a run:

* FLUX.1: forward in "A6W4" (MXFP6 activations x MXFP4 weights), switched permanently to FP8 at
  ``FLUX_FPROP_SWITCH_STEP`` while backward stays MXFP4 (flux1/primus/patches/flux_fprop_switch.py:36-308,
  flux1/primus/config_common.sh:71-75,105-123);
* Llama-2-70B LoRA: MXFP4 "healing" - the linears move to FP8 / MXFP8 at ``HEALING_ITER``
  (llama2_sft/primus/src/llama2_custom.py:1295-1893);
* GPT-OSS / FLUX: weight de-oscillation for MXFP4 (start step 768, period 100, ratio 4.0;
  small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:197-204).

This framework implements two low-precision recipe families with different numerics:

* the micro-scaled family - one UE8M0 scale per 32 contraction elements
  (``tcgen05.mma.kind::mxf8f6f4.block_scale``; ``ops.mxfp8``, ``ops.linear.MX_RECIPES``): ``mxfp8`` (e4m3
  elements, the width the benchmark definition names), ``mxfp6`` (e2m3 / e3m2), ``mxfp4`` (e2m1, stochastic
  gradient rounding, Hadamard transform on the weight-gradient operands) and ``a6w4`` (MXFP6 activations x MXFP4
  weights forward, MXFP4 backward).  The narrow members round their operands to the 6- / 4-bit element format
  and carry them as e4m3 codes - every such value is an e4m3 value - so the GEMM result is the narrow
  format's bit for bit, at the 8-bit operand rate (not the 4-bit rate);
* ``fp8``    per-tensor e4m3 forward operands and e5m2 gradients with delayed scaling
  (``tcgen05.mma.kind::f8f6f4``; ``ops.fp8``) - what the reference calls fp8 / hybrid / delayed.

``PrecisionSchedule`` keeps the reference's surface - named phases with a switch step: switching a
phase changes ``precision`` on the model's modules and drops the cached quantised weights, and
because the recipes round differently the losses after the switch differ from those of a run
that did not switch.

``Deoscillator`` is the weight de-oscillation of the 4-bit recipes: a weight whose master value sits near a
rounding boundary of the coarse grid flips between two codes from step to step, which acts as noise on
the forward pass.  Every step it compares each weight's quantised code with the previous step's; at the end of
every ``period`` steps (from ``start_step`` on) a weight that flipped at least ``ratio`` times per grid
step of net movement is declared oscillating and its master value is set to the grid value it currently
rounds to (a direct quantise-dequantise of the master weight), which moves it to the centre of its
rounding interval.  State (previous code, code at the period start, flip count) is kept per element of
the rank's optimizer shard.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch

from .linear import bump_weight_epoch

# reference recipe names -> precision implemented here
FORMAT_MAP = {
    "bf16": "bf16", "none": "bf16",
    "mxfp8": "mxfp8", "mxfp6": "mxfp6", "mxfp4": "mxfp4", "e2m1": "mxfp4", "nvfp4": "mxfp4", "a4w4": "mxfp4", "a6w4": "a6w4",
    "mxfp8_fwd_mxfp4_bwd": "mxfp8_fwd_mxfp4_bwd", "fp8_fwd_mxfp4_bwd": "mxfp8_fwd_mxfp4_bwd",
    "fp8": "fp8", "fp8_hybrid": "fp8", "hybrid": "fp8", "e4m3": "fp8", "delayed": "fp8", "tensorwise": "fp8",
}


def resolve_format(name: str) -> str:
    key = str(name).strip().lower()
    if key not in FORMAT_MAP:
        raise ValueError(f"unknown linear precision '{name}' (known: {sorted(FORMAT_MAP)})")
    return FORMAT_MAP[key]


@dataclass
class DeoscConfig:
    enabled: bool = False
    start_step: int = 768
    period: int = 100
    ratio: float = 4.0

    def status(self, precision: str) -> str:
        if not self.enabled:
            return "deosc: off"
        from .linear import MX_RECIPES
        fmt = MX_RECIPES.get(precision, ("", "e4m3"))[1]
        if fmt != "e2m1":
            return (f"deosc: requested (start {self.start_step}, period {self.period}, ratio {self.ratio}) - idle: "
                    f"weights are {precision} ({fmt} elements), the oscillation it damps is a 4-bit-weight effect")
        return f"deosc: on (start {self.start_step}, period {self.period}, ratio {self.ratio})"


class Deoscillator:
    """Tracks code flips of the 4-bit-quantised weights of ``engine``'s parameters and snaps oscillating master
    weights to their grid value (see the module docstring).  ``after_step(step, precision)`` is called once per
    optimizer step; it does nothing unless the active recipe quantises weights to e2m1."""

    def __init__(self, engine, cfg: DeoscConfig, fmt: str = "e2m1"):
        self.engine, self.cfg, self.fmt = engine, cfg, fmt
        self.state: dict = {}
        self.snapped = 0                     # weights snapped so far (this rank's shards)
        self.history: list = []              # (step, snapped at that period end)
        self._grid = None

    def _keys(self, b):
        """Per element of this rank's shard of bucket ``b``: (tracked?, scale-and-code key, code, grid value)."""
        from . import mxfp8 as MX
        dev = b.param_buf.device
        n = b.hi - b.lo
        tracked = torch.zeros(n, dtype=torch.bool, device=dev)
        key = torch.zeros(n, dtype=torch.int32, device=dev)
        code = torch.zeros(n, dtype=torch.int32, device=dev)
        value = torch.zeros(n, dtype=torch.float32, device=dev)
        if self._grid is None or self._grid.device != dev:
            pos = MX.round_to_format(torch.linspace(0.0, MX.ELEMENT_FORMATS[self.fmt][2], 4097), self.fmt).unique()
            self._grid = torch.cat([-pos.flip(0)[:-1], pos]).to(dev)
        v_max = MX.ELEMENT_FORMATS[self.fmt][2]
        for (name, p), o in zip(b.params, b.offsets):
            # only matrices that a micro-scaled linear, or stacks of them that the grouped expert MLP, has quantised
            seen = getattr(p, "_mx_cache", None) is not None if p.dim() == 2 else getattr(p, "_mx_stack", None) is not None
            if p.dim() not in (2, 3) or p.shape[-1] % 32 or not seen:
                continue
            lo, hi = max(o, b.lo), min(o + p.numel(), b.hi)
            if lo >= hi:
                continue
            w = p.detach().float().reshape(-1, p.shape[-1] // 32, 32)
            sf = MX._e8m0(w.abs().amax(-1), v_max)
            scale = torch.exp2(sf.float() - 127.0)[..., None]
            r = MX.round_to_format(w / scale, self.fmt)
            c = torch.bucketize(r, self._grid).to(torch.int32)
            k = sf.to(torch.int32)[..., None] * 64 + c
            sl = slice(lo - b.lo, hi - b.lo)
            src = slice(lo - o, hi - o)
            tracked[sl] = True
            key[sl] = k.reshape(-1)[src]
            code[sl] = c.reshape(-1)[src]
            value[sl] = (r * scale).reshape(-1)[src]
        return tracked, key, code, value

    def state_dict(self) -> dict:
        """Per-bucket flip state (in bucket order), for this rank's optimizer-shard checkpoint."""
        per = []
        for b in self.engine.buckets:
            st = self.state.get(id(b))
            per.append(None if st is None else {k: v.detach().cpu() for k, v in st.items()})
        return {"buckets": per, "snapped": self.snapped, "history": list(self.history)}

    def load_state_dict(self, sd: dict) -> None:
        self.snapped, self.history = int(sd.get("snapped", 0)), [tuple(h) for h in sd.get("history", [])]
        for b, st in zip(self.engine.buckets, sd.get("buckets", [])):
            if st is not None:
                self.state[id(b)] = {k: v.to(b.param_buf.device) for k, v in st.items()}

    def after_step(self, step: int, precision: str) -> int:
        """Returns the number of weights snapped at this step (non-zero only at a period end)."""
        from .linear import MX_RECIPES
        cfg = self.cfg
        if not cfg.enabled or step < cfg.start_step or MX_RECIPES.get(precision, ("", ""))[1] != self.fmt:
            return 0
        period_end = (step - cfg.start_step + 1) % max(cfg.period, 1) == 0
        n_snapped = 0
        with torch.no_grad():
            for b in self.engine.buckets:
                tracked, key, code, value = self._keys(b)
                if not bool(tracked.any()):
                    continue
                st = self.state.get(id(b))
                if st is None:
                    st = self.state[id(b)] = {"prev": key.clone(), "start_key": key.clone(), "start_code": code.clone(),
                                              "flips": torch.zeros_like(key, dtype=torch.int16)}
                else:
                    st["flips"] += (key != st["prev"]).to(torch.int16)
                    st["prev"] = key
                if not period_end:
                    continue
                same_scale = (key // 64) == (st["start_key"] // 64)
                moved = torch.where(same_scale, (code - st["start_code"]).abs(), torch.full_like(code, 64))
                osc = tracked & (st["flips"].to(torch.float32) >= cfg.ratio * (1 + moved).to(torch.float32))
                k = int(osc.sum())
                if k:
                    shard = b.p_shard()
                    shard[osc] = value[osc].to(shard.dtype)
                    if b.master is not None:
                        b.master[osc] = value[osc]
                n_snapped += k
                st["start_key"], st["start_code"] = key.clone(), code.clone()
                st["flips"].zero_()
        if period_end:
            # every rank's shard of every touched bucket goes back to all replicas (the call is collective: ranks
            # agree on "touched" through the reduced count)
            total = torch.tensor([n_snapped], dtype=torch.int64, device=self.engine.device)
            if self.engine.world > 1:
                import torch.distributed as dist
                dist.all_reduce(total, group=self.engine.group)
                if int(total) > 0:
                    for b in self.engine.buckets:
                        if id(b) in self.state and not getattr(b, "local_only", False):
                            self.engine._all_gather(b)
            if int(total) > 0:
                bump_weight_epoch()
            self.snapped += n_snapped
            self.history.append((step, n_snapped))
        return n_snapped


@dataclass
class PrecisionSchedule:
    """``phases``: ``[(first_step, format_name), ...]`` sorted by step; the last phase whose first
    step is <= the current step is active."""
    phases: list = field(default_factory=lambda: [(0, "mxfp8")])
    deosc: DeoscConfig = field(default_factory=DeoscConfig)
    _active: str | None = None
    log: list = field(default_factory=list)

    @staticmethod
    def from_spec(spec) -> "PrecisionSchedule":
        """``spec``: a format name, or ``{"initial": "a6w4", "switch_step": 400, "final": "fp8",
        "deosc": {...}}``; the environment (``FLUX_FPROP_SWITCH_STEP``, ``HEALING_ITER``) overrides
        the switch step when set."""
        if spec is None or isinstance(spec, str):
            return PrecisionSchedule([(0, spec or "mxfp8")])
        phases = [(0, spec.get("initial", "mxfp8"))]
        sw = spec.get("switch_step")
        for var in ("FLUX_FPROP_SWITCH_STEP", "HEALING_ITER"):
            if os.environ.get(var):
                sw = int(os.environ[var])
        if sw is not None and int(sw) > 0 and spec.get("final"):
            phases.append((int(sw), spec["final"]))
        return PrecisionSchedule(phases, DeoscConfig(**(spec.get("deosc") or {})))

    def at(self, step: int) -> str:
        name = self.phases[0][1]
        for first, fmt in self.phases:
            if step >= first:
                name = fmt
        return resolve_format(name)

    def apply(self, model, step: int) -> bool:
        """Set the precision of ``step`` on every module / config that carries one.  Returns True when
        it changed (cached quantised weights are dropped then)."""
        want = self.at(step)
        if want == self._active:
            return False
        cfg = getattr(model, "cfg", None)
        if cfg is not None and hasattr(cfg, "precision"):
            cfg.precision = want
        for m in model.modules():
            if hasattr(m, "precision") and isinstance(getattr(m, "precision"), str):
                m.precision = want
        bump_weight_epoch()
        self.log.append((step, want))
        self._active = want
        return True

"""Linear-layer precision recipes and their schedule over a run.

The reference trains with micro-scaled low-precision linears and changes the recipe during a run:

* FLUX.1: forward in "A6W4" (MXFP6 activations x MXFP4 weights), switched permanently to FP8 at
  ``FLUX_FPROP_SWITCH_STEP`` while backward stays MXFP4 (flux1/primus/patches/flux_fprop_switch.py:36-308,
  flux1/primus/config_common.sh:71-75,105-123);
* Llama-2-70B LoRA: MXFP4 "healing" - the linears move to FP8 / MXFP8 at ``HEALING_ITER``
  (llama2_sft/primus/src/llama2_custom.py:1295-1893);
* GPT-OSS / FLUX: weight de-oscillation for MXFP4 (start step 768, period 100, ratio 4.0;
  small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:197-204).

This framework implements two low-precision recipes with different numerics:

* ``mxfp8``  e4m3 codes with one UE8M0 scale per 32 contraction elements
  (``tcgen05.mma.kind::mxf8f6f4.block_scale``; ``ops.mxfp8``) - the micro-scaled family; the
  reference's 4- and 6-bit micro-scaled names (mxfp4, a6w4, ...) select it, as the widest member
  this hardware path offers and the one the benchmark definition names;
* ``fp8``    per-tensor e4m3 forward operands and e5m2 gradients with delayed scaling
  (``tcgen05.mma.kind::f8f6f4``; ``ops.fp8``) - what the reference calls fp8 / hybrid / delayed.

``PrecisionSchedule`` keeps the reference's surface - named phases with a switch step: switching a
phase changes ``precision`` on the model's modules and drops the cached quantised weights, and
because the two recipes round differently the losses after the switch differ from those of a run
that did not switch.  De-oscillation is accepted, recorded, and reported as inactive with its
reason: it repairs a 4-bit-weight artefact that e4m3 weights do not show.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

from .linear import bump_weight_epoch

# reference recipe names -> precision implemented here
FORMAT_MAP = {
    "bf16": "bf16", "none": "bf16",
    "mxfp8": "mxfp8", "mxfp4": "mxfp8", "e2m1": "mxfp8", "nvfp4": "mxfp8", "a6w4": "mxfp8", "mxfp6": "mxfp8",
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
        return (f"deosc: requested (start {self.start_step}, period {self.period}, ratio {self.ratio}) - inactive: "
                f"weights are {precision} (8-bit mantissa/exponent codes), the oscillation it damps is a 4-bit effect")


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

"""LoRA supervised fine-tuning run (Llama-2-70B LoRA workload).

The run loop is ``trainer.loop.run``; this module fixes what makes a run an SFT run and is the
target of ``cli posttrain``:

* the base model is frozen and only the LoRA adapters (rank 16, alpha 32, dropout 0.1 on the fused
  QKV and the output projection) are trained and sharded by the engine
  (llama2_sft/primus/src/llama2_custom.py:596-610);
* batches are packed fine-tuning samples ``(tokens, labels)`` with -100 where ``loss_mask`` is 0, or
  synthetic tokens with the loss on the last ``loss_last`` positions;
* evaluation starts after ``skip_evals`` intervals, averages over labelled tokens, and the run stops
  at ``target_eval_loss`` (0.925) (llama2_custom.py:752-915, 919-1028);
* tensor + sequence parallel size ``tensor_parallel`` with the fused all-gather->GEMM and
  GEMM->reduce-scatter kernels (``tp_comm_overlap: fused``) or NCCL collectives (``nccl``);
* the base weights come from a Megatron ``torch_dist`` checkpoint when ``pretrained_checkpoint`` is
  set (``finetune=True``: no optimizer state, no RNG state; llama2_custom.py:711-725).
"""
from __future__ import annotations

from .loop import run as _run

SFT_DEFAULTS = {
    "benchmark": "llama2_70b_lora",
    "lr": 6.0e-4, "weight_decay": 1.0e-4, "adam_beta1": 0.9, "adam_beta2": 0.999, "adam_eps": 1e-8,
    "clip_grad": 0.3, "lr_warmup_iters": 0, "min_lr_ratio": 0.0,
    "eval_interval": 48, "eval_iters": 24, "skip_evals": 3, "target_eval_loss": 0.925,
    "warmup_train_steps": 2, "warmup_eval_steps": 1,
}


def run(exp: dict, device: str | None = None, stream=None) -> dict:
    merged = dict(SFT_DEFAULTS)
    merged.update(exp or {})
    model = dict(merged.get("model") or {})
    model.setdefault("lora_rank", 16)
    model.setdefault("lora_alpha", 32.0)
    model.setdefault("lora_dropout", 0.1)
    merged["model"] = model
    return _run(merged, device=device, stream=stream)

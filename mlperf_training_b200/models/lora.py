"""LoRA adapters over frozen base linears: ``y = W x + (alpha / r) * B A dropout(x)``.

Rank 16, alpha 32, dropout 0.1 applied before the adapter, ``A`` Xavier-uniform and ``B`` zero, on
the fused QKV and output projections - the adapter configuration of the reference's SFT recipe
(llama2_sft/primus/src/llama2_custom.py:596-610).  ``freeze_base`` marks every non-adapter
parameter as frozen so the engine only shards / updates adapter state and the wgrad GEMMs of the
base weights are skipped; with ``precision="mxfp8"`` the frozen weights are quantised once and the
copies are kept for the whole run (the reference pre-quantises its frozen base the same way,
llama2_custom.py:1904-1910).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F


class LoRAAdapter(nn.Module):
    def __init__(self, n_in: int, n_out: int, rank: int, alpha: float, dropout: float, dtype, device):
        super().__init__()
        self.a = nn.Parameter(torch.empty(rank, n_in, dtype=dtype, device=device))
        self.b = nn.Parameter(torch.zeros(n_out, rank, dtype=dtype, device=device))
        bound = math.sqrt(6.0 / (n_in + rank))
        with torch.no_grad():
            self.a.uniform_(-bound, bound)
        self.scale = alpha / rank
        self.dropout = dropout

    def drop(self, x):
        return TF.dropout(x, self.dropout) if (self.dropout > 0 and self.training) else x

    def down(self, x):
        """``dropout(x) A^T`` ``[T, rank]``: on the tcgen05 GEMM (a skinny-N tile) for CUDA bf16 rows."""
        return _mm(self.drop(x), self.a)

    def up(self, u):
        """``scale * u B^T`` ``[T, n_out]``."""
        return _mm(u * self.scale, self.b)

    def forward(self, x):
        return self.up(self.down(x))


def _mm(x, w):
    """``x W^T`` through the package's GEMM (forward, dgrad and wgrad) when the operands allow it
    (2-D, inner dimensions multiples of 8 elements = 16 bytes), else a plain matmul."""
    if x.dim() == 2 and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and x.dtype == w.dtype:
        return F.linear(x, w)
    return x @ w.t()


def freeze_base(model: nn.Module) -> list[str]:
    """Freeze everything except LoRA adapters.  Returns the names left trainable."""
    trainable = []
    for name, p in model.named_parameters():
        p.requires_grad_("lora" in name)
        if p.requires_grad:
            trainable.append(name)
    return trainable


def merge_adapters(model: nn.Module) -> None:
    """Fold the adapters into the base weights (for export): ``W += scale * B A``."""
    with torch.no_grad():
        for blk in getattr(model, "blocks", []):
            for adapter, weight in ((blk.lora_qkv, blk.w_qkv), (blk.lora_proj, blk.w_proj)):
                if adapter is not None:
                    weight.add_((adapter.b.float() @ adapter.a.float() * adapter.scale).to(weight.dtype))
                    adapter.b.zero_()

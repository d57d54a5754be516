"""Mixture-of-experts MLP of the GPT-OSS architecture: fp32 router GEMM, top-k with softmax over
the selected logits, SwiGLU experts, no auxiliary loss, no token dropping; optional expert
parallelism (experts sharded over an ``ep_group``, token all-to-all dispatch / combine).

Reference configuration: small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:115-120,130-167,205-222
(``moe_token_dispatcher_type: alltoall``, grouped GEMM, permute fusion, identity-sort skip at EP=1).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as F
from ..ops import moe_ops as M
from ..parallel.expert import ExpertParallelDispatcher, FusedExpertDispatcher


class MoEMLP(nn.Module):
    def __init__(self, cfg, dtype, device, ep_group=None, ep_comm: str = "nccl"):
        super().__init__()
        self.cfg = cfg
        d, f, E = cfg.hidden, cfg.moe_ffn_hidden, cfg.n_experts
        self.ep_group = ep_group
        self.ep = dist.get_world_size(ep_group) if ep_group is not None else 1
        self.ep_rank = dist.get_rank(ep_group) if ep_group is not None else 0
        if E % self.ep:
            raise ValueError(f"{E} experts do not divide over expert-parallel size {self.ep}")
        self.local_experts = E // self.ep
        self.router = nn.Parameter(torch.empty(E, d, dtype=torch.float32, device=device))
        self.w1 = nn.Parameter(torch.empty(self.local_experts, 2 * f, d, dtype=dtype, device=device))
        self.w2 = nn.Parameter(torch.empty(self.local_experts, d, f, dtype=dtype, device=device))
        # expert weights belong to this expert-parallel rank only: data-parallel reductions of their
        # gradients run over the ranks that hold the same experts
        self.w1.expert_parallel = self.w2.expert_parallel = self.ep > 1
        if self.ep > 1:
            # (expert-parallel size, this rank's index): which block of the stacked expert dimension this rank holds
            self.w1.expert_shard = self.w2.expert_shard = (self.ep, self.ep_rank)
        self.dispatcher = ExpertParallelDispatcher(ep_group, E) if self.ep > 1 else None
        self.ep_comm = ep_comm
        self._fused = None      # built on first use: its slab size depends on the number of tokens per step

    def forward(self, h, norm_w, eps):
        cfg = self.cfg
        hn = F.rms_norm(h, norm_w, eps)
        logits = F.router_logits(hn, self.router)          # fp32 logits on the tcgen05 GEMM (split-precision weight)
        idx, w, counts = M.RouterFn.apply(logits, cfg.top_k)
        prec = M.expert_precision(getattr(cfg, "precision", "bf16"), self.w1, self.w2)
        if self.dispatcher is None:
            y = M.moe_experts(hn, idx, w, counts, self.w1, self.w2, prec)
        elif self.ep_comm == "fused" and hn.is_cuda and hn.dtype == torch.bfloat16:
            y = self._fused_dispatcher(hn.shape[0] * cfg.top_k, hn.device, M.pad_rows(prec))(hn, idx, w, counts, self.w1,
                                                                                             self.w2, prec)
        else:
            y = self.dispatcher(hn, idx, w, counts, self.w1, self.w2, prec)
        return h + y

    _shared: dict = {}

    def _fused_dispatcher(self, pairs: int, device, pad: int = M.PAD):
        """Every layer owns its input slab (it is read again in backward); the output and gradient
        slabs of all layers of one (group, shape) are the same buffers."""
        if self._fused is None or self._fused_pairs != (pairs, pad):
            key = (id(self.ep_group), self.cfg.n_experts, self.cfg.hidden, pairs, pad, str(device))
            first = MoEMLP._shared.get(key)
            self._fused = FusedExpertDispatcher(self.ep_group, self.cfg.n_experts, self.cfg.hidden, pairs, device,
                                                share_with=first, pad=pad)
            self._fused_pairs = (pairs, pad)
            if first is None:
                MoEMLP._shared[key] = self._fused
        return self._fused

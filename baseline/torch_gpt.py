"""Library baseline of the GPT pre-training step: the same architecture and step structure as
``mlperf_training_b200.trainer.pretrain.PretrainTrainer`` built only from stock PyTorch pieces -
``F.linear`` (cuBLAS), ``scaled_dot_product_attention``, ``F.rms_norm``, ``F.cross_entropy``,
``torch.optim.AdamW(fused=True)``, ``DistributedDataParallel`` over NCCL.  None of the package's
kernels, models or engine is on this path.  Used by ``bench.py --impl baseline``.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class _Block(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        d, hd = cfg.hidden, cfg.head_dim
        self.cfg = cfg
        self.n1 = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.n2 = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.qkv = nn.Linear(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd, bias=False, dtype=dtype, device=device)
        self.proj = nn.Linear(cfg.n_heads * hd, d, bias=False, dtype=dtype, device=device)
        self.gate_up = nn.Linear(d, 2 * cfg.ffn_hidden, bias=False, dtype=dtype, device=device)
        self.down = nn.Linear(cfg.ffn_hidden, d, bias=False, dtype=dtype, device=device)

    def forward(self, x, cos, sin):
        cfg = self.cfg
        B, S, _ = x.shape
        Hq, Hkv, D = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        qkv = self.qkv(F.rms_norm(x, (cfg.hidden,), self.n1, cfg.norm_eps))
        q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        q = q.view(B, S, Hq, D)
        k = k.view(B, S, Hkv, D)
        v = v.view(B, S, Hkv, D)

        def rope(t):
            t1, t2 = t[..., :D // 2], t[..., D // 2:]
            c, s = cos[None, :S, None, :], sin[None, :S, None, :]
            return torch.cat([t1 * c - t2 * s, t2 * c + t1 * s], dim=-1).to(t.dtype)

        q, k = rope(q), rope(k)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=True).transpose(1, 2).reshape(B, S, Hq * D)
        h = x + self.proj(o)
        gu = self.gate_up(F.rms_norm(h, (cfg.hidden,), self.n2, cfg.norm_eps))
        g, u = gu.chunk(2, dim=-1)
        return h + self.down(F.silu(g) * u)


class _GPT(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([_Block(cfg, dtype, device) for _ in range(cfg.n_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden, dtype=dtype, device=device))
        self.head = nn.Linear(cfg.hidden, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float64) / cfg.head_dim))
        ang = torch.outer(torch.arange(cfg.seq_len, dtype=torch.float64), inv)
        self.register_buffer("cos", ang.cos().float().to(device), persistent=False)
        self.register_buffer("sin", ang.sin().float().to(device), persistent=False)
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, 0.0, cfg.init_std)

    def forward(self, tokens, labels):
        x = self.embed(tokens)
        for b in self.blocks:
            x = b(x, self.cos, self.sin)
        logits = self.head(F.rms_norm(x, (self.cfg.hidden,), self.norm, self.cfg.norm_eps))
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1))


class BaselineTrainer:
    def __init__(self, cfg, opt, train, device):
        self.cfg, self.train_cfg, self.device = cfg, train, torch.device(device)
        torch.manual_seed(train.seed)
        self.model = _GPT(cfg, torch.bfloat16, self.device)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.ddp = nn.parallel.DistributedDataParallel(self.model, device_ids=[self.device.index]) \
            if self.world > 1 else self.model
        decay = [p for n, p in self.model.named_parameters() if p.dim() >= 2]
        nodecay = [p for n, p in self.model.named_parameters() if p.dim() < 2]
        self.optim = torch.optim.AdamW([{"params": decay, "weight_decay": opt.weight_decay},
                                        {"params": nodecay, "weight_decay": 0.0}], lr=opt.lr,
                                       betas=(opt.beta1, opt.beta2), eps=opt.eps, fused=True)
        self.clip = opt.clip_grad
        self.n_micro = train.local_batch // train.micro_batch
        self._staging = None

    def train_step_device(self, tokens):
        mb = self.train_cfg.micro_batch
        total = None
        for i in range(self.n_micro):
            chunk = tokens[i * mb:(i + 1) * mb]
            sync = (i == self.n_micro - 1) or self.world == 1
            ctx = torch.enable_grad() if sync or self.world == 1 else self.ddp.no_sync()
            with ctx:
                loss = self.ddp(chunk[:, :-1], chunk[:, 1:]) / self.n_micro
                loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if self.clip > 0:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip, foreach=True)
        self.optim.step()
        self.optim.zero_grad(set_to_none=True)
        return total

    def train_step(self, batch):
        if self._staging is None or self._staging.shape != batch.shape:
            self._staging = torch.empty(batch.shape, dtype=torch.int64, device=self.device)
        self._staging.copy_(batch, non_blocking=True)
        return float(self.train_step_device(self._staging).item())

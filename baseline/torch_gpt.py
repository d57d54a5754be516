"""Library baseline of the GPT pre-training step: the same architecture and step structure as
``mlperf_training_b200.trainer.pretrain.PretrainTrainer`` built only from stock PyTorch pieces -
``F.linear`` (cuBLAS), ``scaled_dot_product_attention``, ``F.rms_norm``, ``F.cross_entropy``,
``torch.optim.AdamW(fused=True)``, ``DistributedDataParallel`` or FSDP2 ``fully_shard`` over NCCL.
None of the package's kernels, models or engine is on this path.  Used by ``bench.py --impl baseline``
and by the stock arms that ``bench.py`` times next to its own arm.

``precision="mxfp8"`` gives the equal-precision arm: every block linear runs its three GEMMs
(forward, dgrad, wgrad) through ``torch._scaled_mm`` with e4m3 codes and UE8M0 scales per 32
contraction elements (the cuBLASLt block-scaled GEMM), the operands quantised by plain torch ops
(compiled with ``torch.compile`` when that works on the box, eager otherwise).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _to_mx(x: torch.Tensor):
    """bf16 ``[R, K]`` -> (e4m3 codes ``[R, K]``, UE8M0 scales in the 128 x 4 blocked layout cuBLASLt reads)."""
    R, K = x.shape
    xb = x.float().view(R, K // 32, 32)
    amax = xb.abs().amax(-1)
    e = torch.ceil(torch.log2(amax.clamp_min(2.0 ** -120) / 448.0)).clamp(-127, 127)
    q = (xb * torch.exp2(-e)[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(R, K)
    sf = (e + 127).to(torch.uint8)
    rb, cb = (R + 127) // 128, (K // 32 + 3) // 4
    if rb * 128 != R or cb * 4 != K // 32:
        sf = F.pad(sf, (0, cb * 4 - K // 32, 0, rb * 128 - R))
    sf = sf.view(rb, 128, cb, 4).permute(0, 2, 1, 3).reshape(-1, 4, 32, 4).transpose(1, 2).reshape(-1)
    return q, sf.contiguous().view(torch.float8_e8m0fnu)


_to_mx_impl = None


def to_mx(x):
    global _to_mx_impl
    if _to_mx_impl is None:
        try:
            import torch._dynamo
            torch._dynamo.config.cache_size_limit = max(torch._dynamo.config.cache_size_limit, 128)   # one graph per operand shape
            fn = torch.compile(_to_mx, dynamic=False)
            fn(torch.zeros(128, 128, dtype=torch.bfloat16, device=x.device))
            _to_mx_impl = fn
        except Exception:                      # no working inductor / triton on this box: eager ops
            _to_mx_impl = _to_mx
    return _to_mx_impl(x)


def _mx_mm(a, b):
    """``a [M, K] @ b [N, K]^T`` through the library's block-scaled GEMM, bf16 result; ``a`` / ``b`` are
    bf16 matrices or already quantised ``(codes, scales)`` pairs."""
    qa, sa = a if isinstance(a, tuple) else to_mx(a)
    qb, sb = b if isinstance(b, tuple) else to_mx(b)
    return torch._scaled_mm(qa, qb.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)


def _weight_mx(w, transposed: bool):
    """Quantised copy of a weight (or of its transpose), kept until the optimizer changes the weight."""
    key = "_mx_t" if transposed else "_mx"
    hit = getattr(w, key, None)
    if hit is not None and hit[0] == w._version:
        return hit[1]
    op = to_mx(w.detach().t().contiguous() if transposed else w.detach())
    setattr(w, key, (w._version, op))
    return op


class _MXLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return _mx_mm(x.reshape(-1, x.shape[-1]), _weight_mx(w, False)).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        x2, dy2 = x.reshape(-1, x.shape[-1]), dy.reshape(-1, dy.shape[-1])
        dx = _mx_mm(dy2, _weight_mx(w, True)).view_as(x)         # contraction over the output features
        dw = _mx_mm(dy2.t().contiguous(), x2.t().contiguous())   # contraction over the tokens
        return dx, dw


class _Linear(nn.Linear):
    mx = False

    def forward(self, x):
        if self.mx:
            return _MXLinearFn.apply(x, self.weight)
        return F.linear(x, self.weight)


class _Block(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        d, hd = cfg.hidden, cfg.head_dim
        self.cfg = cfg
        self.n1 = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.n2 = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.qkv = _Linear(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd, bias=False, dtype=dtype, device=device)
        self.proj = _Linear(cfg.n_heads * hd, d, bias=False, dtype=dtype, device=device)
        self.gate_up = _Linear(d, 2 * cfg.ffn_hidden, bias=False, dtype=dtype, device=device)
        self.down = _Linear(cfg.ffn_hidden, d, bias=False, dtype=dtype, device=device)
        for lin in (self.qkv, self.proj, self.gate_up, self.down):
            lin.mx = getattr(cfg, "precision", "bf16") == "mxfp8"

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
        self.head = _Linear(cfg.hidden, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        self.head.mx = getattr(cfg, "precision", "bf16") == "mxfp8" and cfg.vocab_size % 128 == 0
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
    """``parallel``: "ddp" (replicated parameters) or "fsdp" (FSDP2 ``fully_shard`` per block, ZeRO-3)."""

    def __init__(self, cfg, opt, train, device, parallel: str = "ddp"):
        self.cfg, self.train_cfg, self.device = cfg, train, torch.device(device)
        torch.manual_seed(train.seed)
        self.model = _GPT(cfg, torch.bfloat16, self.device)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.parallel = parallel if self.world > 1 else "none"
        if self.parallel == "fsdp":
            from torch.distributed.fsdp import fully_shard
            for blk in self.model.blocks:
                fully_shard(blk)
            fully_shard(self.model)
            self.ddp = self.model
        elif self.parallel == "ddp":
            self.ddp = nn.parallel.DistributedDataParallel(self.model, device_ids=[self.device.index])
        else:
            self.ddp = self.model
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
            if self.parallel == "fsdp":
                self.model.set_requires_gradient_sync(sync)
            ctx = self.ddp.no_sync() if (self.parallel == "ddp" and not sync) else torch.enable_grad()
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

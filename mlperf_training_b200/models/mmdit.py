"""FLUX.1-schnell-architecture MMDiT (multimodal diffusion transformer) with the rectified-flow
training objective.

19 double-stream blocks (separate image / text weights, joint attention over the concatenated
512 tokens) and 38 single-stream blocks (fused QKV+MLP projection), hidden 3072, 24 heads of 128,
multi-axis rotary embedding (16 + 56 + 56 frequency pairs over (index, row, column)), AdaLN
modulation from the timestep and pooled-text vector, per-head RMS q/k norm, tanh-GELU MLPs; no
guidance embedding (schnell).  Inputs are pre-encoded: 16-channel 32x32 latents patchified 2x2 into
256 tokens of 64, 256 T5 tokens of 4096, a 768-d pooled CLIP vector.

The reference trains this model through the Primus diffusion backend
(flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml, flux1/primus/README.md:66-67) with fused
norm+RoPE, fused dGELU MLP and gate fusions (flux1/primus/config_common.sh:84-150).  Here every
GEMM, LayerNorm / RMSNorm, GELU and the joint attention run on this package's sm_100a kernels; the
per-sample modulate / gate arithmetic is plain tensor algebra on ``[B, S, D]`` views.

Rotary convention: rotate-half pairs ``(i, i + 64)`` instead of FLUX's interleaved pairs - the same
rotation group, a fixed permutation of head channels, immaterial for training from random init.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import kernels as K


@dataclass
class MMDiTConfig:
    name: str = "mmdit"
    n_double: int = 19
    n_single: int = 38
    hidden: int = 3072
    n_heads: int = 24
    head_dim: int = 128
    mlp_ratio: float = 4.0
    in_channels: int = 64          # 16 latent channels x 2 x 2 patch
    txt_dim: int = 4096
    vec_dim: int = 768
    img_size: int = 256
    txt_tokens: int = 256
    axes_dim: tuple = (16, 56, 56)
    rope_theta: float = 10000.0
    dtype: str = "bf16"
    precision: str = "bf16"
    # activation recompute: "full" runs the first ``recompute_ratio`` of the double and of the single blocks
    # again in backward and keeps only their inputs (gradient checkpointing ratio 1.0 in
    # flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:62-70)
    recompute: str = "none"
    recompute_ratio: float = 1.0

    @property
    def img_tokens(self) -> int:
        return (self.img_size // 16) ** 2     # VAE /8, patch /2

    @property
    def mlp_hidden(self) -> int:
        return int(self.hidden * self.mlp_ratio)

    def torch_dtype(self):
        return {"bf16": torch.bfloat16, "fp32": torch.float32}[self.dtype]

    def to_dict(self):
        return asdict(self)

    def flops_per_sample(self) -> float:
        d, m, S = self.hidden, self.mlp_hidden, self.img_tokens + self.txt_tokens
        double = 2 * (4 * d * d + 2 * d * m)                       # per token per stream: qkv+proj, mlp
        single = 2 * (3 * d * d + d * m + (d + m) * d)
        gemm = S * (self.n_double * double + self.n_single * single)
        attn = (self.n_double + self.n_single) * 4 * S * S * d
        return 3.0 * gemm + 3.5 * attn


def flux1_schnell(**over) -> MMDiTConfig:
    return MMDiTConfig(name="flux1-schnell", **over)


def tiny_mmdit(**over) -> MMDiTConfig:
    base = dict(name="tiny-mmdit", n_double=1, n_single=2, hidden=128, n_heads=2, head_dim=64, in_channels=16,
                txt_dim=64, vec_dim=32, img_size=64, txt_tokens=16, axes_dim=(8, 28, 28), dtype="fp32")
    base.update(over)
    return MMDiTConfig(**base)


PRESETS = {"flux1-schnell": flux1_schnell, "tiny-mmdit": tiny_mmdit}


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0, factor: float = 1000.0):
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = (t.float() * factor)[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def rope_tables_nd(ids: torch.Tensor, axes_dim, theta: float):
    """cos / sin ``[S, head_dim / 2]`` for position ids ``[S, n_axes]``: axis ``a`` owns
    ``axes_dim[a] / 2`` consecutive frequency pairs."""
    cos, sin = [], []
    for a, d in enumerate(axes_dim):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        ang = ids[:, a].double()[:, None] * inv[None]
        cos.append(ang.cos())
        sin.append(ang.sin())
    return torch.cat(cos, -1).float(), torch.cat(sin, -1).float()


class Linear(nn.Module):
    def __init__(self, n_in, n_out, dtype, device, bias=True, std=0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_out, n_in, dtype=dtype, device=device).normal_(0, std))
        self.bias = nn.Parameter(torch.zeros(n_out, dtype=dtype, device=device)) if bias else None

    def forward(self, x, precision="bf16", residual=None):
        return F.linear(x, self.weight, self.bias, residual, precision)


class QKNorm(nn.Module):
    """Per-head RMS norm of queries and keys with learned scales."""

    def __init__(self, hd, dtype, device):
        super().__init__()
        self.q_scale = nn.Parameter(torch.ones(hd, dtype=dtype, device=device))
        self.k_scale = nn.Parameter(torch.ones(hd, dtype=dtype, device=device))

    def forward(self, q, k):
        shp = q.shape
        q = F.rms_norm(q.reshape(-1, shp[-1]), self.q_scale, 1e-6).view(shp)
        k = F.rms_norm(k.reshape(-1, shp[-1]), self.k_scale, 1e-6).view(shp)
        return q, k


def _ln(x2d):
    return F.layer_norm(x2d, None, None, 1e-6)


def _ln_modulate(x2d, shift, scale, B):
    """LayerNorm(x) * (1 + scale[b]) + shift[b] for the tokens of sample b: one fused kernel each way."""
    return F.ln_modulate(x2d, shift, scale, B, 1e-6)


def _gate(res2d, y2d, gate, B):
    """res + y * gate[b]: one fused kernel forward, the per-sample gate gradient reduced by a kernel."""
    return F.gate_residual(res2d, y2d, gate, B)


def _rope(x, cos, sin):
    """x ``[B, S, H, D]`` rotate-half with the n-D position tables ``[S, D/2]`` (rotary kernel)."""
    return F.rope_bshd(x, cos, sin)


def _attention(q, k, v, sp):
    """Joint (non-causal) attention; with ``sp = (group, ...)`` the tokens are sharded over the group and
    the sequence shards are traded for head shards around the kernel (Ulysses).  Non-causal attention does
    not care in which order the exchange lines the chunks up, as long as q, k and v agree - and they do."""
    if sp is None:
        return F.attention(q, k, v, causal=False)
    from ..parallel.context import ulysses_attention
    return ulysses_attention(q.contiguous(), k.contiguous(), v.contiguous(), sp[0], causal=False)


class DoubleBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, dtype, device):
        super().__init__()
        d, m, hd = cfg.hidden, cfg.mlp_hidden, cfg.head_dim
        self.cfg = cfg
        self.sp = None
        for s in ("img", "txt"):
            setattr(self, f"{s}_mod", Linear(d, 6 * d, dtype, device))
            setattr(self, f"{s}_qkv", Linear(d, 3 * d, dtype, device))
            setattr(self, f"{s}_qknorm", QKNorm(hd, dtype, device))
            setattr(self, f"{s}_proj", Linear(d, d, dtype, device))
            setattr(self, f"{s}_fc1", Linear(d, m, dtype, device))
            setattr(self, f"{s}_fc2", Linear(m, d, dtype, device))

    def forward(self, img, txt, vec_act, cos, sin, B):
        cfg = self.cfg
        H, hd, pr = cfg.n_heads, cfg.head_dim, cfg.precision
        parts = {}
        for s, x in (("img", img), ("txt", txt)):
            mod = getattr(self, f"{s}_mod")(vec_act).chunk(6, dim=-1)
            qkv = getattr(self, f"{s}_qkv")(_ln_modulate(x, mod[0], mod[1], B), pr)
            S = x.shape[0] // B
            q, k, v = qkv.view(B, S, 3, H, hd).unbind(2)
            q, k = getattr(self, f"{s}_qknorm")(q, k)
            parts[s] = (q, k, v, mod, S)
        St = parts["txt"][4]
        q = _rope(torch.cat([parts["txt"][0], parts["img"][0]], 1), cos, sin)
        k = _rope(torch.cat([parts["txt"][1], parts["img"][1]], 1), cos, sin)
        v = torch.cat([parts["txt"][2], parts["img"][2]], 1)
        attn = _attention(q, k, v, self.sp)
        outs = {}
        for s, x, a in (("txt", txt, attn[:, :St]), ("img", img, attn[:, St:])):
            mod = parts[s][3]
            a2 = a.reshape(-1, H * hd)
            x = _gate(x, getattr(self, f"{s}_proj")(a2, pr), mod[2], B)
            h = F.gelu(getattr(self, f"{s}_fc1")(_ln_modulate(x, mod[3], mod[4], B), pr))
            outs[s] = _gate(x, getattr(self, f"{s}_fc2")(h, pr), mod[5], B)
        return outs["img"], outs["txt"]


class SingleBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, dtype, device):
        super().__init__()
        d, m = cfg.hidden, cfg.mlp_hidden
        self.cfg = cfg
        self.sp = None
        self.mod = Linear(d, 3 * d, dtype, device)
        self.linear1 = Linear(d, 3 * d + m, dtype, device)
        self.linear2 = Linear(d + m, d, dtype, device)
        self.qknorm = QKNorm(cfg.head_dim, dtype, device)

    def forward(self, x, vec_act, cos, sin, B):
        cfg = self.cfg
        H, hd, d, pr = cfg.n_heads, cfg.head_dim, cfg.hidden, cfg.precision
        shift, scale, gate = self.mod(vec_act).chunk(3, dim=-1)
        y = self.linear1(_ln_modulate(x, shift, scale, B), pr)
        S = x.shape[0] // B
        qkv, mlp = y[:, :3 * d], y[:, 3 * d:]
        q, k, v = qkv.reshape(B, S, 3, H, hd).unbind(2)
        q, k = self.qknorm(q, k)
        attn = _attention(_rope(q, cos, sin), _rope(k, cos, sin), v.contiguous(), self.sp).reshape(-1, d)
        out = self.linear2(torch.cat([attn, F.gelu(mlp.contiguous())], dim=-1), pr)
        return _gate(x, out, gate, B)


class MMDiT(nn.Module):
    """``forward(img_tokens [B,Si,64], txt [B,St,4096], pooled [B,768], t [B])`` -> predicted
    velocity ``[B, Si, 64]``; ``loss(...)`` draws the noise / timestep and returns the flow-matching MSE."""

    def __init__(self, cfg: MMDiTConfig, device="cpu", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        dtype = cfg.torch_dtype()
        torch.manual_seed(seed)
        d = cfg.hidden
        self.img_in = Linear(cfg.in_channels, d, dtype, device)
        self.txt_in = Linear(cfg.txt_dim, d, dtype, device)
        self.time_in1, self.time_in2 = Linear(256, d, dtype, device), Linear(d, d, dtype, device)
        self.vec_in1, self.vec_in2 = Linear(cfg.vec_dim, d, dtype, device), Linear(d, d, dtype, device)
        self.double_blocks = nn.ModuleList([DoubleBlock(cfg, dtype, device) for _ in range(cfg.n_double)])
        self.single_blocks = nn.ModuleList([SingleBlock(cfg, dtype, device) for _ in range(cfg.n_single)])
        self.final_mod = Linear(d, 2 * d, dtype, device)
        self.final_out = Linear(d, cfg.in_channels, dtype, device)
        self._rope = None
        self.sp = None

    def rope(self, device):
        if self._rope is None or self._rope[0].device != torch.device(device):
            cfg = self.cfg
            side = cfg.img_size // 16
            txt_ids = torch.zeros(cfg.txt_tokens, 3)
            rows, cols = torch.meshgrid(torch.arange(side), torch.arange(side), indexing="ij")
            img_ids = torch.stack([torch.zeros(side * side), rows.reshape(-1).float(), cols.reshape(-1).float()], -1)
            cos, sin = rope_tables_nd(torch.cat([txt_ids, img_ids], 0), cfg.axes_dim, cfg.rope_theta)
            self._rope = (cos.to(device), sin.to(device))
        return self._rope

    def set_sequence_parallel(self, group) -> None:
        """Shard the image and the text tokens of every sample over ``group`` (rank r keeps the r-th
        chunk of each): ``forward`` still takes whole samples and returns this rank's chunk of the
        prediction, ``loss`` the mean over that chunk.  Parameters are replicated over the group, so the
        gradient reduction must span it (``sp_size`` of flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:48)."""
        import torch.distributed as dist
        W = dist.get_world_size(group) if group is not None else 1
        cfg = self.cfg
        if W > 1 and (cfg.n_heads % W or cfg.img_tokens % W or cfg.txt_tokens % W):
            raise ValueError(f"{cfg.n_heads} heads, {cfg.img_tokens} image and {cfg.txt_tokens} text tokens must divide over {W} ranks")
        self.sp = (group, W, dist.get_rank(group)) if W > 1 else None
        for blk in list(self.double_blocks) + list(self.single_blocks):
            blk.sp = self.sp

    def _chunk(self, x, n_tokens: int):
        """This rank's tokens of ``[B, n_tokens, ...]`` (all of them without sequence parallelism)."""
        if self.sp is None:
            return x
        _, W, r = self.sp
        c = n_tokens // W
        return x[:, r * c:(r + 1) * c]

    def forward(self, img, txt, pooled, t):
        cfg = self.cfg
        B = img.shape[0]
        dt = cfg.torch_dtype()
        cos, sin = self.rope(img.device)
        St, Si = cfg.txt_tokens, cfg.img_tokens
        if self.sp is not None:
            _, W, r = self.sp
            img, txt = self._chunk(img, Si).contiguous(), self._chunk(txt, St).contiguous()
            ct, ci = St // W, Si // W
            rows = torch.cat([torch.arange(r * ct, (r + 1) * ct), St + torch.arange(r * ci, (r + 1) * ci)]).to(cos.device)
            cos, sin = cos[rows].contiguous(), sin[rows].contiguous()
            St, Si = ct, ci
        x_img = self.img_in(img.reshape(-1, cfg.in_channels).to(dt))
        x_txt = self.txt_in(txt.reshape(-1, cfg.txt_dim).to(dt), cfg.precision)
        temb = timestep_embedding(t).to(dt)
        vec = self.time_in2(torch.nn.functional.silu(self.time_in1(temb))) + \
            self.vec_in2(torch.nn.functional.silu(self.vec_in1(pooled.to(dt))))
        vec_act = torch.nn.functional.silu(vec)
        ckpt = cfg.recompute == "full" and torch.is_grad_enabled()
        if ckpt:
            from torch.utils.checkpoint import checkpoint
        n_d = round(cfg.recompute_ratio * len(self.double_blocks)) if ckpt else 0
        n_s = round(cfg.recompute_ratio * len(self.single_blocks)) if ckpt else 0
        for i, blk in enumerate(self.double_blocks):
            if i < n_d:
                x_img, x_txt = checkpoint(blk, x_img, x_txt, vec_act, cos, sin, B, use_reentrant=False)
            else:
                x_img, x_txt = blk(x_img, x_txt, vec_act, cos, sin, B)
        x = torch.cat([x_txt.view(B, St, -1), x_img.view(B, Si, -1)], 1).reshape(-1, cfg.hidden)
        for i, blk in enumerate(self.single_blocks):
            if i < n_s:
                x = checkpoint(blk, x, vec_act, cos, sin, B, use_reentrant=False)
            else:
                x = blk(x, vec_act, cos, sin, B)
        x = x.view(B, St + Si, -1)[:, St:].reshape(-1, cfg.hidden)
        shift, scale = self.final_mod(vec_act).chunk(2, dim=-1)
        return self.final_out(_ln_modulate(x, shift, scale, B)).view(B, Si, cfg.in_channels)

    def loss(self, latents, txt, pooled, generator=None, prompt_dropout: float = 0.0, empty_txt=None,
             empty_pooled=None):
        """Rectified-flow objective: ``x_t = (1 - t) x0 + t eps``, target velocity ``eps - x0``,
        ``t`` logit-normal; with probability ``prompt_dropout`` a sample's conditioning is replaced
        by the empty-prompt encodings (flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:40-44)."""
        B = latents.shape[0]
        dev = latents.device
        t = torch.sigmoid(torch.randn(B, generator=generator, device=dev))
        eps = torch.randn(latents.shape, generator=generator, device=dev, dtype=torch.float32)
        x0 = latents.float()
        xt = (1 - t)[:, None, None] * x0 + t[:, None, None] * eps
        if prompt_dropout > 0:
            drop = torch.rand(B, generator=generator, device=dev) < prompt_dropout
            e_txt = empty_txt if empty_txt is not None else torch.zeros_like(txt[:1])
            e_pool = empty_pooled if empty_pooled is not None else torch.zeros_like(pooled[:1])
            txt = torch.where(drop[:, None, None], e_txt.expand_as(txt), txt)
            pooled = torch.where(drop[:, None], e_pool.expand_as(pooled), pooled)
        pred = self.forward(xt, txt, pooled, t)
        return ((pred.float() - self._chunk(eps - x0, self.cfg.img_tokens)) ** 2).mean()


def patchify(latents: torch.Tensor, patch: int = 2) -> torch.Tensor:
    """``[B, C, H, W]`` -> ``[B, (H/p)(W/p), C p p]``."""
    B, C, H, W = latents.shape
    x = latents.view(B, C, H // patch, patch, W // patch, patch).permute(0, 2, 4, 1, 3, 5)
    return x.reshape(B, (H // patch) * (W // patch), C * patch * patch)


def unpatchify(tokens: torch.Tensor, channels: int, side: int, patch: int = 2) -> torch.Tensor:
    B = tokens.shape[0]
    x = tokens.view(B, side, side, channels, patch, patch).permute(0, 3, 1, 4, 2, 5)
    return x.reshape(B, channels, side * patch, side * patch)

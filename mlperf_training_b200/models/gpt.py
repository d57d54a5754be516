"""Decoder-only GPT family: Llama-3.1-8B, Llama-2-70B (dense) and GPT-OSS-20B (MoE) architectures.

RMSNorm -> fused QKV GEMM -> RoPE -> flash attention (causal, GQA, optional sliding window and
learned sink logits) -> output GEMM with the residual add in its epilogue -> RMSNorm -> SwiGLU MLP
(dense or routed experts) -> residual; final norm, untied vocabulary GEMM and fused cross-entropy.

The reference takes this model from Megatron-Core's ``GPTModel`` through Primus model presets;
the in-tree YAMLs only override it (small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:12,44-45;
small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:19-33,115-167;
llama2_sft/primus/src/llama2_custom.py:496-500).  Activations are 2-D ``[tokens, features]``
throughout so every GEMM sees one large M.
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass, field, asdict

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import kernels as K


@dataclass
class GPTConfig:
    name: str = "gpt"
    n_layers: int = 2
    hidden: int = 256
    n_heads: int = 8
    n_kv_heads: int = 2
    head_dim: int = 32
    ffn_hidden: int = 512
    vocab_size: int = 2048
    seq_len: int = 256
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02
    # attention variants
    window: int = 0                 # sliding-window length (0 = full attention)
    window_layers: str = "none"     # "none" | "even" | "all": which layers use the window
    sink: bool = False              # learned per-head sink logits
    # mixture of experts (0 experts = dense MLP)
    n_experts: int = 0
    top_k: int = 0
    moe_ffn_hidden: int = 0
    router_dtype: str = "fp32"
    ep_comm: str = "nccl"          # expert-parallel token movement: "nccl" all-to-all | "fused" peer-memory kernels
    # LoRA (rank 0 = off)
    lora_rank: int = 0
    lora_alpha: float = 32.0
    lora_dropout: float = 0.0
    lora_targets: tuple = ("qkv", "proj")
    # activation recompute: "none" | "full" (every block's forward is run again in backward and only
    # its input is kept) | "offload" (nothing is recomputed: what a block saves for backward moves to
    # pinned host memory, the CPU activation offload of llama2_sft/primus/src/llama2_custom.py:522-542);
    # recompute_layers > 0 limits either to the first N blocks
    recompute: str = "none"
    recompute_layers: int = 0
    swiglu_store: str = "bf16"          # "fp8": the fused MXFP8 MLP keeps its gate | up activation for backward as e4m3 codes
    dtype: str = "bf16"
    precision: str = "bf16"         # GEMM precision of the linears: "bf16" | "mxfp8"
    # the first / last N transformer layers keep bf16 linears whatever ``precision`` says (Megatron's
    # first_last_layers_bf16 with num_layers_at_start_in_bf16 / num_layers_at_end_in_bf16, an option of the
    # low-precision recipes: small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:55-57)
    bf16_first_layers: int = 0
    bf16_last_layers: int = 0

    def torch_dtype(self) -> torch.dtype:
        return {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[self.dtype]

    def layer_window(self, layer: int) -> int:
        if self.window <= 0 or self.window_layers == "none":
            return 0
        if self.window_layers == "all":
            return self.window
        return self.window if layer % 2 == 0 else 0

    def num_params(self) -> int:
        d, hd = self.hidden, self.head_dim
        attn = d * (self.n_heads + 2 * self.n_kv_heads) * hd + self.n_heads * hd * d
        if self.n_experts:
            mlp = self.n_experts * 3 * d * self.moe_ffn_hidden + d * self.n_experts
        else:
            mlp = 3 * d * self.ffn_hidden
        per_layer = attn + mlp + 2 * d + (self.n_heads if self.sink else 0)
        return self.n_layers * per_layer + 2 * self.vocab_size * d + d

    def flops_per_token(self, seq_len: int | None = None) -> float:
        """Model FLOPs per trained token (fwd + bwd = 3 x fwd), GEMMs plus causal attention."""
        s = seq_len or self.seq_len
        d, hd = self.hidden, self.head_dim
        attn_proj = d * (self.n_heads + 2 * self.n_kv_heads) * hd + self.n_heads * hd * d
        mlp = (self.top_k * 3 * d * self.moe_ffn_hidden + d * self.n_experts) if self.n_experts else 3 * d * self.ffn_hidden
        gemm = 2 * (self.n_layers * (attn_proj + mlp) + self.vocab_size * d)
        attn = 0.0
        for layer in range(self.n_layers):
            w = self.layer_window(layer)
            keys = min(w, s) if w else s / 2
            attn += 4 * self.n_heads * hd * keys
        return 3 * gemm + 3.5 * attn

    def to_dict(self) -> dict:
        return asdict(self)


def llama31_8b(**over) -> GPTConfig:
    return GPTConfig(name="llama3.1-8b", n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                     ffn_hidden=14336, vocab_size=128256, seq_len=8192, rope_theta=500000.0, norm_eps=1e-5,
                     init_std=0.02, **over)


def llama2_70b(**over) -> GPTConfig:
    return GPTConfig(name="llama2-70b", n_layers=80, hidden=8192, n_heads=64, n_kv_heads=8, head_dim=128,
                     ffn_hidden=28672, vocab_size=32000, seq_len=8192, rope_theta=10000.0, norm_eps=1e-5,
                     init_std=0.02, **over)


def gpt_oss_20b(**over) -> GPTConfig:
    return GPTConfig(name="gpt-oss-20b", n_layers=24, hidden=2880, n_heads=64, n_kv_heads=8, head_dim=64,
                     ffn_hidden=2880, vocab_size=201088, seq_len=8192, rope_theta=150000.0, norm_eps=1e-6,
                     init_std=0.008, window=128, window_layers="even", sink=True, n_experts=32, top_k=4,
                     moe_ffn_hidden=2880, **over)


def tiny_moe(**over) -> GPTConfig:
    """The CPU plumbing config: 4 layers, d 256, 8q/2kv heads of 32, 8 experts top-2, vocab 2048."""
    base = dict(name="tiny-moe", n_layers=4, hidden=256, n_heads=8, n_kv_heads=2, head_dim=32, ffn_hidden=512,
                vocab_size=2048, seq_len=256, rope_theta=10000.0, init_std=0.02, window=128, window_layers="even",
                n_experts=8, top_k=2, moe_ffn_hidden=512, dtype="fp32")
    base.update(over)
    return GPTConfig(**base)


PRESETS = {"llama3.1-8b": llama31_8b, "llama2-70b": llama2_70b, "gpt-oss-20b": gpt_oss_20b, "tiny-moe": tiny_moe}


def shard_of(full: torch.Tensor, kind: str, W: int, r: int, cfg: "GPTConfig") -> torch.Tensor:
    """This rank's slice of a full weight.  ``rows`` / ``cols``: contiguous split of dim 0 / 1;
    ``rows_2``: two stacked matrices (gate | up), each split; ``qkv``: q | k | v head blocks, each split."""
    if kind == "rows":
        return full.chunk(W, 0)[r]
    if kind == "cols":
        return full.chunk(W, 1)[r]
    if kind == "rows_2":
        g, u = full.chunk(2, 0)
        return torch.cat([g.chunk(W, 0)[r], u.chunk(W, 0)[r]], 0)
    if kind == "qkv":
        hd = cfg.head_dim
        q, k, v = full.split([cfg.n_heads * hd, cfg.n_kv_heads * hd, cfg.n_kv_heads * hd], 0)
        return torch.cat([q.chunk(W, 0)[r], k.chunk(W, 0)[r], v.chunk(W, 0)[r]], 0)
    raise ValueError(kind)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, self.weight, self.eps)


class DenseMLP(nn.Module):
    """gate/up projection as one GEMM ([2F, D], gate rows first), SwiGLU, down projection."""

    def __init__(self, cfg: GPTConfig, dtype, device, tp=None):
        super().__init__()
        d, f = cfg.hidden, cfg.ffn_hidden
        self.tp = tp if (tp is not None and tp.world > 1) else None
        if self.tp is not None:
            if f % self.tp.world:
                raise ValueError(f"ffn_hidden {f} is not divisible by the tensor-parallel size {self.tp.world}")
            f //= self.tp.world
        self.precision = cfg.precision
        self.force_bf16 = False          # set for the first / last layers that stay in bf16
        self.fused = True               # MXFP8: one unit with the quantisation folded into SwiGLU / dSwiGLU
        self.store_fp8 = getattr(cfg, "swiglu_store", "bf16") == "fp8"
        self.w_gate_up = nn.Parameter(torch.empty(2 * f, d, dtype=dtype, device=device))
        self.w_down = nn.Parameter(torch.empty(d, f, dtype=dtype, device=device))
        if self.tp is not None:
            self.w_gate_up.tensor_parallel = ("rows_2", self.tp.world, self.tp.rank)   # gate rows | up rows, each split
            self.w_down.tensor_parallel = ("cols", self.tp.world, self.tp.rank)

    def forward(self, h, norm_w, eps):
        if self.tp is not None:
            from ..parallel import tensor as T
            gu = T.column_parallel(F.rms_norm(h, norm_w, eps), self.w_gate_up, self.tp)
            return T.row_parallel(F.swiglu(gu), self.w_down, self.tp, residual=h)
        pr = "bf16" if self.force_bf16 else self.precision
        if pr == "mxfp8" and self.fused and F.fused_mlp_eligible(h, self.w_gate_up, self.w_down):
            return F.fused_mlp(h, norm_w, self.w_gate_up, self.w_down, eps, self.store_fp8)
        gu = F.norm_linear(h, norm_w, self.w_gate_up, eps=eps, precision=pr)
        return F.swiglu_linear(gu, self.w_down, residual=h, precision=pr)


class Block(nn.Module):
    def __init__(self, cfg: GPTConfig, layer: int, dtype, device, mlp: nn.Module | None = None, ep_group=None, tp=None):
        super().__init__()
        self.cfg = cfg
        self.layer = layer
        self.force_bf16 = layer < cfg.bf16_first_layers or layer >= cfg.n_layers - cfg.bf16_last_layers
        d, hd = cfg.hidden, cfg.head_dim
        self.tp = tp if (tp is not None and tp.world > 1) else None
        W = self.tp.world if self.tp is not None else 1
        if cfg.n_heads % W or cfg.n_kv_heads % W:
            raise ValueError(f"heads {cfg.n_heads}/{cfg.n_kv_heads} are not divisible by the tensor-parallel size {W}")
        self.hq, self.hkv = cfg.n_heads // W, cfg.n_kv_heads // W
        self.attn_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.w_qkv = nn.Parameter(torch.empty((self.hq + 2 * self.hkv) * hd, d, dtype=dtype, device=device))
        self.w_proj = nn.Parameter(torch.empty(d, self.hq * hd, dtype=dtype, device=device))
        self.sink = nn.Parameter(torch.zeros(self.hq, dtype=torch.float32, device=device)) if cfg.sink else None
        self.cp = None                   # (group, mode) once GPT.set_context_parallel is called
        self.mlp_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        if self.tp is not None:
            self.w_qkv.tensor_parallel = ("qkv", W, self.tp.rank)
            self.w_proj.tensor_parallel = ("cols", W, self.tp.rank)
            if self.sink is not None:
                self.sink.tensor_parallel = ("rows", W, self.tp.rank)
        if mlp is not None:
            self.mlp = mlp
        elif cfg.n_experts:
            from .moe import MoEMLP
            self.mlp = MoEMLP(cfg, dtype, device, ep_group=ep_group, ep_comm=cfg.ep_comm)
        else:
            self.mlp = DenseMLP(cfg, dtype, device, tp=self.tp)
            self.mlp.force_bf16 = self.force_bf16
        self.lora_qkv = self.lora_proj = None
        if cfg.lora_rank > 0:
            from .lora import LoRAAdapter
            if "qkv" in cfg.lora_targets:
                self.lora_qkv = LoRAAdapter(d, self.w_qkv.shape[0], cfg.lora_rank, cfg.lora_alpha, cfg.lora_dropout,
                                            dtype, device)
                if self.tp is not None:
                    self.lora_qkv.b.tensor_parallel = ("qkv", W, self.tp.rank)      # A stays replicated
            if "proj" in cfg.lora_targets:
                self.lora_proj = LoRAAdapter(self.hq * hd, d, cfg.lora_rank, cfg.lora_alpha, cfg.lora_dropout,
                                             dtype, device)
                if self.tp is not None:
                    self.lora_proj.a.tensor_parallel = ("cols", W, self.tp.rank)    # B stays replicated

    def _forward_tp(self, x, cos, sin, B, S):
        """Sequence-parallel forward: ``x`` is this rank's block of token rows ``[T/W, hidden]``."""
        from ..parallel import tensor as T
        cfg, tp = self.cfg, self.tp
        xn = F.rms_norm(x, self.attn_norm, cfg.norm_eps)
        qkv = T.column_parallel(xn, self.w_qkv, tp)
        if self.lora_qkv is not None:
            lo = self.lora_qkv
            qkv = qkv + lo.up(T.GatherRows.apply(lo.down(xn), tp))
        if self.cp is not None:
            a = self._attention_cp(qkv, cos, sin, B, S, self.hq, self.hkv)       # this rank's heads, sequence over the cp group
        else:
            a = F.attention_packed(qkv, B=B, S=S, Hq=self.hq, Hkv=self.hkv, D=cfg.head_dim, cos=cos, sin=sin,
                                   sink=self.sink, causal=True, window=cfg.layer_window(self.layer))
        h = T.row_parallel(a, self.w_proj, tp, residual=x)
        if self.lora_proj is not None:
            lo = self.lora_proj
            h = h + lo.up(T.ScatterRows.apply(lo.down(a), tp))
        return self.mlp(h, self.mlp_norm, cfg.norm_eps)

    def _attention_cp(self, qkv, cos, sin, B, S, Hq=None, Hkv=None):
        """Attention with the sequence sharded over ``self.cp = (group, mode)``: ``S`` is this rank's
        chunk and ``cos`` / ``sin`` its rows of the tables.  ``mode`` "allgather" gathers keys and
        values of the earlier chunks, "ulysses" trades sequence shards for head shards, "ring" passes key / value
        blocks round the ring over zig-zag chunks."""
        from ..parallel.context import context_parallel_attention, ring_attention, ulysses_attention
        cfg = self.cfg
        group, mode = self.cp
        Hq, Hkv, D = Hq or cfg.n_heads, Hkv or cfg.n_kv_heads, cfg.head_dim
        v3 = F.rope_packed(qkv, cos, sin, S=S, Hq=Hq, Hkv=Hkv, D=D).view(B, S, -1)
        q = v3[:, :, :Hq * D].unflatten(-1, (Hq, D))
        k = v3[:, :, Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
        v = v3[:, :, (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
        window = cfg.layer_window(self.layer)
        if mode == "ulysses":
            a = ulysses_attention(q, k, v, group, causal=True, window=window)
        elif mode == "ring":
            if window:
                raise NotImplementedError("ring attention does not carry a sliding window")
            a = ring_attention(q, k, v, group)
        else:
            a = context_parallel_attention(q, k, v, group, window=window)
        return a.reshape(B * S, Hq * D)

    def forward(self, x, cos, sin, B, S):
        cfg = self.cfg
        if self.tp is not None:
            return self._forward_tp(x, cos, sin, B, S)
        pr = "bf16" if self.force_bf16 else cfg.precision
        if self.lora_qkv is None:
            qkv = F.norm_linear(x, self.attn_norm, self.w_qkv, eps=cfg.norm_eps, precision=pr)
        else:
            xn = F.rms_norm(x, self.attn_norm, cfg.norm_eps)
            qkv = F.linear(xn, self.w_qkv, None, self.lora_qkv(xn), pr)      # adapter output joins in the GEMM epilogue
        if self.cp is not None:
            a = self._attention_cp(qkv, cos, sin, B, S)
        else:
            a = F.attention_packed(qkv, B=B, S=S, Hq=cfg.n_heads, Hkv=cfg.n_kv_heads, D=cfg.head_dim, cos=cos, sin=sin,
                                   sink=self.sink, causal=True, window=cfg.layer_window(self.layer))
        if self.lora_proj is None:
            h = F.linear(a, self.w_proj, None, x, pr)
        else:
            h = F.linear(a, self.w_proj, None, x + self.lora_proj(a), pr)
        return self.mlp(h, self.mlp_norm, cfg.norm_eps)


class GPT(nn.Module):
    """``forward(tokens [B,S], labels [B,S]) -> mean cross-entropy`` (labels -100 are ignored)."""

    def __init__(self, cfg: GPTConfig, device="cpu", seed: int = 0, ep_group=None, tp=None):
        super().__init__()
        self.cfg = cfg
        self.tp = tp if (tp is not None and tp.world > 1) else None
        dtype = cfg.torch_dtype()
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([Block(cfg, i, dtype, device, ep_group=ep_group, tp=self.tp)
                                     for i in range(cfg.n_layers)])
        self.final_norm = nn.Parameter(torch.ones(cfg.hidden, dtype=dtype, device=device))
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device))
        self._rope = None
        self.cp = None
        # optional callable(block_key): told when the backward of a block has produced all its gradients
        self.grad_ready_hook = None
        # optional object with pre_forward(i) / pre_backward(i) / post_backward(i): a sharded-parameter engine
        # gathers a block's matrices before the block runs and reduces its gradients right after its backward
        self.block_hooks = None
        self.reset_parameters(seed)

    @torch.no_grad()
    def reset_parameters(self, seed: int = 0) -> None:
        """N(0, init_std) for matrices (output projections scaled by 1/sqrt(2 L) as Megatron
        does), ones for norm weights, zeros for sinks and LoRA B, seeded Xavier-uniform LoRA A."""
        gen = torch.Generator(device="cpu").manual_seed(seed)
        std = self.cfg.init_std
        out_std = std / math.sqrt(2.0 * self.cfg.n_layers)
        for name, p in self.named_parameters():
            if p.dim() < 2:
                continue
            if "lora" in name:
                # adapters: B zero, A Xavier-uniform over the unsharded shape, from a generator of its own
                # (seeded by the parameter's name) so that every replica draws the same A whatever the
                # process-wide RNG state is, and the base weights do not depend on the adapters' presence
                if name.endswith(".b"):
                    p.zero_()
                    continue
                shard = getattr(p, "tensor_parallel", None)
                W_, r_ = (shard[1], shard[2]) if shard is not None else (1, 0)
                full_in = p.shape[1] * W_
                bound = math.sqrt(6.0 / (full_in + p.shape[0]))
                g = torch.Generator(device="cpu").manual_seed(seed + 7919 + (zlib.crc32(name.encode()) & 0xFFFFFF))
                full = torch.empty((p.shape[0], full_in), dtype=torch.float32).uniform_(-bound, bound, generator=g)
                p.copy_((full.chunk(W_, 1)[r_] if W_ > 1 else full).to(p.dtype))
                continue
            s = out_std if (name.endswith("w_proj") or name.endswith("w_down") or name.endswith("w2")) else std
            shard = getattr(p, "tensor_parallel", None)
            if shard is not None:
                # draw the full matrix (identical on every rank) and keep this rank's slice, so a
                # tensor-parallel model starts from the same weights as the unsharded one
                kind, W, r = shard
                full_shape = (p.shape[0] * W, p.shape[1]) if kind in ("rows", "rows_2", "qkv") else (p.shape[0], p.shape[1] * W)
                if p.device.type == "cpu":
                    full = torch.empty(full_shape, dtype=p.dtype).normal_(0.0, s, generator=gen)
                else:
                    g = torch.Generator(device=p.device).manual_seed(seed + (zlib.crc32(name.encode()) & 0xFFFF))
                    full = torch.empty(full_shape, dtype=p.dtype, device=p.device).normal_(0.0, s, generator=g)
                p.copy_(shard_of(full, kind, W, r, self.cfg))
                del full
            elif p.device.type == "cpu":
                p.normal_(0.0, s, generator=gen)
            else:
                g = torch.Generator(device=p.device).manual_seed(seed + (zlib.crc32(name.encode()) & 0xFFFF))
                p.normal_(0.0, s, generator=g)

    def rope(self, device):
        if self._rope is None or self._rope[0].device != torch.device(device):
            self._rope = K.rope_tables(self.cfg.seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    def set_context_parallel(self, group, mode: str = "allgather") -> None:
        """Shard the sequence over ``group``: ``forward`` then takes this rank's chunk ``[B, S / W]`` of
        tokens and labels (chunk index = rank in the group; with ``mode="ring"`` the two zig-zag chunks ``r`` and
        ``2 W - 1 - r`` side by side) and returns the mean loss of that chunk;
        parameters are replicated over the group, so the optimizer's gradient reduction must span it
        (``context_parallel_size`` of the reference's Megatron model config,
        llama2_sft/primus/src/llama2_custom.py:396-505, llama2_sft/primus/conf/llama2_70b_lora_posttrain.yaml:22)."""
        import torch.distributed as dist
        if group is None or dist.get_world_size(group) == 1:
            self.cp = None
            for blk in self.blocks:
                blk.cp = None
            return
        if self.cfg.sink:
            raise NotImplementedError("context parallelism does not carry attention sink logits")
        if mode not in ("allgather", "ulysses", "ring"):
            raise ValueError(f"unknown context-parallel mode '{mode}'")
        self.cp = (group, dist.get_world_size(group), dist.get_rank(group))
        self.cp_mode = mode
        for blk in self.blocks:
            blk.cp = (group, mode)

    def forward(self, tokens: torch.Tensor, labels: torch.Tensor, n_valid: int | None = None) -> torch.Tensor:
        B, S = tokens.shape
        cos, sin = self.rope(tokens.device)
        if self.cp is not None:
            _, W, r = self.cp
            if S * W > cos.shape[0]:
                raise ValueError(f"sequence {S * W} longer than the configured {cos.shape[0]}")
            if getattr(self, "cp_mode", "allgather") == "ring":
                # zig-zag: this rank's tokens are chunks r and 2 W - 1 - r of the 2 W chunks of the sequence
                from ..parallel.context import zigzag_chunk
                cos, sin = zigzag_chunk(cos[:S * W], W, r, dim=0), zigzag_chunk(sin[:S * W], W, r, dim=0)
            else:
                cos, sin = cos[r * S:(r + 1) * S].contiguous(), sin[r * S:(r + 1) * S].contiguous()
        if S > cos.shape[0]:
            raise ValueError(f"sequence {S} longer than the configured {cos.shape[0]}")
        ids, tgt = tokens.reshape(-1), labels.reshape(-1)
        if self.tp is not None:
            # sequence parallel: every rank embeds and scores its own block of token rows; the
            # embedding, the final norm and the head are replicated and their gradients summed over
            # the tensor-parallel group by the engine.  The returned loss is this rank's share.
            W, r = self.tp.world, self.tp.rank
            rows = ids.numel() // W
            if ids.numel() % W:
                raise ValueError("the number of tokens must be divisible by the tensor-parallel size")
            if n_valid is None:
                n_valid = ids.numel()
            ids, tgt = ids[r * rows:(r + 1) * rows], tgt[r * rows:(r + 1) * rows]
        x = F.embedding(ids, self.embed)
        ckpt = self.cfg.recompute == "full" and torch.is_grad_enabled()
        offload = self.cfg.recompute == "offload" and torch.is_grad_enabled()
        notify = self.grad_ready_hook if (torch.is_grad_enabled() and not ckpt) else None
        hooks = self.block_hooks
        n_blocks = len(self.blocks)
        for i, blk in enumerate(self.blocks):
            if notify is not None and x.requires_grad:
                # the gradient w.r.t. a block's input is the last thing its backward produces
                x.register_hook(lambda g, key=f"block{i:04d}", fn=notify: fn(key))
            if hooks is not None:
                if torch.is_grad_enabled() and x.requires_grad:
                    # boundary between block i - 1 and block i: block i's backward has just finished (its
                    # gradients can leave), block i - 1's is about to start (its parameters must be there)
                    def _boundary(g, i=i, h=hooks):
                        h.post_backward(i)
                        if i > 0:
                            h.pre_backward(i - 1)
                    x.register_hook(_boundary)
                hooks.pre_forward(i)
            if ckpt and (self.cfg.recompute_layers <= 0 or i < self.cfg.recompute_layers):
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(blk, x, cos, sin, B, S, use_reentrant=False)
            elif offload and (self.cfg.recompute_layers <= 0 or i < self.cfg.recompute_layers):
                # keep what this block saves for backward in (pinned) host memory instead of on the device
                with torch.autograd.graph.save_on_cpu(pin_memory=x.is_cuda):
                    x = blk(x, cos, sin, B, S)
            else:
                x = blk(x, cos, sin, B, S)
        if hooks is not None and torch.is_grad_enabled() and x.requires_grad:
            x.register_hook(lambda g, h=hooks, i=n_blocks - 1: h.pre_backward(i))
        return F.lm_head_loss(x, self.final_norm, self.lm_head, tgt, eps=self.cfg.norm_eps,
                              n_valid=n_valid, precision=self.cfg.precision)

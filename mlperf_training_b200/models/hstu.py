"""DLRMv4 / HSTU generative recommender (sequential transducer over jagged user histories).

Pipeline (fp32 oracle spec = the reference's PyTorch path, generative_recommenders/modules/):

    item embeddings (+ action bits)  -> ContextualPreprocessor: content MLP + action MLP (sum)
    -> HSTUPositionalEncoder: x * sqrt(D) + position embedding + time-bucket embedding, input dropout
    -> STU stack: per layer  LN -> UVQK GEMM (+beta) -> u = silu(u) -> jagged SiLU attention
                  -> y = u * LN(attn) -> [u, attn, y] -> dropout -> out-proj GEMM + residual
    -> candidate rows only -> TimestampLayerNorm postprocessor
    item tower: MLP(candidate embeddings); head: MLP(user * item) -> logits -> weighted BCE * 0.2

Sources of the math: dlrm_hstu.py:185-463,807-932,1118-1255 (top model, item MLP, heads),
stu.py:274-328,475-650 (layer parameters / forward, split order u, v, q, k, eps 1e-6),
preprocessors.py:188-323 (MLP shapes), action_encoder.py:27-171, positional_encoder.py:33-167 with
pt_position.py:35-142 (index reversal from the first target, sqrt time buckets, clamp to 2048),
postprocessors.py:99-212 (period features with the literal 3.14), multitask_module.py:132-174
(loss normalisation by the clamped weight sum).

All GEMMs, LayerNorms, the jagged attention and the embedding gather run on this package's sm_100a
kernels for CUDA tensors; the same module runs in eager fp32 on CPU as the oracle.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..ops.hstu_ops import GateCatFn, gate_cat_eligible, hstu_attention


@dataclass
class HSTUConfig:
    name: str = "hstu"
    layers: int = 8
    dim: int = 512
    heads: int = 4
    d_qk: int = 128
    d_v: int = 128
    max_seq_len: int = 4096
    emb_dim: int = 256                 # item-id embedding width
    mlp_hidden: int = 256
    action_bits: tuple = (1, 2, 4)
    action_dim: int = 8
    contextual: int = 0                # contextual tokens prepended to every sequence
    input_dropout: float = 0.2
    linear_dropout: float = 0.1
    fuse_glue: bool = True             # SiLU(u) * LayerNorm(attn) + concat + dropout as one kernel each way (GPU, bf16)
    num_positions: int = 8192
    num_time_buckets: int = 2048
    n_tasks: int = 1
    task_weight_bit: int = 1           # label = (action & bit) > 0
    causal_multitask_weight: float = 0.2
    time_periods: tuple = ((3600.0, 24), (86400.0, 7))   # (period seconds, units): hour of day, day of week
    targets_only_last: bool = True
    dtype: str = "bf16"
    precision: str = "bf16"

    def torch_dtype(self):
        return {"bf16": torch.bfloat16, "fp32": torch.float32}[self.dtype]

    def to_dict(self):
        return asdict(self)

    def layer_flops_per_token(self, avg_len: float) -> float:
        """Forward MACs x 2 per token of one STU layer (the reference's FLOP model,
        dlrm_hstu.py:498-543): UVQK + out-proj GEMMs and causal attention over ``avg_len`` keys."""
        d, h = self.dim, self.heads
        gemm = 2 * (d * (2 * h * self.d_v + 2 * h * self.d_qk) + 3 * h * self.d_v * d)
        attn = 2 * 2 * h * (self.d_qk + self.d_v) / 2 * avg_len / 2 * 2
        return gemm + attn


def tiny_hstu(**over) -> HSTUConfig:
    base = dict(name="tiny-hstu", layers=2, dim=64, heads=2, d_qk=32, d_v=32, max_seq_len=64, emb_dim=32,
                mlp_hidden=32, num_positions=128, num_time_buckets=64, dtype="fp32")
    base.update(over)
    return HSTUConfig(**base)


class _Linear(nn.Module):
    def __init__(self, n_in, n_out, dtype, device, bias=True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_out, n_in, dtype=dtype, device=device))
        nn.init.xavier_uniform_(self.weight)
        self.bias = nn.Parameter(torch.zeros(n_out, dtype=dtype, device=device)) if bias else None

    def forward(self, x, precision="bf16", residual=None):
        if x.shape[1] % 8 or self.weight.shape[0] % 8:      # tiny ragged widths (e.g. 24 action dims)
            y = x @ self.weight.t()
            y = y + self.bias if self.bias is not None else y
            return y + residual if residual is not None else y
        return F.linear(x, self.weight, self.bias, residual, precision)


class _LN(nn.Module):
    def __init__(self, dim, dtype, device, eps=1e-5, swish=False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))
        self.eps, self.swish = eps, swish

    def forward(self, x):
        if self.swish:
            return F.swish_layer_norm(x, self.weight, self.bias, self.eps)
        return F.layer_norm(x, self.weight, self.bias, self.eps)


class _MLP(nn.Module):
    """Linear(in -> hidden) -> SwishLN(hidden) -> Linear(hidden -> out) -> LN(out)."""

    def __init__(self, n_in, hidden, n_out, dtype, device):
        super().__init__()
        self.l1 = _Linear(n_in, hidden, dtype, device)
        self.n1 = _LN(hidden, dtype, device, swish=True)
        self.l2 = _Linear(hidden, n_out, dtype, device)
        self.n2 = _LN(n_out, dtype, device)

    def forward(self, x, precision="bf16"):
        return self.n2(self.l2(self.n1(self.l1(x, precision)), precision))


class ActionEncoder(nn.Module):
    """Per-bit learned rows for history tokens, one learned row for target tokens."""

    def __init__(self, cfg: HSTUConfig, dtype, device):
        super().__init__()
        nb = len(cfg.action_bits)
        self.bits = cfg.action_bits
        self.table = nn.Parameter(torch.randn(nb, cfg.action_dim, dtype=dtype, device=device) * 0.1)
        self.target_row = nn.Parameter(torch.randn(1, nb * cfg.action_dim, dtype=dtype, device=device) * 0.1)

    def forward(self, actions: torch.Tensor, is_target: torch.Tensor) -> torch.Tensor:
        bits = torch.tensor(self.bits, device=actions.device)
        on = ((actions[:, None] & bits[None, :]) > 0).to(self.table.dtype)            # [L, nb]
        emb = (on[:, :, None] * self.table[None]).reshape(actions.shape[0], -1)       # [L, nb * dim]
        return torch.where(is_target[:, None], self.target_row.expand_as(emb), emb)


class STULayer(nn.Module):
    def __init__(self, cfg: HSTUConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.fuse_glue = cfg.fuse_glue
        d, h = cfg.dim, cfg.heads
        self.split = [h * cfg.d_v, h * cfg.d_v, h * cfg.d_qk, h * cfg.d_qk]       # u, v, q, k
        self.uvqk_weight = nn.Parameter(torch.empty(sum(self.split), d, dtype=dtype, device=device))
        nn.init.xavier_uniform_(self.uvqk_weight)
        self.uvqk_beta = nn.Parameter(torch.zeros(sum(self.split), dtype=dtype, device=device))
        self.in_norm_w = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.in_norm_b = nn.Parameter(torch.zeros(d, dtype=dtype, device=device))
        self.out_weight = nn.Parameter(torch.empty(d, 3 * h * cfg.d_v, dtype=dtype, device=device))
        nn.init.xavier_uniform_(self.out_weight)
        self.out_norm_w = nn.Parameter(torch.ones(h * cfg.d_v, dtype=dtype, device=device))
        self.out_norm_b = nn.Parameter(torch.zeros(h * cfg.d_v, dtype=dtype, device=device))

    def forward(self, x, offsets, num_targets, rows: int):
        cfg = self.cfg
        h = cfg.heads
        uvqk = F.norm_linear(x, self.in_norm_w, self.uvqk_weight, norm_b=self.in_norm_b, bias=self.uvqk_beta,
                             eps=1e-6, layer_norm=True, precision=cfg.precision)
        # one split (its backward is a single concatenation; four slices would each build a zero-filled
        # gradient of the whole uvqk matrix)
        u_raw, v_raw, q_raw, k_raw = torch.split(uvqk, list(self.split), dim=1)
        v = v_raw.unflatten(-1, (h, cfg.d_v))
        q = q_raw.unflatten(-1, (h, cfg.d_qk))
        k = k_raw.unflatten(-1, (h, cfg.d_qk))
        attn = hstu_attention(q, k, v, offsets, cfg.max_seq_len + cfg.contextual, cfg.d_qk ** -0.5, num_targets,
                              cfg.contextual).reshape(x.shape[0], h * cfg.d_v)
        if self.fuse_glue and gate_cat_eligible(u_raw, attn):
            # SiLU(u), the layer norm of the attention output, their product and the concatenation in one kernel
            # (and the dropout of the concatenation, its mask regenerated in backward from a Philox seed)
            cat = GateCatFn.apply(u_raw, attn, self.out_norm_w, self.out_norm_b, 1e-6,
                                  cfg.linear_dropout if self.training else 0.0)
        else:
            u = TF.silu(u_raw)
            y = u * F.layer_norm(attn, self.out_norm_w, self.out_norm_b, 1e-6)
            cat = torch.cat([u, attn, y], dim=1)
            if cfg.linear_dropout > 0 and self.training:
                cat = TF.dropout(cat, cfg.linear_dropout)
        return F.linear(cat.contiguous(), self.out_weight, None, x, cfg.precision)


class HSTU(nn.Module):
    """``forward(batch, item_emb)`` -> ``(loss, preds, labels)``.

    ``batch`` (all on the model's device): ``lengths [B]`` (history + targets per sample),
    ``offsets [B+1]`` int32, ``num_targets [B]``, ``timestamps [L]`` (seconds), ``actions [L]``
    (bit mask), ``rows`` = L padded to a multiple of 128.  ``item_emb`` ``[rows, emb_dim]`` is the
    looked-up item embedding of every token (padding rows zero)."""

    def __init__(self, cfg: HSTUConfig, device="cpu", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        dt = cfg.torch_dtype()
        torch.manual_seed(seed)
        d = cfg.dim
        self.content_mlp = _MLP(cfg.emb_dim, cfg.mlp_hidden, d, dt, device)
        self.action_enc = ActionEncoder(cfg, dt, device)
        self.action_mlp = _MLP(len(cfg.action_bits) * cfg.action_dim, cfg.mlp_hidden, d, dt, device)
        bound = math.sqrt(1.0 / cfg.num_positions)
        self.pos_emb = nn.Parameter(torch.empty(cfg.num_positions, d, dtype=dt, device=device).uniform_(-bound, bound))
        self.ts_emb = nn.Parameter(torch.empty(cfg.num_time_buckets + 1, d, dtype=dt, device=device).uniform_(-bound, bound))
        self.layers = nn.ModuleList([STULayer(cfg, dt, device) for _ in range(cfg.layers)])
        n_time = 2 * len(cfg.time_periods)
        self.post_linear = _Linear(d + n_time, d, dt, device)
        self.post_norm = _LN(d, dt, device, eps=1e-5)
        self.item_mlp = _MLP(cfg.emb_dim, d, d, dt, device)
        self.head1 = _Linear(d, d, dt, device)
        self.head_norm = _LN(d, dt, device, swish=True)
        self.head2 = _Linear(d, cfg.n_tasks, dt, device)

    # ------------------------------------------------------------------ pieces
    def position_indices(self, offsets, num_targets, total: int):
        """Position index (history counted backwards from the first target, all targets share one
        index) and sqrt time bucket of every token; padding rows get index 0."""
        dev = offsets.device
        lens = (offsets[1:] - offsets[:-1]).long()
        B = lens.numel()
        seq = torch.repeat_interleave(torch.arange(B, device=dev), lens, output_size=total)
        col = torch.arange(seq.numel(), device=dev) - offsets[:-1].long()[seq]
        high = (lens - num_targets.long())[seq]
        C = self.cfg.contextual
        idx = (high - torch.minimum(col, high) + C).clamp(max=self.cfg.num_positions - 1)
        if C > 0:
            idx = torch.where(col < C, col, idx)
        return seq, col, idx

    def time_buckets(self, timestamps, offsets, seq):
        last = timestamps[(offsets[1:].long() - 1).clamp(min=0)][seq]
        delta = (last - timestamps).float().clamp(min=1e-6) / 60.0
        return torch.sqrt(delta).long().clamp(0, self.cfg.num_time_buckets)

    def time_features(self, ts):
        feats = []
        for period, units in self.cfg.time_periods:
            phase = (torch.floor(ts.float() / period) % units) / units * 2 * 3.14
            feats += [torch.cos(phase), torch.sin(phase)]
        return torch.stack(feats, dim=-1)

    # ------------------------------------------------------------------ forward
    def forward(self, batch: dict, item_emb: torch.Tensor):
        cfg = self.cfg
        dt = cfg.torch_dtype()
        offsets, num_targets = batch["offsets"], batch["num_targets"]
        total = int(batch["total"]) if "total" in batch else int(offsets[-1])   # host-known token count
        rows = item_emb.shape[0]
        ts, actions = batch["timestamps"], batch["actions"]
        seq, col, pos_idx = self.position_indices(offsets, num_targets, total)
        lens = (offsets[1:] - offsets[:-1]).long()
        is_target = col >= (lens - num_targets.long())[seq]

        def pad(t):                                     # [L, ...] -> [rows, ...]
            if t.shape[0] == rows:
                return t
            out = torch.zeros((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            out[:t.shape[0]] = t
            return out

        x = self.content_mlp(item_emb.to(dt), cfg.precision)
        x = x + self.action_mlp(pad(self.action_enc(actions, is_target)).to(dt), cfg.precision)
        bucket = self.time_buckets(ts, offsets, seq)
        x = x * math.sqrt(cfg.dim) + pad(self.pos_emb[pos_idx] + self.ts_emb[bucket]).to(dt)
        if cfg.input_dropout > 0 and self.training:
            x = TF.dropout(x, cfg.input_dropout)
        x = x.contiguous()
        for layer in self.layers:
            x = layer(x, offsets, num_targets, rows)
        # candidate (target) rows only
        tgt_rows = torch.nonzero(is_target, as_tuple=False)[:, 0]
        user = x[tgt_rows]
        user = self.post_norm(self.post_linear(torch.cat([user, self.time_features(ts[tgt_rows]).to(dt)], dim=1)))
        item = self.item_mlp(item_emb[tgt_rows].to(dt))
        logits = self.head2(self.head_norm(self.head1(user * item)))          # [targets, n_tasks]
        labels = ((actions[tgt_rows] & cfg.task_weight_bit) > 0).float()
        weights = torch.ones_like(labels)
        per = TF.binary_cross_entropy_with_logits(logits[:, 0].float(), labels, reduction="none") * weights
        loss = per.sum() / weights.sum().clamp(min=1.0) * cfg.causal_multitask_weight
        return loss, torch.sigmoid(logits[:, 0].float()).detach(), labels

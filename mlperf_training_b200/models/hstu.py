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
    # multitask head: ((name, action bit, "binary" | "regression"), ...); empty = one binary task on task_weight_bit
    tasks: tuple = ()
    contextual_dim: int = 0            # width of the contextual feature embeddings (0 = emb_dim)
    extra_features: int = 0            # additional per-token embedding features (artist, album, ...) of width emb_dim
    causal_multitask_weight: float = 0.2
    time_periods: tuple = ((3600.0, 24), (86400.0, 7))   # (period seconds, units): hour of day, day of week
    targets_only_last: bool = True
    dtype: str = "bf16"
    precision: str = "bf16"
    attn_precision: str = "bf16"       # "fp8": attention forward on per-tensor e4m3 Q, K, V (head dim 128, GPU)
    # stochastic depth: in training every layer is skipped (identity) with this probability, decided per forward from a
    # counter-seeded generator that leaves the global RNG untouched (generative_recommenders/modules/dynamic_stu.py:118-196)
    sd_ratio: float = 0.0
    sd_seed: int = 0
    # recent-window layers: the last `recent_window_layers` layers see, per sample, only the contextual tokens, the most
    # recent `recent_window` history tokens and the targets; older tokens bypass them unchanged (dynamic_stu.py:207-303)
    recent_window: int = 0
    recent_window_layers: int = 0
    postprocessor: str = "timestamp_ln"   # "timestamp_ln" | "ln" | "l2" (modules/postprocessors.py)
    # "sum": one token per event, content + action branches added.  "interleave": every history event becomes a content
    # token followed by an action token, a target stays one content token (modules/contextual_interleave_preprocessor.py)
    preprocessor: str = "sum"
    # "simple": the content / action MLPs are plain MLPs.  "parameterized": their weight matrix and bias are generated per
    # sample from the contextual features (modules/contextualize_mlps.py: ParameterizedContextualizedMLP)
    contextualized_mlp: str = "simple"
    pmlp_contextual_dropout: float = 0.0

    def attn_len(self) -> int:
        """The sequence length the attention normalises by (and sizes its tiles for)."""
        return (2 if self.preprocessor == "interleave" else 1) * self.max_seq_len + self.contextual

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


class _ParameterizedMLP(nn.Module):
    """A linear map whose ``[n_in, n_out]`` matrix and bias are functions of the sample's contextual features:
    ``shared = Linear(ctx)``; ``W_b = LayerNorm_{in,out}(Linear(shared))``; ``bias_b = Linear(SwishLN(Linear(shared)))``;
    every token of sample ``b`` gets ``x W_b + bias_b``
    (generative_recommenders/modules/contextualize_mlps.py:79-141).  The per-sample products run as one batched
    matmul over the padded ``[B, N, n_in]`` view of the jagged tokens."""

    def __init__(self, ctx_flat, n_in, hidden, n_out, dtype, device):
        super().__init__()
        self.n_in, self.n_out = n_in, n_out
        self.compress = _Linear(ctx_flat, hidden, dtype, device)
        self.raw = _Linear(hidden, n_in * n_out, dtype, device)
        self.norm_w = nn.Parameter(torch.ones(n_in, n_out, dtype=dtype, device=device))
        self.norm_b = nn.Parameter(torch.zeros(n_in, n_out, dtype=dtype, device=device))
        self.res1 = _Linear(hidden, hidden, dtype, device)
        self.res_n = _LN(hidden, dtype, device, swish=True)
        self.res2 = _Linear(hidden, n_out, dtype, device)

    def forward(self, x, seq, col, n_samples: int, max_len: int, ctx_flat):
        """``x [rows, n_in]`` (the first ``seq.numel()`` rows are tokens), ``seq`` / ``col``: sample and position of every
        token, ``ctx_flat [B, ctx_flat]``.  Returns ``[rows, n_out]`` (padding rows zero)."""
        shared = self.compress(ctx_flat.to(x.dtype))
        w = TF.layer_norm(self.raw(shared).float().view(n_samples, self.n_in, self.n_out), (self.n_in, self.n_out),
                          self.norm_w.float(), self.norm_b.float(), 1e-5)
        bias = self.res2(self.res_n(self.res1(shared))).float()
        n = seq.numel()
        dense = torch.zeros((n_samples, max_len, self.n_in), dtype=torch.float32, device=x.device)
        dense = dense.index_put((seq, col), x[:n].float())
        y = torch.baddbmm(bias[:, None, :], dense, w)[seq, col]
        out = torch.zeros((x.shape[0], self.n_out), dtype=x.dtype, device=x.device)
        out[:n] = y.to(x.dtype)
        return out


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


class ContentEncoder(nn.Module):
    """Content embedding of every token as one concatenation: the item embedding, additional per-token content
    features, and "target enrichment" features that exist for candidates only - a history token carries a learned
    dummy row in their place (generative_recommenders/modules/content_encoder.py:24-109).  An alternative to the
    additional-feature branch of the preprocessor for feature sets whose extras are concatenated, not summed."""

    def __init__(self, emb_dim: int, additional: dict | None = None, target_enrich: dict | None = None, dtype=torch.float32,
                 device="cpu"):
        super().__init__()
        self.emb_dim = emb_dim
        self.additional = dict(additional or {})              # feature name -> width
        self.target_enrich = dict(target_enrich or {})
        self.dummy = nn.ParameterDict({n: nn.Parameter(torch.empty(1, w, dtype=dtype, device=device).normal_(0, 0.1))
                                       for n, w in self.target_enrich.items()})

    @property
    def output_dim(self) -> int:
        return self.emb_dim + sum(self.additional.values()) + sum(self.target_enrich.values())

    def forward(self, item_emb: torch.Tensor, payloads: dict, is_target: torch.Tensor) -> torch.Tensor:
        """``item_emb [L, emb_dim]``; ``payloads[name]``: ``[L, w]`` for additional features, ``[n_targets, w]`` (rows of
        the candidates, in token order) for enrichment features; ``is_target [L]`` marks the candidate tokens."""
        parts = [item_emb] + [payloads[n].to(item_emb.dtype) for n in self.additional]
        if self.target_enrich:
            tgt = torch.nonzero(is_target, as_tuple=False)[:, 0]
            for n in self.target_enrich:
                full = self.dummy[n].to(item_emb.dtype).expand(item_emb.shape[0], -1).clone()
                parts.append(full.index_copy(0, tgt, payloads[n].to(item_emb.dtype)))
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)


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

    def forward(self, x, offsets, num_targets, rows: int, max_len: int | None = None):
        """``max_len``: the static length bound N of the attention (its 1 / N factor and grid); default the model's."""
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
        attn = hstu_attention(q, k, v, offsets, max_len or cfg.attn_len(), cfg.d_qk ** -0.5, num_targets,
                              cfg.contextual, precision=cfg.attn_precision, owner=self).reshape(x.shape[0], h * cfg.d_v)
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


    def forward_targets_only(self, x, seq, tgt_rows, n_samples: int, offsets=None):
        """Last-layer form for batches with ONE target per sample: keys and values are computed for every
        row, queries / gates only for the target rows, and the output has one row per target
        (generative_recommenders/modules/stu.py:677-798).  A target sees its sample's whole history and
        itself, so its attention is a per-sample weighted sum over all rows of the sample:
        ``out[b] = sum_l silu(alpha <q_b, k_l>) / N * v_l``.  Equals ``forward`` followed by the selection
        of the target rows."""
        cfg = self.cfg
        h, hv, hq = cfg.heads, cfg.heads * cfg.d_v, cfg.heads * cfg.d_qk
        normed = F.layer_norm(x, self.in_norm_w, self.in_norm_b, 1e-6)
        W, beta = self.uvqk_weight, self.uvqk_beta
        n_rows = seq.numel()
        v = F.linear(normed, W[hv:2 * hv], beta[hv:2 * hv], None, cfg.precision)[:n_rows].unflatten(-1, (h, cfg.d_v))
        k = F.linear(normed, W[2 * hv + hq:], beta[2 * hv + hq:], None, cfg.precision)[:n_rows].unflatten(-1, (h, cfg.d_qk))
        nt = normed[tgt_rows]
        # (a handful of target rows: plain matmuls, far below a tensor-core tile)
        u = TF.silu(nt @ W[:hv].t() + beta[:hv])
        q = (nt @ W[2 * hv:2 * hv + hq].t() + beta[2 * hv:2 * hv + hq]).unflatten(-1, (h, cfg.d_qk))
        N = cfg.attn_len()
        # every sample's query over its own rows (segment-sum backward when the group bounds are given)
        q_rows = q[seq] if offsets is None else F.expand_rows(q.reshape(n_samples, hq), seq, offsets).unflatten(-1, (h, cfg.d_qk))
        score = (q_rows.float() * k.float()).sum(-1) * (cfg.d_qk ** -0.5)             # [rows, h]
        p = TF.silu(score) / N
        attn = torch.zeros((n_samples, h, cfg.d_v), dtype=torch.float32, device=x.device)
        attn.index_add_(0, seq, p[..., None] * v.float())
        attn = attn.reshape(n_samples, hv).to(x.dtype)
        y = u * F.layer_norm(attn, self.out_norm_w, self.out_norm_b, 1e-6)
        cat = torch.cat([u, attn, y], dim=1)
        if cfg.linear_dropout > 0 and self.training:
            cat = TF.dropout(cat, cfg.linear_dropout)
        return x[tgt_rows] + cat @ self.out_weight.t()


class MultitaskHead(nn.Module):
    """``Linear(D -> D) -> SwishLN -> Linear(D -> n_tasks)`` on ``user * item`` and the per-task losses:
    binary tasks ``BCEWithLogits * weight``, regression tasks squared error ``* weight``, each summed over
    the candidates, divided by the clamped weight sum and scaled by ``causal_multitask_weight``
    (generative_recommenders/modules/multitask_module.py:34-295, head built at dlrm_hstu.py:322-326)."""

    def __init__(self, cfg: HSTUConfig, dtype, device):
        super().__init__()
        self.tasks = tuple(cfg.tasks) if cfg.tasks else (("task0", cfg.task_weight_bit, "binary"),)
        d = cfg.dim
        self.l1 = _Linear(d, d, dtype, device)
        self.norm = _LN(d, dtype, device, swish=True)
        self.l2 = _Linear(d, len(self.tasks), dtype, device)
        self.scale = cfg.causal_multitask_weight

    def forward(self, user, item, actions, values=None, weights=None):
        """``actions [T]`` bit masks of the candidates; ``values [T]`` regression targets (watch time ...);
        ``weights [n_tasks, T]`` supervision weights (default 1).  Returns (losses dict, preds, labels, weights)."""
        logits = self.l2(self.norm(self.l1(user * item))).float().t()                 # [n_tasks, T]
        T = logits.shape[1]
        labels, preds, losses = [], [], {}
        w = torch.ones_like(logits) if weights is None else weights.float()
        for i, (name, bit, kind) in enumerate(self.tasks):
            if kind == "regression":
                lab = values.float() if values is not None else torch.zeros(T, device=logits.device)
                per = (logits[i] - lab) ** 2
                preds.append(logits[i])
            else:
                lab = ((actions & int(bit)) > 0).float()
                per = TF.binary_cross_entropy_with_logits(logits[i], lab, reduction="none")
                preds.append(torch.sigmoid(logits[i]))
            labels.append(lab)
            losses[name] = (per * w[i]).sum() / w[i].sum().clamp(min=1.0) * self.scale
        return losses, torch.stack(preds).detach(), torch.stack(labels), w


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
        self.item_mlp = _MLP(cfg.emb_dim * (1 + cfg.extra_features), d, d, dt, device)
        self.head = MultitaskHead(cfg, dt, device)
        self._sd_iter = 0                # training forwards seen: seeds the stochastic-depth draws (kept in the state dict)
        if cfg.preprocessor not in ("sum", "interleave") or cfg.contextualized_mlp not in ("simple", "parameterized"):
            raise ValueError("preprocessor: 'sum' | 'interleave'; contextualized_mlp: 'simple' | 'parameterized'")
        if cfg.contextualized_mlp == "parameterized":
            if cfg.contextual <= 0:
                raise ValueError("parameterized content / action MLPs are generated from the contextual features: contextual > 0")
            flat = cfg.contextual * (cfg.contextual_dim or cfg.emb_dim)
            self.content_mlp = _ParameterizedMLP(flat, cfg.emb_dim, cfg.mlp_hidden, d, dt, device)
            self.action_mlp = _ParameterizedMLP(flat, len(cfg.action_bits) * cfg.action_dim, cfg.mlp_hidden, d, dt, device)
        # additional-feature branch of the preprocessor: MLP(cat(extra embeddings)) added to the content branch
        self.extra_mlp = _MLP(cfg.emb_dim * cfg.extra_features, cfg.mlp_hidden, d, dt, device) if cfg.extra_features else None
        # contextual tokens: one [ctx_dim, D] matrix and bias per contextual feature (a batched linear)
        if cfg.contextual > 0:
            cd = cfg.contextual_dim or cfg.emb_dim
            std = math.sqrt(2.0 / (cd + d))
            self.ctx_weight = nn.Parameter(torch.empty(cfg.contextual, cd, d, dtype=dt, device=device).normal_(0, std))
            self.ctx_bias = nn.Parameter(torch.zeros(cfg.contextual, d, dtype=dt, device=device))

    # ------------------------------------------------------------------ dynamic layers
    def get_extra_state(self):
        """What a checkpoint needs beside the parameters: the stochastic-depth counter and the per-tensor FP8 scale
        state of every linear and attention site (a frozen calibration must not start over after a resume; the
        reference registers these buffers on the layer for the same reason, modules/stu.py:317-328)."""
        sites = {}
        for n, p in self.named_parameters():
            st = getattr(p, "_fp8_sites", None)
            if st:
                sites[n] = {k: v.state_dict() for k, v in st.items()}
        attn = {n: [s.state_dict() for s in m._attn_fp8_sites] for n, m in self.named_modules()
                if getattr(m, "_attn_fp8_sites", None) is not None}
        return {"sd_iter": self._sd_iter, "fp8_sites": sites, "fp8_attn_sites": attn}

    def set_extra_state(self, state):
        state = state or {}
        self._sd_iter = int(state.get("sd_iter", 0))
        if state.get("fp8_sites") or state.get("fp8_attn_sites"):
            from ..ops import fp8 as F8
            from ..ops.linear import _site
            params, mods = dict(self.named_parameters()), dict(self.named_modules())
            for n, per in (state.get("fp8_sites") or {}).items():
                if n in params:
                    for name, sd in per.items():
                        _site(params[n], name, sd["fmt"]).load_state_dict(sd)
            for n, lst in (state.get("fp8_attn_sites") or {}).items():
                if n in mods:
                    dev = next(self.parameters()).device
                    sites = tuple(F8.DelayedScale(sd["fmt"], dev) for sd in lst)
                    for s_, sd in zip(sites, lst):
                        s_.load_state_dict(sd)
                    mods[n]._attn_fp8_sites = sites

    def skipped_layers(self, it: int) -> list:
        """Layers that stochastic depth turns into the identity in training forward number ``it``."""
        cfg = self.cfg
        if cfg.sd_ratio <= 0:
            return []
        out = []
        for i in range(cfg.layers):
            g = torch.Generator().manual_seed(cfg.sd_seed + 1000003 * i + it)
            if float(torch.rand(1, generator=g)) <= cfg.sd_ratio:
                out.append(i)
        return out

    def _recent_window_layer(self, layer, x, offsets, num_targets, seq, col, total: int, max_targets: int):
        """Run ``layer`` on the contextual tokens, the last ``recent_window`` history tokens and the targets of every
        sample; the older tokens keep their value.  Sizes are static bounds, so nothing is read back to the host."""
        cfg = self.cfg
        C, W = cfg.contextual, cfg.recent_window
        B = offsets.numel() - 1
        lens = (offsets[1:] - offsets[:-1]).long()
        prefix = (lens - W - num_targets.long() - C).clamp(min=0)         # oldest history tokens: bypass
        keep = (col < C) | (col >= (C + prefix)[seq])
        rows2 = min(x.shape[0], (B * (W + C + max_targets) + 127) // 128 * 128)
        pos2 = torch.cumsum(keep.long(), 0) - 1
        idx = torch.where(keep, pos2, torch.full_like(pos2, rows2))        # dropped tokens land in a spare row
        x2 = torch.zeros((rows2 + 1, x.shape[1]), dtype=x.dtype, device=x.device).index_copy(0, idx, x[:total])[:rows2]
        lens2 = lens - prefix
        offsets2 = torch.zeros_like(offsets)
        offsets2[1:] = torch.cumsum(lens2, 0).to(offsets.dtype)
        n2 = min(cfg.attn_len(), W + C + max_targets)
        y2 = layer(x2.contiguous(), offsets2, num_targets, rows2, max_len=n2)
        y2 = torch.cat([y2, y2.new_zeros((1, y2.shape[1]))], dim=0)
        out = torch.where(keep[:, None], y2[idx], x[:total])
        if x.shape[0] > total:
            out = torch.cat([out, x[total:]], dim=0)
        return out

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
    def _token_layout(self, batch: dict):
        """Per-token sample index, position inside the sample and target flag, from the batch alone."""
        offsets0, num_targets = batch["offsets"], batch["num_targets"]
        total0 = int(batch["total"]) if "total" in batch else int(offsets0[-1])
        B = offsets0.numel() - 1
        dev = offsets0.device
        lens0 = (offsets0[1:] - offsets0[:-1]).long()
        seq0 = torch.repeat_interleave(torch.arange(B, device=dev), lens0, output_size=total0)
        col0 = torch.arange(total0, device=dev) - offsets0[:-1].long()[seq0]
        is_target0 = col0 >= (lens0 - num_targets.long())[seq0]
        return total0, lens0, seq0, col0, is_target0

    @staticmethod
    def interleave_layout(lens0, num_targets, seq0, col0, is_target0):
        """Where the tokens of the interleaved sequence go: history event ``i`` of a sample becomes rows ``2 i``
        (content) and ``2 i + 1`` (action) of the sample, target ``j`` row ``2 * history + j``.  Returns
        ``(offsets [B + 1], lengths [B], content row of every token, indices of the history tokens, their action rows)``."""
        hist = lens0 - num_targets.long()
        lens_i = 2 * hist + num_targets.long()
        offsets_i = torch.zeros(lens0.numel() + 1, dtype=torch.long, device=lens0.device)
        offsets_i[1:] = torch.cumsum(lens_i, 0)
        base = offsets_i[:-1][seq0]
        dst_c = torch.where(is_target0, base + hist[seq0] + col0, base + 2 * col0)
        h_rows = torch.nonzero(~is_target0, as_tuple=False)[:, 0]
        return offsets_i, lens_i, dst_c, h_rows, dst_c[h_rows] + 1

    def action_branch(self, batch: dict, rows: int) -> torch.Tensor:
        """The action branch of the preprocessor (action encoder + its MLP), ``[rows, dim]``.  It reads the batch
        only - no embedding - so a trainer may issue it before the embedding rows have arrived and pass the
        result to ``forward(action_out=...)``: it then runs under the lookup's all-to-all instead of behind it
        (generative_recommenders/modules/action_prefill.py:1-80; the sum it enters is formed in the same order,
        so the result is bit-identical)."""
        cfg = self.cfg
        dt = cfg.torch_dtype()
        if cfg.contextualized_mlp != "simple":
            raise ValueError("the action branch reads the contextual embeddings with a parameterized MLP: it cannot run ahead of the lookup")
        _, _, _, _, is_target0 = self._token_layout(batch)
        enc = self.action_enc(batch["actions"], is_target0)
        if enc.shape[0] != rows:
            padded = torch.zeros((rows,) + tuple(enc.shape[1:]), dtype=enc.dtype, device=enc.device)
            padded[:enc.shape[0]] = enc
            enc = padded
        return self.action_mlp(enc.to(dt), cfg.precision)

    def forward(self, batch: dict, item_emb: torch.Tensor, extra_emb: torch.Tensor | None = None,
                contextual_emb: torch.Tensor | None = None, return_all: bool = False,
                action_out: torch.Tensor | None = None):
        """``extra_emb [rows, extra_features * emb_dim]``: the additional per-token features;
        ``contextual_emb [B, contextual, ctx_dim]``: the per-sample contextual features (user id, crosses).
        ``return_all``: also return the per-task losses, predictions ``[n_tasks, T]``, labels and weights.
        ``action_out``: the result of ``action_branch`` issued earlier."""
        cfg = self.cfg
        dt = cfg.torch_dtype()
        C = cfg.contextual
        offsets0, num_targets = batch["offsets"], batch["num_targets"]
        total0 = int(batch["total"]) if "total" in batch else int(offsets0[-1])   # host-known token count
        rows0 = item_emb.shape[0]
        B = offsets0.numel() - 1
        ts0, actions0 = batch["timestamps"], batch["actions"]
        dev = offsets0.device
        lens0 = (offsets0[1:] - offsets0[:-1]).long()
        seq0 = torch.repeat_interleave(torch.arange(B, device=dev), lens0, output_size=total0)
        col0 = torch.arange(total0, device=dev) - offsets0[:-1].long()[seq0]
        is_target0 = col0 >= (lens0 - num_targets.long())[seq0]

        def pad(t, rows):                               # [L, ...] -> [rows, ...]
            if t.shape[0] == rows:
                return t
            out = torch.zeros((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            out[:t.shape[0]] = t
            return out

        # ---- preprocessor: content (+ additional features) and action branches, on the tokens as they came
        if cfg.contextualized_mlp == "parameterized":
            if contextual_emb is None:
                raise ValueError("parameterized MLPs need contextual_emb")
            flat = contextual_emb.reshape(B, -1).to(dt)
            if cfg.pmlp_contextual_dropout > 0 and self.training:
                flat = TF.dropout(flat, cfg.pmlp_contextual_dropout)
            x = self.content_mlp(item_emb.to(dt), seq0, col0, B, cfg.max_seq_len, flat)
            act = self.action_mlp(pad(self.action_enc(actions0, is_target0), rows0).to(dt), seq0, col0, B, cfg.max_seq_len, flat)
        else:
            x = self.content_mlp(item_emb.to(dt), cfg.precision)
            act = (action_out if action_out is not None
                   else self.action_mlp(pad(self.action_enc(actions0, is_target0), rows0).to(dt), cfg.precision))
        if self.extra_mlp is not None:
            if extra_emb is None:
                raise ValueError("the model was built with extra_features: pass extra_emb")
            x = x + self.extra_mlp(extra_emb.to(dt), cfg.precision)
        if cfg.preprocessor == "interleave":
            # history event i of a sample -> rows 2 i (content) and 2 i + 1 (action); target j -> row 2 * history + j
            n_tgt = int(batch["total_targets"]) if "total_targets" in batch else \
                (B if int(batch.get("max_targets", 0)) == 1 else int(num_targets.sum()))
            offsets_i, lens_i, dst_c, h_rows, dst_a = self.interleave_layout(lens0, num_targets, seq0, col0, is_target0)
            total_i = 2 * total0 - n_tgt
            rows_i = (total_i + 127) // 128 * 128
            merged = torch.zeros((rows_i, cfg.dim), dtype=dt, device=dev).index_copy(0, dst_c, x[:total0])
            ts_i = torch.zeros(total_i, dtype=ts0.dtype, device=dev).index_copy(0, dst_c, ts0[:total0])
            x = merged.index_copy(0, dst_a, act[h_rows])
            ts0_l = ts_i.index_copy(0, dst_a, ts0[h_rows])
            # from here on the interleaved tokens are "the tokens as they came"
            offsets_l, total_l, rows_l = offsets_i.to(offsets0.dtype), total_i, rows_i
            seq_l = torch.repeat_interleave(torch.arange(B, device=dev), lens_i, output_size=total_i)
            col_l = torch.arange(total_i, device=dev) - offsets_i[:-1][seq_l]
        else:
            x = x + act
            offsets_l, total_l, rows_l, ts0_l, seq_l, col_l = offsets0, total0, rows0, ts0, seq0, col0
        # ---- contextual tokens in front of every sequence
        if C > 0:
            if contextual_emb is None:
                raise ValueError("the model was built with contextual tokens: pass contextual_emb")
            ctx = torch.baddbmm(self.ctx_bias[:, None, :].float(), contextual_emb.to(dt).float().transpose(0, 1),
                                self.ctx_weight.float()).transpose(0, 1).to(dt)              # [B, C, D]
            offsets = (offsets_l.long() + C * torch.arange(B + 1, device=dev)).to(offsets0.dtype)
            total = total_l + B * C
            rows = (total + 127) // 128 * 128
            dst_tok = offsets[:-1].long()[seq_l] + C + col_l
            dst_ctx = (offsets[:-1].long()[:, None] + torch.arange(C, device=dev)[None]).reshape(-1)
            merged = torch.zeros((rows, cfg.dim), dtype=dt, device=dev)
            merged = merged.index_copy(0, dst_tok, x[:total_l]).index_copy(0, dst_ctx, ctx.reshape(B * C, cfg.dim))
            ts = torch.zeros(total, dtype=ts0.dtype, device=dev).index_copy(0, dst_tok, ts0_l[:total_l])
            x = merged
        else:
            offsets, total, rows, ts = offsets_l, total_l, rows_l, ts0_l
        seq, col, pos_idx = self.position_indices(offsets, num_targets, total)
        lens = (offsets[1:] - offsets[:-1]).long()
        is_target = col >= (lens - num_targets.long())[seq]
        bucket = self.time_buckets(ts, offsets, seq)
        # position and time-bucket rows through the gather / scatter-add kernels (advanced indexing would sort the
        # hundred thousand indices again in backward: two launches of ~2.5 ms each at the benchmark size)
        x = x * math.sqrt(cfg.dim) + pad(F.embedding(pos_idx, self.pos_emb) + F.embedding(bucket, self.ts_emb), rows).to(dt)
        if cfg.input_dropout > 0 and self.training:
            x = TF.dropout(x, cfg.input_dropout)
        x = x.contiguous()
        one_target = int(batch.get("max_targets", 0)) == 1
        if one_target:
            # one candidate per sample, known on the host: the candidate is each sequence's last row (no device read)
            tgt_rows, tgt_rows0 = offsets[1:].long() - 1, offsets0[1:].long() - 1
        else:
            tgt_rows = torch.nonzero(is_target, as_tuple=False)[:, 0]
            tgt_rows0 = torch.nonzero(is_target0, as_tuple=False)[:, 0]
        last = len(self.layers) - 1
        skipped = []
        if self.training and cfg.sd_ratio > 0:
            skipped = self.skipped_layers(self._sd_iter)
            self._sd_iter += 1
        first_windowed = len(self.layers) - cfg.recent_window_layers if cfg.recent_window > 0 else len(self.layers)
        max_t = int(batch.get("max_targets", 0)) or int(num_targets.max())
        user = None
        for i, layer in enumerate(self.layers):
            if i in skipped:
                continue                                                     # stochastic depth: identity this time
            if i >= first_windowed:
                x = self._recent_window_layer(layer, x, offsets, num_targets, seq, col, total, max_t)
                continue
            if i == last and cfg.targets_only_last and one_target:
                user = layer.forward_targets_only(x, seq, tgt_rows, B, offsets)   # candidate rows only, no split afterwards
                break
            x = layer(x, offsets, num_targets, rows)
        if user is None:
            user = x[tgt_rows]
        if cfg.postprocessor == "timestamp_ln":
            user = self.post_norm(self.post_linear(torch.cat([user, self.time_features(ts[tgt_rows]).to(dt)], dim=1)))
        elif cfg.postprocessor == "ln":
            user = self.post_norm(user)
        elif cfg.postprocessor == "l2":
            user = (user.float() / user.float().norm(dim=-1, keepdim=True).clamp(min=1e-6)).to(dt)
        else:
            raise ValueError(f"unknown postprocessor '{cfg.postprocessor}'")
        cand = item_emb[tgt_rows0] if extra_emb is None else torch.cat([item_emb[tgt_rows0], extra_emb[tgt_rows0]], dim=1)
        item = self.item_mlp(cand.to(dt))
        losses, preds, labels, weights = self.head(user, item, actions0[tgt_rows0], batch.get("values"), batch.get("weights"))
        loss = sum(losses.values())
        if return_all:
            return loss, losses, preds, labels, weights
        return loss, preds[0], labels[0]

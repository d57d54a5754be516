"""Megatron / NeMo ``torch_dist`` distributed-checkpoint compatibility for the GPT family.

A Megatron-Bridge checkpoint directory looks like
``iter_0000000/{__0_0.distcp, __0_1.distcp, common.pt, .metadata, metadata.json, run_config.yaml}``
plus ``latest_checkpointed_iteration.txt`` next to it (llama2_sft/primus/README.md:53-76); the SFT
workload loads such a base checkpoint with ``finetune=True, load_optim=False, load_rng=False``
(llama2_sft/primus/src/llama2_custom.py:711-725).  This module

* maps parameter names between this package's ``GPT`` and Megatron-Core's ``GPTModel`` and converts
  the fused-QKV layout (Megatron interleaves per KV group: ``[q_0 .. q_{g-1}, k, v]`` for each
  group; here all query heads come first, then all keys, then all values);
* writes / reads the ``.distcp`` shards and ``.metadata`` through ``torch.distributed.checkpoint``
  with one full-shape entry per Megatron key.  Under tensor parallelism a rank reads a key at its
  full shape (a few keys at a time), converts the fused-QKV layout on the full tensor and keeps its
  own slice; on save the slices are gathered over the tensor-parallel group first, so the file holds
  the same unsharded tensors whatever the parallel layout of the writer;
* writes ``common.pt``, ``metadata.json`` and ``latest_checkpointed_iteration.txt``.
"""
from __future__ import annotations

import json
import re
from pathlib import Path

import torch
import torch.distributed.checkpoint as dcp

from ..models.gpt import GPT, GPTConfig, shard_of

_LAYER = re.compile(r"blocks\.(\d+)\.(.+)")

_BLOCK_MAP = {
    "attn_norm": "self_attention.linear_qkv.layer_norm_weight",
    "w_qkv": "self_attention.linear_qkv.weight",
    "w_proj": "self_attention.linear_proj.weight",
    "sink": "self_attention.core_attention.softmax_offset",
    "mlp_norm": "mlp.linear_fc1.layer_norm_weight",
    "mlp.w_gate_up": "mlp.linear_fc1.weight",
    "mlp.w_down": "mlp.linear_fc2.weight",
    "mlp.router": "mlp.router.weight",
    "mlp.w1": "mlp.experts.linear_fc1.weight",
    "mlp.w2": "mlp.experts.linear_fc2.weight",
    "lora_qkv.a": "self_attention.linear_qkv.adapter.linear_in.weight",
    "lora_qkv.b": "self_attention.linear_qkv.adapter.linear_out.weight",
    "lora_proj.a": "self_attention.linear_proj.adapter.linear_in.weight",
    "lora_proj.b": "self_attention.linear_proj.adapter.linear_out.weight",
}
_TOP_MAP = {"embed": "embedding.word_embeddings.weight", "final_norm": "decoder.final_layernorm.weight",
            "lm_head": "output_layer.weight"}


def megatron_name(name: str, moe_pre_norm: bool = False) -> str:
    if name in _TOP_MAP:
        return _TOP_MAP[name]
    m = _LAYER.match(name)
    if not m:
        raise KeyError(f"no Megatron name for parameter '{name}'")
    layer, rest = m.group(1), m.group(2)
    if rest == "mlp_norm" and moe_pre_norm:
        return f"decoder.layers.{layer}.pre_mlp_layernorm.weight"
    if rest not in _BLOCK_MAP:
        raise KeyError(f"no Megatron name for parameter '{name}'")
    return f"decoder.layers.{layer}.{_BLOCK_MAP[rest]}"


def local_name(meg: str) -> str:
    for k, v in _TOP_MAP.items():
        if v == meg:
            return k
    m = re.match(r"decoder\.layers\.(\d+)\.(.+)", meg)
    if not m:
        raise KeyError(meg)
    if m.group(2) == "pre_mlp_layernorm.weight":
        return f"blocks.{m.group(1)}.mlp_norm"
    for k, v in _BLOCK_MAP.items():
        if v == m.group(2):
            return f"blocks.{m.group(1)}.{k}"
    raise KeyError(meg)


def qkv_to_megatron(w: torch.Tensor, n_heads: int, n_kv: int, hd: int) -> torch.Tensor:
    """``[q_all | k_all | v_all]`` rows -> Megatron's per-group interleave."""
    g = n_heads // n_kv
    rest = w.shape[1:]
    q = w[: n_heads * hd].reshape(n_kv, g * hd, *rest)
    k = w[n_heads * hd:(n_heads + n_kv) * hd].reshape(n_kv, hd, *rest)
    v = w[(n_heads + n_kv) * hd:].reshape(n_kv, hd, *rest)
    return torch.cat([q, k, v], dim=1).reshape(-1, *rest)


def qkv_from_megatron(w: torch.Tensor, n_heads: int, n_kv: int, hd: int) -> torch.Tensor:
    g = n_heads // n_kv
    rest = w.shape[1:]
    x = w.reshape(n_kv, (g + 2) * hd, *rest)
    q = x[:, : g * hd].reshape(n_heads * hd, *rest)
    k = x[:, g * hd:(g + 1) * hd].reshape(n_kv * hd, *rest)
    v = x[:, (g + 1) * hd:].reshape(n_kv * hd, *rest)
    return torch.cat([q, k, v], dim=0)


def _stages_of(model):
    """Pipeline stages inside ``model`` (a stage itself, or a list of them), else None."""
    def is_stage(m):
        return hasattr(m, "layers") and hasattr(m, "stage") and hasattr(m, "n_stages")
    if is_stage(model):
        return [("", model)]
    if isinstance(model, torch.nn.ModuleList) and len(model) and all(is_stage(m) for m in model):
        return [(f"{i}.", m) for i, m in enumerate(model)]
    return None


def model_config_of(model):
    stages = _stages_of(model)
    return model.cfg if stages is None else stages[0][1].cfg


def global_named_parameters(model):
    """``(name, parameter)`` with the names of the unsplit model: a pipeline stage numbers its blocks by
    position inside the stage, a checkpoint by the layer's index in the whole network."""
    stages = _stages_of(model)
    if stages is None:
        yield from model.named_parameters()
        return
    for _, stage in stages:
        for name, p in stage.named_parameters():
            parts = name.split(".")
            if parts[0] == "blocks":
                parts[1] = str(stage.layers[int(parts[1])])
            yield ".".join(parts), p


def full_shape_of(p: torch.Tensor) -> tuple:
    """Shape of the unsharded tensor behind a (possibly tensor-parallel) parameter."""
    shard = getattr(p, "tensor_parallel", None)
    if shard is None:
        ep = getattr(p, "expert_shard", None)
        if ep is not None:                       # stacked experts [E / EP, ...]: a block of the expert dimension
            return (p.shape[0] * ep[0], *p.shape[1:])
        return tuple(p.shape)
    kind, W, _ = shard
    if kind == "cols":
        return (p.shape[0], p.shape[1] * W)
    return (p.shape[0] * W, *p.shape[1:])


def unshard(parts: list[torch.Tensor], kind: str, cfg: GPTConfig) -> torch.Tensor:
    """Inverse of ``models.gpt.shard_of``: the full tensor from the slices of ranks 0..W-1."""
    W = len(parts)
    if kind == "rows":
        return torch.cat(parts, 0)
    if kind == "cols":
        return torch.cat(parts, 1)
    if kind == "rows_2":
        halves = [t.chunk(2, 0) for t in parts]
        return torch.cat([h[0] for h in halves] + [h[1] for h in halves], 0)
    if kind == "qkv":
        hd = cfg.head_dim
        sizes = [cfg.n_heads * hd // W, cfg.n_kv_heads * hd // W, cfg.n_kv_heads * hd // W]
        pieces = [t.split(sizes, 0) for t in parts]
        return torch.cat([pc[i] for i in range(3) for pc in pieces], 0)
    raise ValueError(kind)


def _ep_group_of(model):
    """Process group over which the model's experts are split (None: every rank holds all experts)."""
    for m in model.modules():
        if getattr(m, "ep_group", None) is not None and getattr(m, "ep", 1) > 1:
            return m.ep_group
    return None


def _full_tensor(p: torch.Tensor, cfg: GPTConfig, tp_group, ep_group=None) -> torch.Tensor:
    """The unsharded value of parameter ``p`` (gathered over ``tp_group`` / ``ep_group`` when it is a slice)."""
    shard = getattr(p, "tensor_parallel", None)
    t = p.detach()
    if shard is None:
        ep = getattr(p, "expert_shard", None)
        if ep is None:
            return t
        if ep_group is None or torch.distributed.get_world_size(ep_group) != ep[0]:
            raise ValueError("an expert-parallel parameter needs its expert-parallel group to be gathered")
        parts = [torch.empty_like(t) for _ in range(ep[0])]
        torch.distributed.all_gather(parts, t.contiguous(), group=ep_group)
        return torch.cat(parts, 0)
    kind, W, _ = shard
    if tp_group is None or torch.distributed.get_world_size(tp_group) != W:
        raise ValueError("a tensor-parallel parameter needs its tensor-parallel group to be gathered")
    parts = [torch.empty_like(t) for _ in range(W)]
    torch.distributed.all_gather(parts, t.contiguous(), group=tp_group)
    return unshard(parts, kind, cfg)


def to_megatron_state(model: GPT, tp_group=None) -> dict[str, torch.Tensor]:
    """Megatron-named state with every tensor at its full (unsharded) shape.  Collective over
    ``tp_group`` when the model holds tensor-parallel slices."""
    cfg = model_config_of(model)
    ep_group = _ep_group_of(model) if isinstance(model, torch.nn.Module) else None
    out = {}
    for name, p in global_named_parameters(model):
        t = _full_tensor(p, cfg, tp_group, ep_group)
        if name.endswith("w_qkv") or name.endswith("lora_qkv.b"):
            t = qkv_to_megatron(t, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
        out[megatron_name(name, moe_pre_norm=cfg.n_experts > 0)] = t.contiguous()
    return out


def sharded_megatron_state(model: GPT, tp_group) -> dict:
    """Megatron-named state in which every tensor-parallel parameter is a ``ShardedTensor`` over ``tp_group``: each
    rank contributes only its slice, described by its offsets inside the full tensor, so the checkpoint records
    the sharding (one or two chunks per rank and tensor) instead of a gathered copy, and a run with another
    tensor-parallel degree reads the chunks it needs.  The fused q | k | v weight is stored in Megatron's per-group
    layout, in which a rank's heads are one contiguous row block; the stacked gate | up weight contributes two
    chunks, one inside each half.  Replicated parameters stay plain tensors.  Collective over ``tp_group``."""
    from torch.distributed._shard.sharded_tensor import Shard, ShardMetadata, init_from_local_shards
    cfg = model_config_of(model)
    ep_group = _ep_group_of(model) if isinstance(model, torch.nn.Module) else None
    out = {}
    for name, p in global_named_parameters(model):
        key = megatron_name(name, moe_pre_norm=cfg.n_experts > 0)
        shard = getattr(p, "tensor_parallel", None)
        t = p.detach()
        ep = getattr(p, "expert_shard", None)
        if shard is None and ep is not None and ep_group is not None:
            # stacked experts: this rank's block of the expert dimension, over the expert-parallel group
            n, r = ep
            dev = f"rank:{_global_rank(ep_group, r)}/{'cpu' if t.device.type == 'cpu' else str(t.device)}"
            meta = ShardMetadata(shard_offsets=[r * t.shape[0]] + [0] * (t.dim() - 1), shard_sizes=list(t.shape), placement=dev)
            out[key] = init_from_local_shards([Shard(tensor=t.contiguous(), metadata=meta)], *full_shape_of(p),
                                              process_group=ep_group)
            continue
        if shard is None:
            if name.endswith("w_qkv") or name.endswith("lora_qkv.b"):
                t = qkv_to_megatron(t, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
            out[key] = t.contiguous()
            continue
        kind, W, r = shard
        full = full_shape_of(p)
        if kind == "qkv":
            t = qkv_to_megatron(t, cfg.n_heads // W, cfg.n_kv_heads // W, cfg.head_dim)
        tail = [0] * (t.dim() - 1)
        if kind in ("rows", "qkv"):
            pieces = [(t, [r * t.shape[0]] + tail)]
        elif kind == "cols":
            pieces = [(t, [0, r * t.shape[1]] + tail[1:])]
        elif kind == "rows_2":
            h = t.shape[0] // 2
            pieces = [(t[:h], [r * h] + tail), (t[h:], [full[0] // 2 + r * h] + tail)]
        else:
            raise ValueError(kind)
        dev = f"rank:{_global_rank(tp_group, r)}/{'cpu' if t.device.type == 'cpu' else str(t.device)}"
        shards = [Shard(tensor=x.contiguous(), metadata=ShardMetadata(shard_offsets=list(off), shard_sizes=list(x.shape),
                                                                      placement=dev)) for x, off in pieces]
        out[key] = init_from_local_shards(shards, *full, process_group=tp_group)
    return out


def _global_rank(group, r: int) -> int:
    """Global rank of member ``r`` of ``group`` (a shard's placement names global ranks, also inside a sub-group)."""
    if group is None or group is torch.distributed.group.WORLD:
        return r
    return torch.distributed.get_global_rank(group, r)


def _tp_group_of(model):
    tp = getattr(model, "tp", None)
    return getattr(tp, "group", None) if tp is not None else None


def _load_named(named, state: dict[str, torch.Tensor], cfg: GPTConfig) -> list[str]:
    """Copy the entries of ``state`` (Megatron names, full shapes or this rank's slices) into the
    parameters of ``named``; returns the names without an entry."""
    missing = []
    with torch.no_grad():
        for name, p in named:
            key = megatron_name(name, moe_pre_norm=cfg.n_experts > 0)
            if key not in state:
                missing.append(name)
                continue
            t = state[key]
            if name.endswith("w_qkv") or name.endswith("lora_qkv.b"):
                t = qkv_from_megatron(t, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
            shard = getattr(p, "tensor_parallel", None)
            if shard is not None and tuple(t.shape) == full_shape_of(p):
                t = shard_of(t, shard[0], shard[1], shard[2], cfg)     # the layout conversion ran on the full tensor
            ep = getattr(p, "expert_shard", None)
            if shard is None and ep is not None and tuple(t.shape) == full_shape_of(p):
                t = t.chunk(ep[0], 0)[ep[1]]                           # this rank's experts
            if tuple(t.shape) != tuple(p.shape):
                raise ValueError(f"{key}: checkpoint shape {tuple(t.shape)} vs model {tuple(p.shape)}")
            p.copy_(t.to(p.dtype))
    return missing


def load_megatron_state(model: GPT, state: dict[str, torch.Tensor], strict: bool = True) -> list[str]:
    """Copy a (Megatron-named) state dict into ``model``.  Returns the model parameters that were
    not found (e.g. freshly initialised LoRA adapters when loading a base checkpoint)."""
    missing = _load_named(list(global_named_parameters(model)), state, model_config_of(model))
    if strict and any("lora" not in m for m in missing):
        raise KeyError(f"checkpoint lacks parameters: {[m for m in missing if 'lora' not in m]}")
    return missing


def save_torch_dist(model: GPT, root: str, iteration: int = 0, extra_common: dict | None = None,
                    sharded: bool = True) -> Path:
    """Write ``<root>/iter_<iteration:07d>/`` in the ``torch_dist`` layout.  Collective when a
    process group is initialised (every rank calls it).  Under tensor parallelism every rank writes its own
    slices with their offsets (``sharded``; ``False`` gathers full tensors first)."""
    d = Path(root) / f"iter_{iteration:07d}"
    rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
    if rank == 0:
        d.mkdir(parents=True, exist_ok=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
    tp_group = _tp_group_of(model)
    ep_group = _ep_group_of(model) if isinstance(model, torch.nn.Module) else None
    tp_sharded = sharded and ((tp_group is not None and torch.distributed.get_world_size(tp_group) > 1) or ep_group is not None)
    megatron_state = sharded_megatron_state(model, tp_group) if tp_sharded else to_megatron_state(model, tp_group)
    state = {f"model.{k}": v for k, v in megatron_state.items()}
    dcp.save(state, checkpoint_id=str(d))
    if rank == 0:
        common = {"iteration": iteration, "checkpoint_version": 3.0, "args": None, "model_config": model.cfg.to_dict(),
                  "tensor_parallel_shards": torch.distributed.get_world_size(tp_group) if (tp_sharded and tp_group is not None) else 1,
                  "expert_parallel_shards": torch.distributed.get_world_size(ep_group) if (tp_sharded and ep_group is not None) else 1}
        common.update(extra_common or {})
        torch.save(common, d / "common.pt")
        (d / "metadata.json").write_text(json.dumps({"sharded_backend": "torch_dist", "sharded_backend_version": 1,
                                                      "common_backend": "torch", "common_backend_version": 1}))
        (Path(root) / "latest_checkpointed_iteration.txt").write_text(str(iteration))
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
    return d


def load_torch_dist(model: GPT, root: str, iteration: int | None = None, strict: bool = True) -> dict:
    """Load model weights from a ``torch_dist`` checkpoint (finetune semantics: no optimizer state,
    no RNG).  Architecture fields recorded in ``common.pt`` are asserted against the model."""
    rootp = Path(root)
    if iteration is None:
        f = rootp / "latest_checkpointed_iteration.txt"
        iteration = int(f.read_text().strip()) if f.exists() else 0
    d = rootp / f"iter_{iteration:07d}"
    if not d.exists():
        raise FileNotFoundError(d)
    common = torch.load(d / "common.pt", map_location="cpu", weights_only=False) if (d / "common.pt").exists() else {}
    saved_cfg = common.get("model_config") or {}
    for k in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "vocab_size"):
        if k in saved_cfg and saved_cfg[k] != getattr(model_config_of(model), k):
            raise ValueError(f"checkpoint {k}={saved_cfg[k]} but model has {getattr(model_config_of(model), k)}")
    cfg = model_config_of(model)
    reader = dcp.FileSystemReader(str(d))
    present = set(reader.read_metadata().state_dict_metadata.keys())
    # full-shape destinations, read and consumed a group of keys at a time (a tensor-parallel rank keeps
    # only its slice of each, so the full tensors of the whole model never sit in memory together)
    named = list(global_named_parameters(model))
    sharded = any(getattr(p, "tensor_parallel", None) is not None or getattr(p, "expert_shard", None) is not None for _, p in named)
    per_group = 16 if sharded else len(named)
    missing = []
    for g0 in range(0, len(named), max(per_group, 1)):
        group = named[g0:g0 + per_group]
        want = {}
        for name, p in group:
            key = "model." + megatron_name(name, moe_pre_norm=cfg.n_experts > 0)
            if key in present:
                want[key] = torch.empty(full_shape_of(p), dtype=p.dtype, device="cpu")
        if want:
            dcp.load(want, checkpoint_id=str(d))
        missing += _load_named(group, {k[len("model."):]: v for k, v in want.items()}, cfg)
    if strict and any("lora" not in m for m in missing):
        raise KeyError(f"checkpoint lacks parameters: {[m for m in missing if 'lora' not in m]}")
    return {"iteration": iteration, "missing": missing, "common": common}

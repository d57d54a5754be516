"""MLPerf-style training run for the GPT family (pre-training and LoRA SFT).

``run(exp)`` takes a resolved experiment dictionary and performs one timed run:

    cache_clear / init_start -> build model, engine, data -> load checkpoint (resume or finetune base)
    -> synthetic warm-up with state restoration -> init_stop / run_start (barrier-aligned)
    -> for step: train_step ; train_loss event ; evaluation every ``eval_interval`` steps
       (block_stop, eval_start, eval_accuracy, eval_stop, block_start) ; stop when the evaluation
       loss reaches ``target_eval_loss`` ; checkpoint cadence ; optional fault injection
    -> run_stop{success|aborted}, run_duration, overall_throughput

which is the event sequence of the reference's ``MLPerfMegatronPretrainTrainer``
(primus_mllog/mlperf_pre_training.py:100-241 in the bundled wheel) and of its SFT loop
(llama2_sft/primus/src/llama2_custom.py:1295-1893: evaluation every ``eval_interval`` steps after
skipping the first ``skip_evals`` ones, sticky early exit below the target loss).
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..checkpoint.manager import CheckpointManager, select_checkpoint_reason
from ..data.indexed import GPTSampleDataset, PackedSFTDataset, SyntheticTokens
from ..mllog import core as ml
from ..models.gpt import PRESETS, GPTConfig
from ..parallel.engine import OptimConfig
from .pretrain import PretrainTrainer, TrainConfig
from .warmup import run_synthetic_warmup


@dataclass
class RunConfig:
    benchmark: str = "llama31_8b"
    model: dict = field(default_factory=dict)          # preset name under "preset" + field overrides
    global_batch: int = 32
    micro_batch: int = 1
    train_iters: int = 100
    lr: float = 8e-4
    min_lr_ratio: float = 0.1
    lr_warmup_iters: int = 64
    lr_decay_iters: int = 1_200_000
    weight_decay: float = 0.1
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-5
    use_precision_aware_optimizer: bool = False   # with exp_avg_dtype / exp_avg_sq_dtype bf16: bf16 Adam moments
    exp_avg_dtype: str = "fp32"
    exp_avg_sq_dtype: str = "fp32"
    clip_grad: float = 1.0
    seed: int = 0
    eval_interval: int = 0
    eval_iters: int = 0
    skip_evals: int = 0
    target_eval_loss: float = 0.0
    warmup_train_steps: int = 2
    warmup_eval_steps: int = 0
    data: dict = field(default_factory=lambda: {"kind": "synthetic"})
    eval_data: dict | None = None                       # validation source (same keys as ``data``); synthetic runs may omit it
    checkpoint_dir: str = ""
    checkpoint_every: int = 0
    keep_last: int = 2
    pretrained_checkpoint: str = ""
    log_interval: int = 1
    die_at_step: int = 0                                # fault injection: exit(42) after this step's save
    mllog_file: str = ""
    dp_replicate: int = 1                               # hybrid sharding: copies of each optimizer-state shard
    tensor_parallel: int = 1                            # tensor + sequence parallel size (Megatron layout)
    sequence_parallel: int = 1
    expert_parallel: int = 1                            # ranks an MoE layer's experts are spread over (a divisor of the world)
    moe_dispatch: str = "fused"                         # "fused": peer-memory push / pull kernels (GPUs); "nccl": all-to-all
    pipeline_parallel: int = 1
    virtual_pipeline_parallel: int | None = None        # model chunks per pipeline rank (interleaved 1F1B)
    context_parallel: int = 1
    context_parallel_mode: str = "allgather"            # "allgather" (keys / values of earlier chunks) | "ulysses" (head exchange) | "ring" (zig-zag chunks, p2p ring)
    tp_comm_overlap: str = "fused"                      # "fused": in-kernel all-gather / reduce-scatter; "nccl"
    comm: str = "nccl"                                  # optimizer-step collectives: "nccl" | "fused"
    zero_stage: int = 1                                 # 3: block matrices sharded too (gathered per block, parallel/zero3.py)
    # no loss at the positions whose input token is the end-of-document token (Megatron's ``eod_mask_loss``,
    # small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:86; off for Llama-3.1-8B)
    grad_reduce_in_bf16: bool = False                   # gradients cross the wire in bf16 (library-collective engine)
    eod_mask_loss: bool = False
    eod_token: int = 128001                              # <|end_of_text|> of the Llama-3 tokenizer
    precision_schedule: dict | str | None = None        # ops.recipe.PrecisionSchedule spec (phase switch at a step)
    vanish_at_step: int = 0                             # fault injection: rank ``vanish_rank`` leaves silently before this step
    vanish_rank: int = 1
    heartbeat_timeout_s: float = 0.0                    # > 0: watch the other ranks' heartbeats between steps
    straggler_interval: int = 0                         # > 0: compare mean step time across ranks every N steps
    check_replicas_every: int = 0                       # > 0: compare parameter checksums across replicas every N steps
    async_checkpoint: bool = False                      # write checkpoints on a background thread (single process)
    energy_monitor: bool = False                        # integrate GPU power over the run
    perf_jsonl: str = ""                                # durable per-interval performance lines
    profile_step_start: int = 0
    profile_step_end: int = 0
    profile_dir: str = ""

    @staticmethod
    def from_dict(d: dict) -> "RunConfig":
        known = {f for f in RunConfig.__dataclass_fields__}
        unknown = sorted(k for k in d if k not in known)
        if unknown:
            import warnings
            warnings.warn(f"run configuration: keys without a meaning here are ignored: {unknown}", stacklevel=2)
        return RunConfig(**{k: v for k, v in d.items() if k in known})


def build_model_config(spec: dict) -> GPTConfig:
    spec = dict(spec or {})
    preset = spec.pop("preset", None)
    cfg = PRESETS[preset]() if preset else GPTConfig()
    for k, v in spec.items():
        if not hasattr(cfg, k):
            raise KeyError(f"unknown model field '{k}'")
        if k == "lora_targets" and isinstance(v, list):
            v = tuple(v)
        setattr(cfg, k, v)
    return cfg


def build_data(spec: dict, cfg: GPTConfig, seed: int):
    kind = spec.get("kind", "synthetic")
    if kind == "synthetic":
        return SyntheticTokens(cfg.vocab_size, cfg.seq_len, seed=seed, loss_last=int(spec.get("loss_last", 0)))
    if kind == "indexed":
        return GPTSampleDataset(list(spec["prefixes"]), spec.get("weights"), cfg.seq_len, seed=seed)
    if kind == "packed_sft":
        return PackedSFTDataset(spec["path"], cfg.seq_len, spec.get("metadata"))
    raise ValueError(f"unknown data kind '{kind}'")


def eod_masked(batch, eod_token: int):
    """``(inputs, labels)`` with label -100 wherever the input token is ``eod_token``: the prediction that follows an
    end-of-document token belongs to the next document and carries no loss.  ``batch``: token rows ``[b, S + 1]`` or an
    ``(inputs, labels)`` pair."""
    if isinstance(batch, (tuple, list)):
        x, y = batch[0], batch[1].clone()
    else:
        x, y = batch[:, :-1].contiguous(), batch[:, 1:].clone()
    y[x == eod_token] = -100
    return x, y


def eval_spec(rc: "RunConfig") -> dict:
    """The validation data source of a run.  The reference evaluates on a held-out set
    (``valid_data_path`` c4-validation of the pretraining configs, ``packed_val_data_path`` of the SFT
    recipe: small_llm_pretraining/primus/README.md:97-101, llama2_sft/primus/src/llama2_custom.py:1521);
    a synthetic run draws another stream from another seed; a real-data run must name its validation
    files (``eval_data``, or the shorthands ``valid_prefixes`` / ``valid_path`` inside ``data``), and a
    run with a convergence target refuses to decide it on training samples."""
    if rc.eval_data:
        spec = dict(rc.data)
        spec.update(rc.eval_data)
        return spec
    kind = rc.data.get("kind", "synthetic")
    spec = dict(rc.data)
    if kind == "indexed" and rc.data.get("valid_prefixes"):
        spec["prefixes"], spec["weights"] = list(rc.data["valid_prefixes"]), rc.data.get("valid_weights")
        return spec
    if kind == "packed_sft" and rc.data.get("valid_path"):
        spec["path"], spec["metadata"] = rc.data["valid_path"], rc.data.get("valid_metadata")
        return spec
    if kind != "synthetic" and rc.eval_interval and rc.target_eval_loss > 0:
        raise ValueError(f"data kind '{kind}' with target_eval_loss needs a validation source: set eval_data "
                         "(or data.valid_prefixes / data.valid_path)")
    return spec


def _dist_info():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _optim_shard(trainer, with_params: bool) -> dict:
    state = trainer.engine.optimizer_state()
    if with_params:
        state["stage_param_bufs"] = [b.param_buf.detach().cpu() for b in trainer.engine.buckets]
    return state


def _moment_dtype(rc) -> torch.dtype:
    if not rc.use_precision_aware_optimizer:
        return torch.float32
    kinds = {str(rc.exp_avg_dtype).lower(), str(rc.exp_avg_sq_dtype).lower()}
    if kinds <= {"fp32", "float32"}:
        return torch.float32
    if kinds <= {"bf16", "bfloat16"}:
        return torch.bfloat16
    raise ValueError(f"exp_avg_dtype / exp_avg_sq_dtype {sorted(kinds)}: both moments are kept in one of fp32, bf16")


def run(exp: dict, device: str | None = None, stream=None) -> dict:
    rc = RunConfig.from_dict(exp)
    rank, world = _dist_info()
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    sync = dist.barrier if world > 1 else None
    resume_mgr = CheckpointManager(rc.checkpoint_dir, rank, world, rc.keep_last, sync) if rc.checkpoint_dir else None
    resuming = bool(resume_mgr and resume_mgr.present())
    log = ml.MLLogger(rank=rank, stream=stream or sys.stdout, filename=rc.mllog_file or None, sync=sync,
                      append=resuming)
    if not resuming:
        log.log_init_start()
        log.log_submission(rc.benchmark, platform=f"1xB200x{world}")

    cfg = build_model_config(rc.model)
    pp_size, cp_size = int(rc.pipeline_parallel), int(rc.context_parallel)
    if pp_size > 1 and (int(rc.dp_replicate) > 1 or (cp_size > 1 and int(rc.tensor_parallel) > 1)
                        or world % (pp_size * max(int(rc.tensor_parallel), 1) * max(cp_size, 1))):
        raise NotImplementedError("pipeline stages combine with data parallelism and ONE of tensor / context / expert "
                                  "parallelism here (dp_replicate = 1, world divisible by the product of the sizes)")
    if cp_size > 1 and (int(rc.dp_replicate) > 1 or world % (cp_size * max(int(rc.tensor_parallel), 1))):
        raise NotImplementedError("context parallelism combines with data and tensor parallelism here (dp_replicate = 1, "
                                  "world divisible by context_parallel x tensor_parallel)")
    tp_size = min(int(rc.tensor_parallel), world)
    ep_size = min(int(rc.expert_parallel), world) if cfg.n_experts else 1
    tp_ctx, dp_group, dp_rank, dp_world, rep_group = None, None, rank, world, None
    replicate = max(int(rc.dp_replicate), 1)
    if tp_size > 1 or (replicate > 1 and world > 1):
        from ..parallel.mesh import Mesh, MeshSpec
        mesh = Mesh(MeshSpec(tp=tp_size, pp=pp_size, cp=cp_size if tp_size > 1 else 1, ep=ep_size if (tp_size > 1 and pp_size == 1) else 1,
                             dp_replicate=replicate))
        if replicate > 1:
            rep_group = mesh.group("dp_replicate")
    if tp_size > 1:
        if not int(rc.sequence_parallel) and rank == 0:
            print("[parallel] sequence_parallel: 0 ignored - the tensor-parallel blocks always shard the activations "
                  "between them over the sequence (all-gather -> GEMM, GEMM -> reduce-scatter)", flush=True)
        from ..parallel.tensor import TPContext
        # (stages of a pipeline keep the library collectives: the fused kernels' symmetric buffers are per process group)
        fused_tp = str(rc.tp_comm_overlap).lower() == "fused" and str(device).startswith("cuda") and pp_size == 1
        # low-precision recipes run the frozen linears of the fused tensor-parallel path (the base of a LoRA run) on
        # per-tensor FP8 operands; trainable tensor-parallel linears run the bf16 tcgen05 GEMMs
        tp_prec = "fp8" if (fused_tp and cfg.precision != "bf16") else "bf16"
        tp_ctx = TPContext(mesh.group("tp"), comm="fused" if fused_tp else "nccl", device=device if fused_tp else None,
                           precision=tp_prec)
        dp_rank, dp_world = mesh.index("dp"), mesh.size("dp")
        dp_group = mesh.group("dp_shard") if replicate > 1 else mesh.group("dp")
        if cfg.precision != "bf16":
            cfg.precision = "bf16"       # everything outside the tensor-parallel linears stays bf16
    cp_group = ep_group = edp_group = None
    if ep_size > 1:
        others = (tp_size > 1) + (pp_size > 1) + (cp_size > 1)
        if others > 1 or replicate > 1 or (world // (pp_size * tp_size * cp_size)) % ep_size or cfg.n_experts % ep_size:
            raise NotImplementedError("expert parallelism combines with data parallelism and with ONE of pipeline / tensor / "
                                      "context parallelism here (dp_replicate = 1; data-parallel size and experts divisible by "
                                      "expert_parallel)")
        if cp_size > 1:
            # experts spread over (a block of) the data-parallel ranks that hold the same chunk of the sequences; the copies
            # of an expert - in the other blocks and in the other chunks - sum their gradients
            from ..parallel.mesh import Mesh, MeshSpec
            mesh = Mesh(MeshSpec(cp=cp_size, ep=ep_size))
            ep_group = mesh.group("ep")
            edp_group = mesh.group("edp_cp") if mesh.size("edp_cp") > 1 else None
        elif tp_size > 1:
            # experts spread over (a block of) the data-parallel ranks that share a tensor-parallel index; every
            # tensor-parallel rank routes its own block of token rows through them
            ep_group = mesh.group("ep")
            edp_group = mesh.group("edp") if mesh.size("edp") > 1 else None
        elif pp_size > 1:
            # experts spread over (a block of) the data-parallel replicas of every pipeline stage
            from ..parallel.mesh import Mesh, MeshSpec
            mesh = Mesh(MeshSpec(pp=pp_size, ep=ep_size))
            ep_group = mesh.group("ep")
            edp_group = mesh.group("edp") if mesh.size("edp") > 1 else None
        elif ep_size == world:
            ep_group = dist.group.WORLD
        else:
            from ..parallel.mesh import Mesh, MeshSpec
            ep_mesh = Mesh(MeshSpec(ep=ep_size))
            ep_group, edp_group = ep_mesh.group("ep"), ep_mesh.group("edp")
        fused_ep = str(rc.moe_dispatch).lower() == "fused" and str(device).startswith("cuda") and others == 0
        cfg.ep_comm = "fused" if fused_ep else "nccl"
    if pp_size > 1 and tp_size == 1:
        if ep_size == 1:
            from ..parallel.mesh import Mesh, MeshSpec
            mesh = Mesh(MeshSpec(pp=pp_size, cp=cp_size))
            if cp_size > 1:
                cp_group = mesh.group("cp")
        elif cp_size > 1:
            raise NotImplementedError("pipeline stages take context OR expert parallelism")
        dp_rank, dp_world = mesh.index("dp"), mesh.size("dp")
    elif cp_size > 1:
        if tp_size == 1 and ep_size == 1:
            from ..parallel.mesh import Mesh, MeshSpec
            mesh = Mesh(MeshSpec(cp=cp_size))
        dp_rank, dp_world = mesh.index("dp"), mesh.size("dp")
        cp_group, dp_group = mesh.group("cp"), mesh.group("dp_cp")     # gradients are reduced over data x context
    if rc.global_batch % dp_world:
        raise ValueError("global_batch must be divisible by the data-parallel size")
    local_batch = rc.global_batch // dp_world
    opt = OptimConfig(lr=rc.lr, beta1=rc.adam_beta1, beta2=rc.adam_beta2, eps=rc.adam_eps,
                      weight_decay=rc.weight_decay, clip_grad=rc.clip_grad, moment_dtype=_moment_dtype(rc),
                      reduce_dtype=torch.bfloat16 if rc.grad_reduce_in_bf16 else None)
    tc = TrainConfig(micro_batch=rc.micro_batch, local_batch=local_batch, warmup_steps=rc.lr_warmup_iters,
                     decay_steps=rc.lr_decay_iters, min_lr_ratio=rc.min_lr_ratio, seed=rc.seed, comm=rc.comm,
                     zero_stage=int(rc.zero_stage))
    if tp_size == 1 and replicate > 1 and world > 1:
        dp_group = mesh.group("dp_shard")
    if pp_size > 1:
        from .pipeline_train import PipelineTrainer
        trainer = PipelineTrainer(cfg, opt, tc, device, mesh, virtual_stages=rc.virtual_pipeline_parallel or 1,
                                  freeze_base=cfg.lora_rank > 0, tp=tp_ctx, ep_group=ep_group, expert_dp_group=edp_group,
                                  cp_group=cp_group, cp_mode=rc.context_parallel_mode)
    else:
        trainer = PretrainTrainer(cfg, opt, tc, device, group=dp_group, ep_group=ep_group, tp=tp_ctx,
                                  freeze_base=cfg.lora_rank > 0, replicate_group=rep_group, cp_group=cp_group,
                                  cp_mode=rc.context_parallel_mode, expert_dp_group=edp_group)
    if os.environ.get("INIT_CHECKSUM", "0") == "1":
        from ..utils.metrics import model_fingerprint
        digest, _ = model_fingerprint(trainer.model)
        if rank == 0:
            print(f"[init] model fingerprint {digest}", flush=True)
    data = build_data(rc.data, cfg, rc.seed)
    eval_data = build_data(eval_spec(rc), cfg, rc.seed + 7919)

    def host_batch(ds, i):
        """One step's batch for this data-parallel rank: tokens ``[b, S+1]``, or (tokens, labels)."""
        b = ds.batch(i, dp_rank, dp_world, local_batch)
        if not isinstance(b, (tuple, list)) and getattr(ds, "loss_last", 0) > 0:
            b = (b[:, :-1].contiguous(), ds.labels(b))
        if rc.eod_mask_loss:
            b = eod_masked(b, int(rc.eod_token))
        return b

    # pipeline stages, expert shards and tensor-parallel slices differ per rank: those parameters travel
    # with the rank's own optimizer shard instead of rank 0's dense file
    per_rank_params = pp_size > 1 or ep_size > 1 or tp_size > 1 or (int(rc.zero_stage) == 3 and world > 1)
    if rc.pretrained_checkpoint and (not resuming or cfg.lora_rank > 0):
        # a LoRA run checkpoints its adapters only (the engine owns the trainable parameters), so a
        # resumed run needs the frozen base from the pretrained checkpoint again
        from ..checkpoint.megatron import load_torch_dist
        load_torch_dist(trainer.model, rc.pretrained_checkpoint, strict=True)
    start_step, resumed_evals = 0, 0
    if resuming:
        ck = resume_mgr.load()
        # pipeline stages and expert shards differ per rank: their parameters travel with the rank's optimizer shard
        bufs = ck["optim"].get("stage_param_bufs") if (per_rank_params and ck["optim"] is not None) else ck["dense"]["param_bufs"]
        written_by = int(ck["meta"].get("world", world))
        if written_by != world and not per_rank_params:
            # another number of data-parallel ranks than the writer's: re-cut the sharded optimizer state
            from ..checkpoint.reshard import copy_param_bufs, resharded_optimizer_state
            copy_param_bufs(trainer.engine, bufs)
            trainer.engine.load_optimizer_state(resharded_optimizer_state(ck["path"], trainer.engine))
            ck["optim"] = None
        elif written_by != world:
            raise ValueError(f"checkpoint written by {written_by} ranks, resumed on {world}: only plain data-parallel runs "
                             "re-cut their optimizer state")
        else:
            for b, saved in zip(trainer.engine.buckets, bufs):
                b.param_buf.copy_(saved.to(b.param_buf.device))
        if ck["optim"] is not None:
            trainer.engine.load_optimizer_state(ck["optim"])
        CheckpointManager.restore_rng(ck["rng"])
        start_step = int(ck["meta"]["step"])
        resumed_evals = int(ck["meta"].get("evals_done", 0))      # the skip-first-evaluations count survives a restart
        trainer.step_idx = start_step

    if not resuming:
        log.log_hyperparameters({
            "global_batch_size": rc.global_batch, "seed": rc.seed, "opt_base_learning_rate": rc.lr,
            "opt_learning_rate_warmup_steps": rc.lr_warmup_iters, "opt_learning_rate_decay_steps": rc.lr_decay_iters,
            "opt_learning_rate_decay_schedule": "cosine with linear warmup", "opt_adamw_beta_1": rc.adam_beta1,
            "opt_adamw_beta_2": rc.adam_beta2, "opt_adamw_epsilon": rc.adam_eps,
            "opt_adamw_weight_decay": rc.weight_decay, "opt_gradient_clip_norm": rc.clip_grad,
            "gradient_accumulation_steps": trainer.n_micro, "max_sequence_length": cfg.seq_len,
            "eval_samples": rc.eval_iters * rc.global_batch, "lora_rank": cfg.lora_rank, "lora_alpha": cfg.lora_alpha})
        run_synthetic_warmup(trainer, rc.warmup_train_steps, rc.warmup_eval_steps)
        log.log_init_stop_run_start()
        log.start(ml.EPOCH_START, metadata={"epoch_num": 0})
        log.start(ml.BLOCK_START, metadata={"samples_count": 0})

    sched = None
    if rc.precision_schedule:
        from ..ops.recipe import PrecisionSchedule
        sched = PrecisionSchedule.from_spec(rc.precision_schedule)
        if tp_size > 1 and rank == 0:
            print("[precision] the schedule governs the linears outside the tensor-parallel blocks; the tensor-parallel linears "
                  f"keep the precision of their context ({tp_ctx.precision})", flush=True)
    deosc = None
    if sched is not None and sched.deosc.enabled:
        from ..ops.recipe import Deoscillator
        deosc = Deoscillator(trainer.engine, sched.deosc)
        if resuming and ck["optim"] is not None and ck["optim"].get("deosc") is not None:
            deosc.load_state_dict(ck["optim"]["deosc"])        # flip counts of the period the checkpoint fell into
    hb = None
    if rc.heartbeat_timeout_s > 0 and world > 1:
        from ..parallel.health import Heartbeat
        hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, interval_s=rc.heartbeat_timeout_s / 4).start()
    straggler = None
    if rc.straggler_interval > 0:
        from ..parallel.health import StragglerDetector
        straggler = StragglerDetector(interval=rc.straggler_interval)
    energy = None
    if rc.energy_monitor and rank == 0:
        from ..utils.energy import EnergyMonitor
        energy = EnergyMonitor().start()
    perf = None
    if rc.perf_jsonl and rank == 0:
        from ..utils.metrics import PerfLogger
        from ..utils.profiler import gpu_peak_tflops
        perf = PerfLogger(cfg.flops_per_token() * cfg.seq_len, world=world, peak_tflops=gpu_peak_tflops(), jsonl=rc.perf_jsonl)
    from ..utils.alloc import GrowthMonitor
    growth = GrowthMonitor(trainer.device if str(trainer.device).startswith("cuda") else None)   # growth after RUN_START
    timer = ml.ThroughputTimer(rc.global_batch)
    t_run0 = time.perf_counter()
    last_ckpt_t = time.perf_counter()
    reached, evals_done, last_eval = False, resumed_evals, None
    losses = []
    prof = None
    step = start_step - 1                               # a run resumed at its last step executes nothing
    for step in range(start_step, rc.train_iters):
        if rc.profile_step_end > rc.profile_step_start and step == rc.profile_step_start and rank == 0:
            from ..utils.profiler import StepProfiler
            prof = StepProfiler(rc.profile_dir or ".", rank)
            prof.start()
        if sched is not None and sched.apply(trainer.model, step) and rank == 0:
            print(f"[precision] step {step}: linears run in {sched.at(step)}; {sched.deosc.status(sched.at(step))}", flush=True)
        if rc.vanish_at_step and step == rc.vanish_at_step and rank == rc.vanish_rank:
            # fault injection: this rank leaves between steps, silently (nothing of it is in flight); once per
            # checkpoint directory, so that the relaunched run gets past the step
            marker = os.path.join(rc.checkpoint_dir or ".", "vanished_once")
            if not os.path.exists(marker):
                open(marker, "w").close()
                if hb is not None:
                    hb.stop()
                from ..parallel.health import clean_exit
                clean_exit(0)
        if hb is not None:
            hb.check(rc.heartbeat_timeout_s)          # raises RankFailure before any kernel of the step is launched
            hb.arrive(step, rc.heartbeat_timeout_s)   # and nobody starts a step that a peer will not join
        timer.step_start()
        batch = host_batch(data, step)
        if torch.cuda.is_available() and str(device).startswith("cuda"):
            batch = tuple(t.pin_memory() for t in batch) if isinstance(batch, tuple) else batch.pin_memory()
        if prof is not None:
            with prof.step_range(step):
                loss = trainer.train_step(batch)
        else:
            loss = trainer.train_step(batch)
        if deosc is not None:
            n_snap = deosc.after_step(step, sched.at(step))
            if n_snap and rank == 0:
                print(f"[deosc] step {step}: {n_snap} oscillating weights of this rank's shards set to their grid value", flush=True)
        step_s = timer.step_stop()
        losses.append(loss)
        if perf is not None:
            perf.step(rc.global_batch)
            if rc.log_interval and (step + 1) % max(rc.log_interval, 1) == 0:
                perf.line(step + 1, {"loss": loss})
        if straggler is not None:
            rep = straggler.record(step_s)
            if rep and rep["stragglers"] and rank == 0:
                print(f"[straggler] ranks {rep['stragglers']} are slower than {straggler.factor} x median "
                      f"({rep['median'] * 1e3:.1f} ms)", flush=True)
        if rc.check_replicas_every and (step + 1) % rc.check_replicas_every == 0:
            spread = trainer.engine.replica_checksum_spread()
            if spread > 0:
                raise RuntimeError(f"step {step + 1}: data-parallel replicas hold different weights (checksum spread {spread})")
        if prof is not None and step + 1 == rc.profile_step_end:
            prof.stop()
            prof = None
        samples = (step + 1) * rc.global_batch
        if rc.log_interval and (step + 1) % rc.log_interval == 0:
            log.event(ml.TRAIN_LOSS, loss, metadata={"samples_count": samples, "lr": trainer.lr()})
        # ---- evaluation ----
        if rc.eval_interval and (step + 1) % rc.eval_interval == 0:
            evals_done += 1
            if evals_done > rc.skip_evals:
                log.end(ml.BLOCK_STOP, metadata={"samples_count": samples})
                log.start(ml.EVAL_START, metadata={"samples_count": samples})
                sums = torch.zeros(2, dtype=torch.float64, device=trainer.device)
                for i in range(max(rc.eval_iters, 1)):
                    eb = host_batch(eval_data, i)
                    if isinstance(eb, tuple):
                        sums += trainer.eval_sums(eb[0].to(trainer.device), eb[1].to(trainer.device))
                    else:
                        sums += trainer.eval_sums(eb.to(trainer.device))
                last_eval = float(sums[0] / sums[1].clamp(min=1))
                log.event(ml.EVAL_ACCURACY, last_eval, metadata={"samples_count": samples})
                log.end(ml.EVAL_STOP, metadata={"samples_count": samples})
                if rc.target_eval_loss > 0 and last_eval <= rc.target_eval_loss:
                    reached = True
                    break
                log.start(ml.BLOCK_START, metadata={"samples_count": samples})
        # ---- checkpoint cadence ----
        if resume_mgr is not None:
            reason = select_checkpoint_reason(global_step=step + 1, batch_in_window=0,
                                              elapsed_since_last_s=time.perf_counter() - last_ckpt_t,
                                              every_steps=rc.checkpoint_every)
            if reason or (rc.die_at_step and step + 1 == rc.die_at_step):
                saver = resume_mgr.save_async if (rc.async_checkpoint and not (rc.die_at_step and step + 1 == rc.die_at_step)) \
                    else resume_mgr.save
                saver(step + 1,
                                dense={"param_bufs": [b.param_buf.detach().cpu() for b in trainer.engine.buckets],
                                       "model_config": cfg.to_dict()},
                                optim_shard=dict(_optim_shard(trainer, per_rank_params),
                                                 deosc=deosc.state_dict() if deosc is not None else None),
                                meta={"samples": samples, "run_started": True, "window": 0, "batch_idx_in_window": -1,
                                      "evals_done": evals_done})
                last_ckpt_t = time.perf_counter()
        if rc.die_at_step and step + 1 == rc.die_at_step:
            if world > 1:
                dist.barrier()
            log.close()
            sys.exit(42)

    if hb is not None:
        hb.stop()
    if resume_mgr is not None:
        resume_mgr.finalize_async()
    duration = time.perf_counter() - t_run0
    success = reached or rc.target_eval_loss <= 0
    if not reached:
        log.end(ml.BLOCK_STOP, metadata={"samples_count": (step + 1) * rc.global_batch})
    log.end(ml.EPOCH_STOP, metadata={"epoch_num": 0})
    log.log_run_stop(success, samples=timer.samples, duration_s=duration)
    log.event(ml.TRACKED_STATS, {"throughput_samples_per_s": timer.throughput(),
                                 "tokens_per_s": timer.throughput() * cfg.seq_len}, metadata={"step": step + 1})
    if energy is not None:
        rep = energy.stop()
        log.event(ml.TRACKED_STATS, {"energy_kwh": rep["energy_kwh"], "peak_power_w": rep["peak_w"]}, metadata={"step": step + 1})
    growth.check(step + 1)
    if rank == 0 and os.environ.get("ALLOC_REPORT", "0") == "1":
        print("[alloc] " + growth.report(), flush=True)
    log.close()
    return {"steps": step + 1 - start_step, "losses": losses, "eval_loss": last_eval, "reached": reached,
            "throughput": timer.throughput(), "records": log.lines, "trainer": trainer, "alloc_growth": growth.events,
            "precision_log": list(sched.log) if sched is not None else [],
            "deosc_history": list(deosc.history) if deosc is not None else []}

"""FLUX.1-schnell MMDiT flow-matching training run.

Constant-with-warm-up LR, AdamW (beta2 0.95, wd 0.1), prompt dropout 0.1, evaluation every
``eval_every_samples`` samples against a target validation loss, FSDP-sharded optimizer state with
parameters kept gathered after forward (``reshard_after_forward: 0`` as in the reference's
submission, flux1/primus/config_common.sh:134), synthetic warm-up steps whose traces are removed
before the clock starts, checkpoints every ``checkpoint_every`` steps (keep the last ``keep_last``,
resume from the latest: flux.1_schnell_t2i-pretrain.yaml:33-37) and ``die_at_step`` fault injection.  Event stream and hyper-parameters follow
flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:25-89 and config_MI355X_1x8x32.sh:7-12.
"""
from __future__ import annotations

import sys
import time

import torch
import torch.distributed as dist

from ..checkpoint.manager import CheckpointManager
from ..mllog import core as ml
from ..models.mmdit import PRESETS, MMDiT, MMDiTConfig
from ..parallel.engine import OptimConfig, ZeroEngine


def flux_bucket_of(name: str) -> str:
    parts = name.split(".")
    if parts[0] in ("double_blocks", "single_blocks"):
        return f"{'d' if parts[0][0] == 'd' else 's'}{int(parts[1]):04d}"
    return "a_io"


class SyntheticFluxData:
    """Pre-encoded sample stand-ins: latents N(0,1) ``[B, Si, 64]`` (already patchified), T5 states
    N(0,1) ``[B, St, 4096]``, pooled CLIP N(0,1) ``[B, 768]`` - a pure function of (seed, step, rank)."""

    def __init__(self, cfg: MMDiTConfig, seed: int = 0):
        self.cfg, self.seed = cfg, seed

    def batch(self, step: int, rank: int, local_batch: int):
        g = torch.Generator().manual_seed((self.seed * 1000003 + step) * 4099 + rank)
        c = self.cfg
        return (torch.randn(local_batch, c.img_tokens, c.in_channels, generator=g),
                torch.randn(local_batch, c.txt_tokens, c.txt_dim, generator=g),
                torch.randn(local_batch, c.vec_dim, generator=g))


class _EncodedView:
    """The ``batch(step, rank, local_batch)`` call of the run loop over an on-disk training set; steps at or above
    10**6 are the loop's evaluation and warm-up requests and read the evaluation set in file order."""

    def __init__(self, train_set, eval_set, world: int):
        self.train, self.eval, self.world = train_set, eval_set, world

    def batch(self, step: int, rank: int, local_batch: int):
        if step >= 10**6:
            per = max(self.eval.steps_per_epoch(local_batch, self.world), 1)
            return self.eval.batch(step % per, rank, local_batch, self.world)
        return self.train.batch(step, rank, local_batch, self.world)


class FluxTrainer:
    def __init__(self, cfg: MMDiTConfig, opt: OptimConfig, device, local_batch: int, warmup_iters: int = 0,
                 prompt_dropout: float = 0.1, comm: str = "nccl", seed: int = 0, micro_batch: int | None = None,
                 sp_group=None, group=None, replicate_group=None):
        """``sp_group``: ranks that share every sample and split its tokens (Ulysses); ``group`` the ranks the
        optimizer shards over and averages gradients across (all ranks when None) - it must contain the
        sequence-parallel ranks, which all draw the same noise and timesteps from the shared seed."""
        self.cfg, self.device = cfg, torch.device(device)
        self.model = MMDiT(cfg, device=self.device, seed=seed)
        if sp_group is not None:
            self.model.set_sequence_parallel(sp_group)
        self.engine = ZeroEngine(self.model, opt, bucket_of=flux_bucket_of, comm=comm, group=group,
                                 replicate_group=replicate_group)
        self.local_batch = local_batch
        self.micro_batch = micro_batch or local_batch
        self.warmup_iters = warmup_iters
        self.prompt_dropout = prompt_dropout
        self.step_idx = 0
        self.gen = torch.Generator(device=self.device).manual_seed(seed + 17)
        self._lr_scale = 1.0
        self.empty_txt = self.empty_pooled = None       # encodings of the empty prompt (prompt dropout); zeros when absent

    def lr(self) -> float:
        base = self.engine.opt.lr * self._lr_scale
        return base * min(1.0, (self.step_idx + 1) / self.warmup_iters) if self.warmup_iters > 0 else base

    def train_step_device(self, latents, txt, pooled) -> torch.Tensor:
        n_micro = max(self.local_batch // self.micro_batch, 1)
        total = None
        for i in range(n_micro):
            sl = slice(i * self.micro_batch, (i + 1) * self.micro_batch)
            loss = self.model.loss(latents[sl], txt[sl], pooled[sl], generator=self.gen,
                                   prompt_dropout=self.prompt_dropout, empty_txt=self.empty_txt, empty_pooled=self.empty_pooled)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        self.engine.step(self.lr(), grad_scale=1.0 / n_micro)
        self.step_idx += 1
        return total / n_micro

    def train_step(self, batch) -> float:
        dev = [t.to(self.device, non_blocking=True) for t in batch]
        return float(self.train_step_device(*dev).item())

    # ------------------------------------------------------------------ state (checkpoints, warm-up restore)
    def snapshot(self) -> dict:
        """Everything a step changes, copied to host memory: flat parameters, this rank's optimizer
        shard, step counters and the noise / timestep generator."""
        e = self.engine

        def host(t):
            return None if t is None else t.detach().to("cpu", copy=True)
        return {"param_bufs": [host(b.param_buf) for b in e.buckets], "m": [host(b.m) for b in e.buckets],
                "v": [host(b.v) for b in e.buckets], "master": [host(b.master) for b in e.buckets],
                "step_count": e.step_count, "step_idx": self.step_idx, "gen": self.gen.get_state().clone()}

    def run_warmup(self, train_batches, eval_batches) -> None:
        """Untimed steps before the clock starts, leaving no trace and needing no copy of the state: the
        steps run with learning rate 0 (AdamW then leaves every weight bit-identical), and afterwards the
        moments - zero before, because a warm-up only precedes a fresh start - the gradients, the step
        counters and the generator are put back."""
        e = self.engine
        if e.step_count != 0 or any(float(b.m.abs().max()) != 0 for b in e.buckets):
            raise RuntimeError("warm-up steps precede the first optimizer step of a fresh run")
        gen, idx = self.gen.get_state().clone(), self.step_idx
        self._lr_scale = 0.0
        try:
            for b in train_batches:
                self.train_step(b)
            for b in eval_batches:
                self.eval_loss(b)
        finally:
            self._lr_scale = 1.0
        for b in e.buckets:
            b.m.zero_()
            b.v.zero_()
            b.grad_buf.zero_()
        e.step_count, self.step_idx = 0, idx
        self.gen.set_state(gen)

    def restore(self, snap: dict) -> None:
        e = self.engine
        for b, p, m, v, w in zip(e.buckets, snap["param_bufs"], snap["m"], snap["v"], snap["master"]):
            b.param_buf.copy_(p.to(b.param_buf.device))
            b.m.copy_(m.to(b.m.device))
            b.v.copy_(v.to(b.v.device))
            if b.master is not None and w is not None:
                b.master.copy_(w.to(b.master.device))
            b.grad_buf.zero_()
        e.step_count, self.step_idx = int(snap["step_count"]), int(snap["step_idx"])
        self.gen.set_state(snap["gen"].cpu() if self.device.type == "cpu" else snap["gen"])
        from ..ops.linear import bump_weight_epoch
        bump_weight_epoch()              # cached low-precision weight copies belong to the old weights

    @torch.no_grad()
    def eval_loss(self, batch) -> float:
        g = torch.Generator(device=self.device).manual_seed(1234)
        dev = [t.to(self.device) for t in batch]
        l = self.model.loss(*dev, generator=g, prompt_dropout=0.0)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(l, op=dist.ReduceOp.AVG)
        return float(l)


def run(exp: dict, device: str | None = None, stream=None) -> dict:
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        from ..config.loader import warn_unknown_keys
        warn_unknown_keys(exp, run, "flux experiment")
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    sync = dist.barrier if world > 1 else None
    ck_dir = str(exp.get("checkpoint_dir") or "")
    mgr = CheckpointManager(ck_dir, rank, world, int(exp.get("keep_last", 3)), sync) if ck_dir else None
    resuming = bool(mgr and mgr.present())
    log = ml.MLLogger(rank=rank, stream=stream or sys.stdout, filename=str(exp.get("mllog_file") or "") or None, sync=sync,
                      append=resuming)
    if not resuming:
        log.log_init_start()
        log.log_submission(exp.get("benchmark", "flux1"), platform=f"1xB200x{world}")
    spec = dict(exp.get("model") or {})
    cfg = PRESETS[spec.pop("preset", "flux1-schnell")]()
    for k, v in spec.items():
        if not hasattr(cfg, k):
            raise KeyError(f"unknown model field '{k}'")
        setattr(cfg, k, tuple(v) if isinstance(v, list) else v)
    ratio = float(exp.get("grad_checkpoint_ratio", 0.0) or 0.0)
    if ratio > 0:
        cfg.recompute, cfg.recompute_ratio = "full", min(ratio, 1.0)
    gbs = int(exp.get("global_batch", 256))
    sp_size = int(exp.get("sp_size", 1))
    sp_group, dp_rank, dp_world = None, rank, world
    if sp_size > 1:
        # sequence-parallel ranks share their samples: the data-parallel coordinate picks the batch
        from ..parallel.mesh import Mesh, MeshSpec
        mesh = Mesh(MeshSpec(cp=sp_size))
        sp_group, dp_rank, dp_world = mesh.group("cp"), mesh.index("dp"), mesh.size("dp")
    replicate = int((exp.get("fsdp") or {}).get("dp_replicate", 1) or 1)
    if int((exp.get("fsdp") or {}).get("reshard_after_forward", 0) or 0) and rank == 0:
        print("[parallel] fsdp.reshard_after_forward: 1 ignored - this trainer shards the optimizer state and keeps the "
              "parameters gathered (the setting of the reference's submission, reshard_after_forward: 0)", flush=True)
    shard_group = rep_group = None
    if replicate > 1 and world > 1:
        # hybrid sharding: optimizer state sharded inside a group of world / replicate ranks, replicated across groups
        if sp_size > 1:
            raise NotImplementedError("dp_replicate is not combined with sp_size")
        from ..parallel.mesh import Mesh, MeshSpec
        hmesh = Mesh(MeshSpec(dp_replicate=replicate))
        shard_group, rep_group = hmesh.group("dp_shard"), hmesh.group("dp_replicate")
    local_batch = int(exp.get("local_batch", gbs // dp_world))
    opt = OptimConfig(lr=float(exp.get("lr", 2.5e-4)), beta1=0.9, beta2=float(exp.get("adam_beta2", 0.95)), eps=1e-8,
                      weight_decay=float(exp.get("weight_decay", 0.1)), clip_grad=float(exp.get("clip_grad", 1.0)))
    tr = FluxTrainer(cfg, opt, device, local_batch, warmup_iters=int(exp.get("lr_warmup_iters", 0)),
                     prompt_dropout=float(exp.get("prompt_dropout", 0.1)),
                     comm=(exp.get("fsdp") or {}).get("comm", "nccl") if replicate == 1 else "nccl", seed=int(exp.get("seed", 0)),
                     micro_batch=exp.get("micro_batch"), sp_group=sp_group, group=shard_group, replicate_group=rep_group)
    dspec = dict(exp.get("data") or {})
    if str(dspec.get("kind", "synthetic")) == "encoded":
        # pre-encoded latents and text states on disk; ``eval_path`` (default: the training set) for validation
        from ..data.flux_encoded import EncodedFluxData
        train_set = EncodedFluxData(dspec["path"], cfg, seed=int(exp.get("seed", 0)))
        eval_set = EncodedFluxData(dspec.get("eval_path") or dspec["path"], cfg, shuffle=False)
        if train_set.empty_t5 is not None and train_set.empty_clip is not None:
            dt = cfg.torch_dtype()
            tr.empty_txt, tr.empty_pooled = train_set.empty_t5.to(tr.device, dt), train_set.empty_clip.to(tr.device, dt)
        data = _EncodedView(train_set, eval_set, dp_world)
    else:
        data = SyntheticFluxData(cfg, seed=int(exp.get("seed", 0)))
    start_step = 0
    if resuming:
        ck = mgr.load()
        tr.restore(ck["optim"]["flux_state"])
        start_step = int(ck["meta"]["step"])
    else:
        log.log_hyperparameters({"global_batch_size": gbs, "seed": int(exp.get("seed", 0)), "opt_base_learning_rate": opt.lr,
                                 "opt_learning_rate_warmup_steps": tr.warmup_iters, "opt_adamw_beta_2": opt.beta2,
                                 "opt_adamw_weight_decay": opt.weight_decay})
        # MLPerf warm-up before the clock starts: synthetic train and validation steps, then every trace of
        # them is removed (flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:82-89: 2 train + 2 val steps)
        n_wt, n_wv = int(exp.get("warmup_train_steps", 0)), int(exp.get("warmup_eval_steps", 0))
        if n_wt or n_wv:
            tr.run_warmup([data.batch(2 * 10**6 + i, dp_rank, local_batch) for i in range(n_wt)],
                          [data.batch(3 * 10**6 + i, dp_rank, local_batch) for i in range(n_wv)])
        log.log_init_stop_run_start()
    log.start(ml.BLOCK_START, metadata={"samples_count": start_step * gbs})
    iters = int(exp.get("train_iters", 10))
    ck_every, die_at = int(exp.get("checkpoint_every", 0)), int(exp.get("die_at_step", 0))
    eval_every = int(exp.get("eval_every_samples", 0))
    target = float(exp.get("target_eval_loss", 0.0))
    timer = ml.ThroughputTimer(gbs)
    t0 = time.perf_counter()
    losses, reached, last_eval = [], False, None
    next_eval = (start_step * gbs // eval_every + 1) * eval_every if eval_every else 0
    samples = start_step * gbs
    # forward-precision switch (flux1/primus/patches/flux_fprop_switch.py:36-308): e.g. {"initial": "a6w4", "switch_step": N,
    # "final": "mxfp8_fwd_mxfp4_bwd", "deosc": {...}}; FLUX_FPROP_SWITCH_STEP overrides the step
    sched = deosc = None
    if exp.get("precision_schedule"):
        from ..ops.recipe import Deoscillator, PrecisionSchedule
        sched = PrecisionSchedule.from_spec(exp["precision_schedule"])
        if sched.deosc.enabled:
            deosc = Deoscillator(tr.engine, sched.deosc)
    prof, prof_span = None, (int(exp.get("profile_step_start", 0) or 0), int(exp.get("profile_step_end", 0) or 0))
    for step in range(start_step, iters):
        if sched is not None and sched.apply(tr.model, step) and rank == 0:
            print(f"[precision] step {step}: linears run in {sched.at(step)}; {sched.deosc.status(sched.at(step))}", flush=True)
        if prof_span[1] > prof_span[0] and step == prof_span[0] and rank == 0:
            from ..utils.profiler import StepProfiler
            prof = StepProfiler(exp.get("profile_dir") or ".", rank)
            prof.start()
        timer.step_start()
        if prof is not None:
            with prof.step_range(step):
                losses.append(tr.train_step(data.batch(step, dp_rank, local_batch)))
        else:
            losses.append(tr.train_step(data.batch(step, dp_rank, local_batch)))
        timer.step_stop()
        if prof is not None and step + 1 == prof_span[1]:
            prof.stop()
            prof = None
        if deosc is not None:
            deosc.after_step(step, sched.at(step))
        samples = (step + 1) * gbs
        log.event(ml.TRAIN_LOSS, losses[-1], metadata={"samples_count": samples})
        if eval_every and samples >= next_eval:
            next_eval += eval_every
            log.end(ml.BLOCK_STOP, metadata={"samples_count": samples})
            log.start(ml.EVAL_START, metadata={"samples_count": samples})
            last_eval = tr.eval_loss(data.batch(10**6, dp_rank, local_batch))
            log.event(ml.EVAL_ACCURACY, last_eval, metadata={"samples_count": samples})
            log.end(ml.EVAL_STOP, metadata={"samples_count": samples})
            if target > 0 and last_eval <= target:
                reached = True
                break
            log.start(ml.BLOCK_START, metadata={"samples_count": samples})
        dying = die_at and step + 1 == die_at
        if mgr is not None and ((ck_every and (step + 1) % ck_every == 0) or dying):
            mgr.save(step + 1, dense=None, optim_shard={"flux_state": tr.snapshot()},
                     meta={"samples": samples, "run_started": True})
        if dying:
            if world > 1:
                dist.barrier()
            log.close()
            sys.exit(42)
    if not reached:
        log.end(ml.BLOCK_STOP, metadata={"samples_count": samples})
    log.log_run_stop(reached or target <= 0, samples=samples, duration_s=time.perf_counter() - t0)
    return {"losses": losses, "eval_loss": last_eval, "throughput": timer.throughput(), "records": log.lines,
            "trainer": tr, "steps": len(losses)}

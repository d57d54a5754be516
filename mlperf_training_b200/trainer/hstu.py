"""DLRMv4 / HSTU training run: sharded item-embedding lookup, dense HSTU model under the ZeRO
engine, sparse row-wise Adagrad in backward, MLLOG events, window-AUC evaluation with a target,
checkpoint cadence and host-side fault injection.

Step structure (the reference's pipelined step, generative_recommenders/dlrm_v4/train/utils.py:3487-3871,
4989-5255) - three stages in flight at once:

    batch N+2  built on the host by the loader thread
    batch N+1  copied H2D on the copy stream, then its sparse input-dist (id sort / dedup, request counts
               and id exchange) on the dist stream
    batch N    row exchange + HSTU forward -> loss -> backward (sparse update inside) -> dense AdamW on the
               main stream

The train loss is read one step late from a pinned buffer (``PendingScalar``), so no step waits
for a device-to-host copy; a ``StepFence`` bounds how far the host may run ahead
(generative_recommenders/dlrm_v4/host_sync_free.py:595-660).
"""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

from ..checkpoint.manager import CheckpointManager
from ..data.hstu_synth import HSTUSyntheticData
from ..mllog import core as ml
from ..models.hstu import HSTU, HSTUConfig
from ..parallel.embedding import ShardedEmbedding
from ..parallel.engine import OptimConfig, ZeroEngine
from ..utils.metrics import BinnedCumulativeAUC, window_auc


class PendingScalar:
    """A device scalar whose value is read on the host one step later from pinned memory."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.buf = torch.zeros(1, dtype=torch.float32).pin_memory() if self.cuda else torch.zeros(1)
        self.event = None
        self.has = False

    def push(self, t: torch.Tensor) -> float | None:
        """Start copying ``t``; returns the previous value (None on the first call)."""
        prev = self.read()
        self.buf.copy_(t.detach().reshape(1).float(), non_blocking=True)
        if self.cuda:
            self.event = torch.cuda.Event()
            self.event.record()
        self.has = True
        return prev

    def read(self) -> float | None:
        if not self.has:
            return None
        if self.event is not None:
            self.event.synchronize()
        return float(self.buf[0])


class StepFence:
    """Keeps the host at most ``lag`` steps ahead of the device."""

    def __init__(self, lag: int = 1, enabled: bool = True):
        self.lag, self.enabled, self.events = lag, enabled and torch.cuda.is_available(), []

    def step(self) -> None:
        if not self.enabled:
            return
        e = torch.cuda.Event()
        e.record()
        self.events.append(e)
        if len(self.events) > self.lag:
            self.events.pop(0).synchronize()


class _WorldView:
    """Binds the world size into ``batch_at`` so every data source has the same call signature."""

    def __init__(self, ds, world: int):
        self.ds, self.world = ds, world
        self.readahead = 0               # > 0: after building a batch, advise the kernel of the next N steps' bytes

    def batch_at(self, step: int, rank: int = 0, pin: bool = False) -> dict:
        out = self.ds.batch_at(step, rank, pin, self.world)
        if self.readahead > 0 and hasattr(self.ds, "prefetch"):
            self.ds.prefetch(range(step + 2, step + 2 + self.readahead), rank, self.world)     # step + 1 is being built next
        return out


def _tensors_of(obj) -> list:
    """Every tensor inside a (nested) dict / list / dataclass-like plan."""
    out = []
    if torch.is_tensor(obj):
        out.append(obj)
    elif isinstance(obj, dict):
        for v in obj.values():
            out += _tensors_of(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            out += _tensors_of(v)
    elif hasattr(obj, "__dict__"):
        out += _tensors_of(vars(obj))
    return [t for t in out if t.is_cuda]


def hstu_bucket_of(name: str) -> str:
    parts = name.split(".")
    return f"l{int(parts[1]):04d}" if parts[0] == "layers" else "a_misc"


class _YambdaStoreView:
    """An event-store stream whose batches carry the keyed jagged features of the eleven-table set: the store gives the
    events (items, times, actions) and the user of every sample; artists, albums and the hashed crosses are derived per
    batch (``data.hstu_synth.yambda_features``)."""

    def __init__(self, inner, tables):
        self.inner, self.tables = inner, {t.name: t for t in tables}
        self.ds = inner.ds

    def batch_at(self, step: int, rank: int = 0, pin: bool = False) -> dict:
        from ..data.hstu_synth import yambda_features
        b = self.inner.batch_at(step, rank, pin=False)
        out = yambda_features(b, self.tables, b["users"], self.ds.item_artist, self.ds.item_album)
        if pin and torch.cuda.is_available():
            out = {k: (v.pin_memory() if hasattr(v, "pin_memory") else v) for k, v in out.items()}
        return out

    @property
    def readahead(self) -> int:
        return self.inner.readahead

    @readahead.setter
    def readahead(self, n: int) -> None:
        self.inner.readahead = n             # the store view underneath does the read-ahead

    def __getattr__(self, name):
        return getattr(self.inner, name)


class HSTUTrainer:
    def __init__(self, cfg: HSTUConfig, table_rows: int, batch_per_gpu: int, device, *, dense_lr=1e-3, sparse_lr=1e-2,
                 clip_grad=1.0, emb_comm="nccl", dense_comm="nccl", seed=0, data_kw: dict | None = None, group=None,
                 table_set: str | None = None, table_scale: int = 1, column_wise: tuple = (), row_wise_min_bytes: int = 1 << 30):
        """``table_set="yambda"``: the multi-table form - an ``EmbeddingCollection`` over the benchmark's eleven tables
        (item / artist / album ids, user id, seven hashed crosses; rows divided by ``table_scale``), batches that carry
        keyed jagged features, a model with the additional-feature branch and the contextual tokens
        (generative_recommenders/modules/dlrm_hstu.py:989-1116).  ``column_wise`` names tables of that set to shard
        along their width instead of by the planner's row-wise / table-wise choice.  Default: one item table."""
        self.cfg, self.device = cfg, torch.device(device)
        self.table_set = table_set
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.model = HSTU(cfg, device=self.device, seed=seed)
        opt = OptimConfig(lr=dense_lr, beta1=0.95, beta2=0.999, eps=1e-8, weight_decay=0.0, clip_grad=clip_grad)
        self.engine = ZeroEngine(self.model, opt, bucket_of=hstu_bucket_of, comm=dense_comm, group=group)
        data_kw = dict(data_kw or {})
        if table_set == "yambda":
            from ..parallel.embedding_collection import EmbeddingCollection, YAMBDA_TABLES, TableConfig
            from ..data.hstu_synth import YambdaSyntheticSamples
            tables = [TableConfig(t.name, max(t.rows // table_scale, 2), cfg.emb_dim, t.features, cfg.dtype) for t in YAMBDA_TABLES]
            n_ctx = sum(1 for t in tables if t.name == "uid" or t.name.startswith("cross_"))
            if cfg.extra_features != 2 or cfg.contextual != n_ctx:
                raise ValueError(f"the yambda table set needs a model with extra_features=2 and contextual={n_ctx}")
            from ..parallel.embedding_collection import plan_tables
            # tables of at least row_wise_min_bytes are cut by rows over all ranks, smaller ones go whole to one rank
            plan = plan_tables(tables, self.world, row_wise_min_bytes=int(row_wise_min_bytes), column_wise=tuple(column_wise))
            self.table = EmbeddingCollection(tables, group=group, device=self.device, lr=sparse_lr, seed=seed, comm=emb_comm, plan=plan)
            self.ctx_keys = [t.name for t in tables if t.name == "uid" or t.name.startswith("cross_")]
            self._yambda_tables = tables
            if data_kw.get("kind", "synthetic") == "synthetic":
                data_kw.pop("kind", None)
                import inspect
                known = set(inspect.signature(HSTUSyntheticData.__init__).parameters)
                self.data = YambdaSyntheticSamples(tables, batch_per_gpu, seed=seed, **{k: v for k, v in data_kw.items() if k in known})
                self.eval_data = None
                data_kw = {"kind": "_done"}
            elif data_kw.get("kind") != "yambda":
                raise ValueError("the eleven-table feature set reads synthetic samples or an event store (data.kind: yambda)")
        else:
            self.table = ShardedEmbedding(table_rows, cfg.emb_dim, group=group, device=self.device, dtype=cfg.torch_dtype(),
                                          lr=sparse_lr, seed=seed, comm=emb_comm, init_scale=0.05)
        kind = data_kw.pop("kind", "synthetic")

        def only(cls, kw):
            """The keys of ``kw`` that ``cls`` takes: an experiment file names the keys of every data kind."""
            import inspect
            known = set(inspect.signature(cls.__init__).parameters)
            return {k: v for k, v in kw.items() if k in known}
        if kind == "sequences":
            # per-user sequence files (MovieLens / KuaiRand layout), user-hash hold-out for evaluation
            from ..data.sequences import SequenceFileDataset
            path = data_kw.pop("path")
            fmt = data_kw.pop("format", "movielens")
            data_kw = only(SequenceFileDataset, data_kw)
            self.data = _WorldView(SequenceFileDataset(path, batch_per_gpu, kind=fmt, split="train", seed=seed, **data_kw), self.world)
            self.eval_data = _WorldView(SequenceFileDataset(path, batch_per_gpu, kind=fmt, split="eval", seed=seed, **data_kw), self.world)
        elif kind == "yambda":
            # memory-mapped event store: time windows, per-rank slices of each window, user-hash hold-out
            from ..data.yambda import EventStoreDataset
            root = data_kw.pop("root", None) or data_kw.pop("path")
            data_kw = only(EventStoreDataset, data_kw)
            self.data = _WorldView(EventStoreDataset(root, batch_per_gpu, split="train", **data_kw), self.world)
            self.eval_data = _WorldView(EventStoreDataset(root, batch_per_gpu, split="eval", **data_kw), self.world)
            if table_set == "yambda":
                # ids are folded into the tables' row counts (the benchmark's tables are as large as its id ranges)
                self.data, self.eval_data = _YambdaStoreView(self.data, self._yambda_tables), _YambdaStoreView(self.eval_data, self._yambda_tables)
            elif self.data.ds.num_items > table_rows:
                raise ValueError(f"the event store under {root} holds item ids up to {self.data.ds.num_items - 1}: "
                                 f"embedding.rows = {table_rows} is too small")
        elif kind != "_done":
            self.data = HSTUSyntheticData(table_rows, batch_per_gpu, seed=seed, **only(HSTUSyntheticData, data_kw))
            self.eval_data = None
        self.batch_per_gpu = batch_per_gpu
        self.sparse_lr, self.lr_warmup_steps, self.lr_warmup_start_lr = float(sparse_lr), 0, 0.0
        self.step_idx = 0
        self.eval_lookahead = True
        self.pipelined = True            # loader thread + copy stream ahead of the step (the reference's TRAIN_PIPELINE=1)
        self.copy_stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.dist_stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.lookup_stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.action_prefill = True       # issue the preprocessor's action branch under the embedding all-to-all
        self.pipeline_input_dist = table_set is None   # the id half of batch N+1's lookup runs under step N (3-stage sparse pipeline)
        self._next = None
        self._ready = None               # (step, device batch, plan, event) prepared ahead
        self._pool = None

    # ------------------------------------------------------------------ data prefetch
    def _build(self, step: int):
        """Host side of a batch (numpy sampling, one pinned storage).  Runs on the loader thread."""
        return self.data.batch_at(step, self.rank, pin=self.device.type == "cuda")

    def _submit(self, step: int):
        if self._pool is None:
            from concurrent.futures import ThreadPoolExecutor
            self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="hstu-loader")
        return self._pool.submit(self._build, step)

    def _to_device(self, host):
        if self.copy_stream is None:
            return host, None
        with torch.cuda.stream(self.copy_stream):
            dev = HSTUSyntheticData.to_device(host, self.device)
            ev = torch.cuda.Event()
            ev.record()
        return dev, ev

    def _take(self, step: int):
        """Batch ``step`` on the device.  Three stages overlap: the loader thread builds batch N+1 on the
        host while the main thread launches step N, and N+1's H2D copy runs on the copy stream under
        step N's kernels (the reference's data-loader workers + copy stream,
        generative_recommenders/dlrm_v4/train/dd_own_h2d.py:65-168)."""
        if not self.pipelined:
            # the unpipelined loop (``train_pipeline: 0``): build, copy, run, in order
            batch, ev = self._to_device(self._build(step))
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
            return batch
        if not self.pipeline_input_dist:
            if self._next is None or self._next[0] != step:
                self._next = (step, self._submit(step))
            host = self._next[1].result()
            batch, ev = self._to_device(host)
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)       # only this batch's own H2D is awaited
            self._next = (step + 1, self._submit(step + 1))      # built while this step runs
            return batch
        # three stages: (N+2) host build | (N+1) H2D + input-dist on side streams | (N) compute
        if self._ready is None or self._ready[0] != step:
            if self._next is None or self._next[0] != step:
                self._next = (step, self._submit(step))
            self._ready = self._prepare(step, self._next[1].result())
            self._next = (step + 1, self._submit(step + 1))
        _, batch, plan, ev = self._ready
        if ev is not None:
            main = torch.cuda.current_stream()
            main.wait_event(ev)
            for t in _tensors_of(batch) + _tensors_of(plan):     # allocated on side streams, consumed on this one
                t.record_stream(main)
        batch = dict(batch, _plan=plan)
        nxt = self._next[1].result() if self._next[0] == step + 1 else self._build(step + 1)
        self._ready = self._prepare(step + 1, nxt)               # launched now, runs under step N's kernels
        self._next = (step + 2, self._submit(step + 2))
        return batch

    def _prepare(self, step: int, host):
        """H2D of a host batch on the copy stream, then the id half of its embedding lookup on the dist
        stream; returns ``(step, device batch, plan, event)``."""
        batch, ev = self._to_device(host)
        if self.dist_stream is None:
            return step, batch, self.table.input_dist(batch["item_ids"]), None
        with torch.cuda.stream(self.dist_stream):
            self.dist_stream.wait_event(ev)
            plan = self.table.input_dist(batch["item_ids"])
            done = torch.cuda.Event()
            done.record()
        return step, batch, plan, done

    # ------------------------------------------------------------------ steps
    def embed(self, batch):
        rows = batch["rows"]
        if self.table_set is not None:
            return self._embed_features(batch)
        emb = torch.zeros((rows, self.cfg.emb_dim), dtype=self.cfg.torch_dtype(), device=self.device)
        emb[: batch["total"]] = self.table.lookup(batch["item_ids"], batch.get("_plan")).to(emb.dtype)
        return emb

    def _embed_features(self, batch):
        """Multi-table lookup of a keyed jagged batch: ``(item rows, additional-feature rows, contextual rows)`` in the
        token order of the dense model.  Every table is looked up once over the merged history + candidate ids."""
        rows, total, dt = batch["rows"], batch["total"], self.cfg.torch_dtype()
        feats = self.table.lookup(batch["samples"].merged())
        tok = batch["token_row"]

        def per_token(name):
            out = torch.zeros((rows, self.cfg.emb_dim), dtype=dt, device=self.device)
            out[:total] = torch.cat([feats["uih_" + name], feats[name]], dim=0)[tok].to(dt)
            return out
        item = per_token("item_id")
        extra = torch.cat([per_token("artist_id"), per_token("album_id")], dim=1)
        ctx = torch.stack([feats[k].to(dt) for k in self.ctx_keys], dim=1)           # [B, contextual, dim]
        return item, extra, ctx

    def _embed_and_prefill(self, batch):
        """Embedding rows of the batch and, issued under their all-to-all, the embedding-independent action branch
        of the preprocessor: the row exchange runs on its own stream while the main stream computes the branch
        (generative_recommenders/modules/action_prefill.py)."""
        if self.lookup_stream is None or not self.action_prefill or self.cfg.contextualized_mlp != "simple":
            return self.embed(batch), None
        main = torch.cuda.current_stream()
        self.lookup_stream.wait_stream(main)
        with torch.cuda.stream(self.lookup_stream):
            emb = self.embed(batch)
            done = torch.cuda.Event()
            done.record()
        pre = self.model.action_branch(batch, batch["rows"])
        main.wait_event(done)
        for t in (emb if isinstance(emb, tuple) else (emb,)):
            t.record_stream(main)
        return emb, pre

    def train_step_device(self, batch) -> torch.Tensor:
        self.model.train()
        dense_lr, self.table.lr = self.lrs_at(self.step_idx)     # the sparse update runs inside backward
        emb, pre = self._embed_and_prefill(batch)
        if self.table_set is not None:
            loss, _, _ = self.model(batch, emb[0], emb[1], emb[2], action_out=pre)
        else:
            loss, _, _ = self.model(batch, emb, action_out=pre)
        loss.backward()
        self.engine.step(dense_lr)
        self.step_idx += 1
        return loss.detach()

    def lrs_at(self, step: int) -> tuple[float, float]:
        """(dense, sparse) learning rates of global step ``step``: each ramps linearly from
        ``min(lr_warmup_start_lr, base)`` to its base over ``lr_warmup_steps`` steps, then holds
        (generative_recommenders/dlrm_v4/train/utils.py:4853-4884; the ramp scales the dense optimizer
        and the in-backward sparse optimizer alike)."""
        bases = (self.engine.opt.lr, self.sparse_lr)
        if self.lr_warmup_steps <= 0:
            return bases
        f = min(1.0, step / self.lr_warmup_steps)
        return tuple(min(self.lr_warmup_start_lr, b) + (b - min(self.lr_warmup_start_lr, b)) * f for b in bases)

    def train_step(self, step: int | None = None) -> torch.Tensor:
        return self.train_step_device(self._take(self.step_idx if step is None else step))

    def _eval_inputs(self, src, step: int):
        b = HSTUSyntheticData.to_device(src.batch_at(step, self.rank), self.device)
        with torch.enable_grad():           # the lookup Function needs a graph only to skip its backward
            emb = self.embed(b)
            emb = tuple(t.detach() for t in emb) if isinstance(emb, tuple) else emb.detach()
        return b, emb

    def lookahead_ready(self) -> bool:
        """Evaluation lookahead (batch N+1's id exchange and row gather on a side stream while batch N
        runs the dense model) is armed only if every rank can do it: one MIN all-reduce, so no rank
        waits in a collective that another never issues (the reference arms its eval lookahead the
        same way, generative_recommenders/dlrm_v4/train/eval_lookahead.py:170-1330)."""
        ok = torch.tensor([1.0 if (self.eval_lookahead and self.device.type == "cuda") else 0.0], device=self.device)
        if self.world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        return bool(ok.item() > 0)

    @torch.no_grad()
    def eval_batches(self, n_batches: int, start: int = 10**6):
        self.model.eval()
        ps, ls = [], []
        src = self.eval_data if self.eval_data is not None else self.data
        if self.eval_data is not None:
            start = 0
        lookahead = n_batches > 1 and self.lookahead_ready()
        side = torch.cuda.Stream() if lookahead else None
        nxt = self._eval_inputs(src, start)
        for i in range(n_batches):
            b, emb = nxt
            ev = None
            if i + 1 < n_batches:
                if lookahead:
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        nxt = self._eval_inputs(src, start + i + 1)
                        ev = torch.cuda.Event()
                        ev.record()
                else:
                    nxt = self._eval_inputs(src, start + i + 1)
            _, p, l = self.model(b, *emb) if isinstance(emb, tuple) else self.model(b, emb)
            ps.append(p)
            ls.append(l)
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
                for t in (*(nxt[1] if isinstance(nxt[1], tuple) else (nxt[1],)), *[v for v in nxt[0].values() if torch.is_tensor(v)]):
                    t.record_stream(torch.cuda.current_stream())
        return torch.cat(ps), torch.cat(ls)


def _warmup(tr: "HSTUTrainer", steps: int) -> None:
    """Untimed steps before RUN_START (first-use costs of every kernel, allocator growth, NCCL
    channels), after which parameters, optimizer state, the embedding shard and its Adagrad sums are
    put back (the reference's pre-RUN_START warm-ups: generative_recommenders/dlrm_v4/train/blas_warmup.py,
    fp8_warmup.py)."""
    if steps <= 0:
        return
    from .warmup import restore_engine, snapshot_engine
    snap = snapshot_engine(tr.engine)
    table_snap = tr.table.snapshot()
    rng_cpu = torch.get_rng_state()
    rng_dev = torch.cuda.get_rng_state() if tr.device.type == "cuda" else None
    for i in range(steps):
        tr.train_step(10**7 + i)
    torch.set_rng_state(rng_cpu)                 # RNG-neutral: dropout masks of the timed run do not move
    if rng_dev is not None:
        torch.cuda.set_rng_state(rng_dev)
    restore_engine(tr.engine, snap)
    tr.table.restore(table_snap)
    tr.step_idx = 0
    tr._next = None
    tr._ready = None


def run(exp: dict, device: str | None = None, stream=None) -> dict:
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        from ..config.loader import warn_unknown_keys
        warn_unknown_keys(exp, run, "hstu experiment")
    from ..utils.metrics import StartupTimeline
    timeline = StartupTimeline()
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    sync = dist.barrier if world > 1 else None
    ckpt = CheckpointManager(exp["checkpoint_dir"], rank, world, int(exp.get("keep_last", 2)), sync) \
        if exp.get("checkpoint_dir") else None
    resuming = bool(ckpt and ckpt.present())
    log = ml.MLLogger(rank=rank, stream=stream or sys.stdout, sync=sync, append=resuming,
                      filename=exp.get("mllog_file") or None)
    if not resuming:
        log.log_init_start()
        log.log_submission(exp.get("benchmark", "dlrm_v4_hstu"), platform=f"1xB200x{world}")
    m = dict(exp.get("model") or {})
    cfg = HSTUConfig(layers=int(m.get("layers", 8)), dim=int(m.get("dim", 512)), heads=int(m.get("heads", 4)),
                     d_qk=int(m.get("d_qk", 128)), d_v=int(m.get("d_v", 128)), max_seq_len=int(m.get("max_seq_len", 4096)),
                     emb_dim=int((exp.get("embedding") or {}).get("dim", 256)), dtype=m.get("dtype", "bf16"),
                     precision=m.get("precision", "bf16"), attn_precision=str(m.get("attn_precision", "bf16")),
                     mlp_hidden=int(m.get("mlp_hidden", 256)), preprocessor=str(m.get("preprocessor", "sum")),
                     contextualized_mlp=str(m.get("contextualized_mlp", "simple")),
                     pmlp_contextual_dropout=float(m.get("pmlp_contextual_dropout", 0.0)),
                     num_positions=int(m.get("num_positions", 8192)), num_time_buckets=int(m.get("num_time_buckets", 2048)))
    # every other field of the model configuration (stochastic depth, recent-window layers, postprocessor, tasks, dropouts,
    # ...) can be named in the experiment file as well; keys that mean nothing are reported
    from dataclasses import fields as _fields
    _named = {"layers", "dim", "heads", "d_qk", "d_v", "max_seq_len", "dtype", "precision", "attn_precision", "mlp_hidden", "preprocessor",
              "contextualized_mlp", "pmlp_contextual_dropout", "num_positions", "num_time_buckets"}
    _policy_keys = {"fp8_scale_policy", "fp8_calibration_steps", "fp8_margin", "fp8_grad_refresh", "fp8_grad_margin"}
    _types = {f.name: f.type for f in _fields(HSTUConfig)}
    for k, v in m.items():
        if k in _named or k in _policy_keys:
            continue
        if k not in _types or k in ("emb_dim", "name"):
            import warnings
            warnings.warn(f"hstu model configuration: key '{k}' has no meaning here and is ignored", stacklevel=2)
            continue
        cur = getattr(cfg, k)
        if isinstance(cur, tuple):
            v = tuple(tuple(x) if isinstance(x, list) else x for x in v)
        elif isinstance(cur, bool):
            v = bool(int(v)) if not isinstance(v, bool) else v
        elif isinstance(cur, (int, float)):
            v = type(cur)(v)
        setattr(cfg, k, v)
    # per-tensor FP8 scale policy: "reference" = the recommender's recipe - forward sites calibrate for 4 steps (margin 1.5)
    # and freeze, gradient sites republish every 200 steps with margin 8; "rolling" = a 4-step delayed-scaling history
    policy = str(m.get("fp8_scale_policy", "rolling")).lower()
    if policy == "reference":
        from ..ops import fp8 as _F8
        _F8.set_policy("e4m3", mode="frozen", history=int(m.get("fp8_calibration_steps", 4)), margin=float(m.get("fp8_margin", 1.5)))
        _F8.set_policy("e5m2", mode="rolling", history=1, refresh=int(m.get("fp8_grad_refresh", 200)), margin=float(m.get("fp8_grad_margin", 8.0)))
    elif policy != "rolling":
        raise ValueError(f"fp8_scale_policy '{policy}': 'rolling' or 'reference'")
    emb = exp.get("embedding") or {}
    table_set = emb.get("tables") or None            # "yambda": the benchmark's eleven tables instead of one item table
    if table_set == "yambda":
        cfg.extra_features, cfg.contextual = 2, 8     # artist + album per token; user id + seven crosses per sample
    d = dict(exp.get("data") or {})
    data_kw = {k: d[k] for k in ("length_median", "length_min", "length_max", "zipf_alpha", "kind", "root", "max_history",
                                 "min_history", "window_seconds", "holdout", "salt", "path", "format", "num_candidates",
                                 "action_weights", "label_bit", "eval_fraction") if k in d}
    if int(d.get("balance_lengths", 0) or 0) and d.get("kind", "synthetic") == "synthetic":
        import torch.distributed as _dist
        data_kw["balance_world"] = _dist.get_world_size() if _dist.is_available() and _dist.is_initialized() else 1
    bpg = int(exp.get("batch_per_gpu", 128))
    tr = HSTUTrainer(cfg, int(emb.get("rows", 1_000_000)), bpg, device, dense_lr=float(exp.get("dense_lr", 1e-3)),
                     sparse_lr=float(exp.get("sparse_lr", 1e-2)), clip_grad=float(exp.get("clip_grad", 1.0)),
                     emb_comm=exp.get("emb_a2a", "nccl"), seed=int(exp.get("seed", 0)), data_kw=data_kw,
                     table_set=table_set, table_scale=int(emb.get("table_scale", 1) or 1),
                     column_wise=tuple(emb.get("column_wise") or ()),
                     row_wise_min_bytes=int(float(emb.get("row_wise_min_bytes", 1 << 30) or (1 << 30))))
    timeline.mark("model_table_data")
    tr.lr_warmup_steps = int(exp.get("lr_warmup_steps", 0) or 0)
    if hasattr(tr.data, "readahead"):
        tr.data.readahead = int(exp.get("cold_prefetch_steps", 0) or 0)
    tr.pipelined = bool(int(exp.get("train_pipeline", 1)))
    tr.lr_warmup_start_lr = float(exp.get("lr_warmup_start_lr", 0.0) or 0.0)
    start = 0
    # what the train / eval split and the position inside the stream depend on: a resumed run must not change it
    contract = {"data_kind": str(d.get("kind", "synthetic")), "holdout": float(d.get("holdout", d.get("eval_fraction", 0.0)) or 0.0),
                "salt": int(d.get("salt", 0) or 0), "window_seconds": int(d.get("window_seconds", 86_400) or 0),
                "batch_per_gpu": bpg, "world": world}
    if resuming:
        ck = ckpt.load()
        from ..checkpoint.manager import validate_split_contract
        validate_split_contract(ck["meta"].get("split_contract"), contract,
                                allow_mismatch=os.environ.get("ALLOW_SPLIT_MISMATCH", "0") == "1")
        tr.model.load_state_dict(ck["dense"]["model"])
        if (ck["path"] / "sparse" / "dcp").exists():
            # TorchRec-layout sharded state: readable under any number of ranks / placement
            tr.table.load_sharded(str(ck["path"] / "sparse" / "dcp"), prefix="model._embedding_collection.")
        else:
            tr.table.load_state_dict(torch.load(ck["path"] / "sparse" / f"shard_rank{rank}.pt", weights_only=False))
        if ck["optim"] is not None:
            tr.engine.load_optimizer_state(ck["optim"])
        CheckpointManager.restore_rng(ck["rng"])
        start = int(ck["meta"]["step"])
        tr.step_idx = start
    else:
        log.log_hyperparameters({"global_batch_size": bpg * world, "seed": int(exp.get("seed", 0)),
                                 "opt_base_learning_rate": float(exp.get("dense_lr", 1e-3))})
        if float(exp.get("alloc_pregrow_gb", 0)) > 0:
            # map the allocator's segments before the run starts (jagged batches change size every step)
            from ..utils.alloc import pregrow
            pregrow(int(float(exp["alloc_pregrow_gb"]) * 2**30), device=tr.device if tr.device.type == "cuda" else None)
        _warmup(tr, int(exp.get("warmup_steps", 0)))
        timeline.mark("warmup")
        if rank == 0 and os.environ.get("STARTUP_TIMELINE", "0") == "1":
            import json
            print("[startup] " + json.dumps(timeline.report()), flush=True)
        log.log_init_stop_run_start()
        log.start(ml.BLOCK_START, metadata={"samples_count": 0})
    from ..utils.alloc import GrowthMonitor
    growth = GrowthMonitor(tr.device if tr.device.type == "cuda" else None)     # allocator growth after RUN_START is reported
    steps = int(exp.get("train_steps", 10))
    eval_every = int(exp.get("eval_interval_steps", 0))
    # the data-fraction cadence of the benchmark: evaluate every ``eval_every_data_pct`` of the epoch and not before
    # ``skip_eval_epoch_pct`` of it (negative: the MLPerf first-evaluation rule); both become global steps once
    from .cadence import data_pct_to_global_steps, should_eval, skip_eval_until_step
    epoch_samples = int(exp.get("total_train_samples", 0))
    if float(exp.get("eval_every_data_pct", 0) or 0) > 0:
        eval_every = data_pct_to_global_steps(float(exp["eval_every_data_pct"]), epoch_samples, bpg * world)
    skip_until = skip_eval_until_step(float(exp.get("skip_eval_epoch_pct", 0) or 0), epoch_samples, bpg * world)
    n_eval = int(exp.get("num_eval_batches", 2))
    thr = float(exp.get("auc_threshold", 0.0))
    die_at = int(exp.get("die_at_step", 0))
    every = int(exp.get("checkpoint_every", 0))
    timer = ml.ThroughputTimer(bpg * world)
    pending, fence = PendingScalar(device), StepFence(1)
    lifetime = BinnedCumulativeAUC(device=device)
    losses, aucs, reached = [], [], False
    t0 = time.perf_counter()
    window_of = getattr(getattr(tr.data, "ds", tr.data), "window_of_step", None)
    last_window, barrier_debug = None, os.environ.get("WINDOW_BARRIER_DEBUG", "0") == "1"
    # torch profiler over steps [profile_step_start, profile_step_end) on rank 0, every step marked for the trace
    # post-processing (generative_recommenders/dlrm_v4/utils.py:451-822)
    prof, prof_span = None, (int(exp.get("profile_step_start", 0) or 0), int(exp.get("profile_step_end", 0) or 0))
    for step in range(start, steps):
        if window_of is not None:
            w = window_of(step, world)
            if w != last_window:
                # window boundary: ranks finish a window's host work at different times; meet here, and say so
                # when somebody had to wait long (generative_recommenders/dlrm_v4/train/utils.py:356-402)
                from ..parallel.health import timed_barrier
                waited = timed_barrier(label=f"window {w}") if world > 1 else 0.0
                if barrier_debug and rank == 0:
                    print(f"[window-barrier] step {step} window {w} waited {waited:.3f} s", flush=True)
                last_window = w
        if prof_span[1] > prof_span[0] and step == prof_span[0] and rank == 0:
            from ..utils.profiler import StepProfiler
            prof = StepProfiler(exp.get("profile_dir") or ".", rank)
            prof.start()
        timer.step_start()
        if prof is not None:
            with prof.step_range(step):
                loss = tr.train_step(step)
        else:
            loss = tr.train_step(step)
        prev = pending.push(loss)
        fence.step()
        timer.step_stop()
        if prof is not None and step + 1 == prof_span[1]:
            prof.stop()
            prof = None
        if prev is not None:
            losses.append(prev)
            log.event(ml.TRAIN_LOSS, prev, metadata={"samples_count": step * bpg * world})
        samples = (step + 1) * bpg * world
        if should_eval(step + 1, eval_every, skip_until):
            log.end(ml.BLOCK_STOP, metadata={"samples_count": samples})
            log.start(ml.EVAL_START, metadata={"samples_count": samples})
            p, l = tr.eval_batches(n_eval)
            lifetime.update(p, l)
            auc = window_auc(p, l)
            aucs.append(auc)
            log.event(ml.EVAL_ACCURACY, auc, metadata={"samples_count": samples})
            log.end(ml.EVAL_STOP, metadata={"samples_count": samples})
            stop = torch.tensor([1.0 if (thr > 0 and auc >= thr) else 0.0], device=device)
            if world > 1:
                dist.broadcast(stop, 0)                      # rank 0 decides, everyone leaves together
            if stop.item() > 0:
                reached = True
                break
            log.start(ml.BLOCK_START, metadata={"samples_count": samples})
        if ckpt is not None and ((every and (step + 1) % every == 0) or (die_at and step + 1 == die_at)):
            if str(exp.get("sparse_checkpoint", "per_rank")) == "sharded":
                # every rank writes its rows as ShardedTensor chunks under TorchRec's key names (collective)
                writer = lambda d_: tr.table.save_sharded(str(d_ / "dcp"), prefix="model._embedding_collection.")
            else:
                sd = tr.table.state_dict()
                writer = lambda d_: torch.save(sd, d_ / f"shard_rank{rank}.pt")
            ckpt.save(step + 1, dense={"model": tr.model.state_dict()}, optim_shard=tr.engine.optimizer_state(),
                      meta={"samples": samples, "window": 0, "batch_idx_in_window": step + 1, "split_contract": contract},
                      sparse_writer=writer)
        if die_at and step + 1 == die_at:
            if world > 1:
                dist.barrier()
            log.close()
            sys.exit(42)
    last = pending.read()
    if last is not None:
        losses.append(last)
    if not reached:
        log.end(ml.BLOCK_STOP, metadata={"samples_count": timer.samples})
    lifetime.sync()
    log.log_run_stop(reached or thr <= 0, samples=timer.samples, duration_s=time.perf_counter() - t0)
    growth.check(steps)
    if rank == 0 and os.environ.get("ALLOC_REPORT", "0") == "1":
        print("[alloc] " + growth.report(), flush=True)
    log.close()
    return {"losses": losses, "aucs": aucs, "lifetime_auc": lifetime.compute(), "throughput": timer.throughput(),
            "records": log.lines, "trainer": tr, "alloc_growth": growth.events}

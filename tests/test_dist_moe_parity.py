"""Tiny GPT-OSS-style MoE on CPU / gloo with world size 2 and expert parallelism 2: per-step loss
parity against a single process over 10 AdamW steps.  A second case spreads the experts over 2 of 4
ranks (two copies of every expert): their gradients are summed over the copies and the clipping norm
counts every expert once.

4 layers, d_model 256, 8 query / 2 KV heads of 32, alternating full and 128-token sliding-window
attention, 8 SwiGLU experts (FFN 512) with a top-2 softmax router, vocab 2048, fp32, seq 256,
micro-batch 4 per rank, uniform token ids from seed 0, AdamW lr 1e-4 wd 0.1.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlperf_training_b200.models.gpt import GPT, tiny_moe
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine

STEPS, MB = 10, 4


def _data(cfg, world, steps):
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, cfg.vocab_size, (steps, world * MB, cfg.seq_len + 1), generator=g)


def _opt():
    return OptimConfig(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, clip_grad=1.0)


def _single(cfg, WORLD, steps):
    torch.manual_seed(0)
    model = GPT(cfg, "cpu", seed=0)
    eng = ZeroEngine(model, _opt())
    data = _data(cfg, WORLD, steps)
    losses = []
    for s in range(steps):
        tot = 0.0
        for r in range(WORLD):  # the ranks' micro-batches as gradient accumulation
            chunk = data[s, r * MB:(r + 1) * MB]
            loss = model(chunk[:, :-1], chunk[:, 1:])
            loss.backward()
            tot += float(loss.detach())
        eng.step(grad_scale=1.0 / WORLD)
        losses.append(tot / WORLD)
    return losses


def _worker(rank, port, cfg, q, WORLD, EP, steps):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        full = GPT(cfg, "cpu", seed=0)                       # same init as the single process
        if EP == WORLD:
            ep_group, edp_group, ep_rank = dist.group.WORLD, None, rank
        else:
            from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec
            mesh = Mesh(MeshSpec(ep=EP))
            ep_group, edp_group, ep_rank = mesh.group("ep"), mesh.group("edp"), mesh.index("ep")
        model = GPT(cfg, "cpu", seed=0, ep_group=ep_group)
        L = cfg.n_experts // EP
        with torch.no_grad():
            src = dict(full.named_parameters())
            for n, p in model.named_parameters():
                t = src[n]
                p.copy_(t[ep_rank * L:(ep_rank + 1) * L] if getattr(p, "expert_parallel", False) else t)
        del full
        eng = ZeroEngine(model, _opt(), expert_dp_group=edp_group)
        data = _data(cfg, WORLD, steps)
        losses = []
        for s in range(steps):
            chunk = data[s, rank * MB:(rank + 1) * MB]
            loss = model(chunk[:, :-1], chunk[:, 1:])
            loss.backward()
            eng.step()
            l = loss.detach().clone()
            dist.all_reduce(l)
            losses.append(float(l) / WORLD)
        if rank == 0:
            q.put(losses)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("WORLD,EP,steps", [(2, 2, STEPS), (4, 2, 4)])
def test_moe_ep2_loss_parity(WORLD, EP, steps):
    cfg = tiny_moe()
    ref = _single(cfg, WORLD, steps)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, cfg, q, WORLD, EP, steps)) for r in range(WORLD)]
    for p in procs:
        p.start()
    got = q.get(timeout=800)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    diffs = [abs(a - b) for a, b in zip(ref, got)]
    assert max(diffs) < 2e-4, (ref, got)
    assert got[-1] < got[0]

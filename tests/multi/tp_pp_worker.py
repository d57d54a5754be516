"""Worker (gloo, 4 ranks): tensor-parallel stages of a pipeline (tensor 2 x pipeline 2, plain or interleaved
schedule) follow the loss, the gradient norm and the parameters of the unsplit model that every rank trains beside
them on the same batches; then the run loop drives the same mesh from a configuration.
argv: <virtual stages>"""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, GPTConfig, shard_of  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec  # noqa: E402
from mlperf_training_b200.parallel.tensor import TPContext  # noqa: E402
from mlperf_training_b200.trainer.loop import run  # noqa: E402
from mlperf_training_b200.trainer.pipeline_train import PipelineTrainer  # noqa: E402
from mlperf_training_b200.trainer.pretrain import TrainConfig  # noqa: E402


def main():
    v = int(sys.argv[1])
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(4)][rank]
    cfg = GPTConfig(n_layers=4, hidden=32, n_heads=4, n_kv_heads=2, head_dim=8, ffn_hidden=64, vocab_size=64, seq_len=16, dtype="fp32")
    full = GPT(cfg, device="cpu", seed=3)
    opt = OptimConfig(lr=3e-3, weight_decay=0.01, clip_grad=1.0)
    e_full = ZeroEngine(full, opt, group=solo)
    mesh = Mesh(MeshSpec(tp=2, pp=2))
    tp = TPContext(mesh.group("tp"), comm="nccl")
    ok = mesh.ranks["tp"] == ([0, 1] if rank < 2 else [2, 3]) and mesh.ranks["pp"] == [rank % 2, rank % 2 + 2]
    n_micro = 2
    tr = PipelineTrainer(cfg, opt, TrainConfig(micro_batch=1, local_batch=n_micro, seed=0), "cpu", mesh, virtual_stages=v, tp=tp)
    for chunk in tr.chunks:
        chunk.load_from_full(full)
    for b in tr.engine.buckets:                      # the engine's flat buffers are the storage: nothing to re-pack
        assert b.param_buf.abs().sum() > 0
    ok &= tr.chunks[0].blocks[0].w_qkv.shape[0] * 2 == full.blocks[0].w_qkv.shape[0]
    for step in range(4):
        g = torch.Generator().manual_seed(100 + step)
        tok = torch.randint(0, cfg.vocab_size, (n_micro, cfg.seq_len + 1), generator=g)
        # the unsplit model: the same micro-batches, gradients accumulated, one step
        ref = 0.0
        for i in range(n_micro):
            l = full(tok[i:i + 1, :-1].contiguous(), tok[i:i + 1, 1:].contiguous())
            l.backward()
            ref += float(l.detach()) / n_micro
        e_full.step(tr.lr(), grad_scale=1.0 / n_micro)
        loss = float(tr.train_step_device(tok))
        n_ref, n_pp = e_full.grad_norm(), tr.engine.grad_norm()
        good = abs(loss - ref) < 2e-4 * max(1.0, abs(ref)) and abs(n_ref - n_pp) < 2e-3 * max(1.0, n_ref)
        ok &= good
        if rank == 0:
            print(f"step {step} unsplit {ref:.5f} tp x pp {loss:.5f} gnorm {n_ref:.4f} {n_pp:.4f}", flush=True)
    # after four steps the slices still equal the unsplit model's
    for chunk in tr.chunks:
        for blk, i in zip(chunk.blocks, chunk.layers):
            want = shard_of(full.blocks[i].w_qkv, "qkv", 2, tp.rank, cfg)
            ok &= bool((blk.w_qkv - want).abs().max() < 5e-5)
    ev = tr.eval_sums(tok)
    with torch.no_grad():
        want = full(tok[:, :-1].contiguous(), tok[:, 1:].contiguous(), n_valid=1)
    ok &= abs(float(ev[0]) - float(want)) < 1e-3 * float(want) and int(ev[1]) == tok[:, 1:].numel()

    # the run loop on the same mesh
    tiny = dict(n_layers=4, hidden=32, n_heads=4, n_kv_heads=2, head_dim=8, ffn_hidden=64, vocab_size=64, seq_len=16, dtype="fp32")
    out = run(dict(model=tiny, global_batch=4, micro_batch=1, train_iters=3, lr=5e-3, lr_warmup_iters=1, tensor_parallel=2,
                   pipeline_parallel=2, virtual_pipeline_parallel=v, eval_interval=3, eval_iters=1, clip_grad=1.0),
              device="cpu", stream=io.StringIO())
    losses = torch.tensor(out["losses"], dtype=torch.float64)
    first = losses.clone()
    dist.broadcast(first, src=0)
    ok &= out["steps"] == 3 and bool(torch.isfinite(losses).all()) and bool((first - losses).abs().max() < 1e-9)
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

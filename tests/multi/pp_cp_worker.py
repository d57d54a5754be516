"""Worker (gloo, 4 ranks): pipeline 2 x context 2 (all-gather and zig-zag ring forms, plain and masked labels) follows
the unsplit model trained on whole sequences; then the run loop on the same mesh.  argv: <virtual stages>"""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec  # noqa: E402
from mlperf_training_b200.trainer.loop import run  # noqa: E402
from mlperf_training_b200.trainer.pipeline_train import PipelineTrainer  # noqa: E402
from mlperf_training_b200.trainer.pretrain import TrainConfig  # noqa: E402


def main():
    v = int(sys.argv[1])
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(4)][rank]
    mesh = Mesh(MeshSpec(pp=2, cp=2))
    cfg = GPTConfig(n_layers=4, hidden=32, n_heads=4, n_kv_heads=2, head_dim=8, ffn_hidden=64, vocab_size=64, seq_len=32, dtype="fp32")
    opt = OptimConfig(lr=3e-3, weight_decay=0.01, clip_grad=1.0)
    ok = True
    for mode, masked in (("allgather", False), ("ring", False), ("ring", True)):
        full = GPT(cfg, device="cpu", seed=3)
        e_full = ZeroEngine(full, opt, group=solo)
        tr = PipelineTrainer(cfg, opt, TrainConfig(micro_batch=1, local_batch=2, seed=0), "cpu", mesh, virtual_stages=v,
                             cp_group=mesh.group("cp"), cp_mode=mode)
        for chunk in tr.chunks:
            chunk.load_from_full(full)
        for step in range(3):
            g = torch.Generator().manual_seed(100 + step)
            tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=g)
            x, y = tok[:, :-1].contiguous(), tok[:, 1:].clone()
            if masked:
                y[:, :19] = -100
            ref = 0.0
            for i in range(2):
                n = max(int((y[i:i + 1] != -100).sum()), 1) if masked else None
                l = full(x[i:i + 1], y[i:i + 1], n_valid=n)
                l.backward()
                ref += float(l.detach()) / 2
            e_full.step(tr.lr(), grad_scale=0.5)
            loss = float(tr.train_step_device(x, y) if masked else tr.train_step_device(tok))
            good = abs(loss - ref) < 3e-5 * max(1.0, abs(ref)) and abs(e_full.grad_norm() - tr.engine.grad_norm()) < 2e-3
            ok &= good
            if rank == 0:
                print(f"{mode} masked={masked} step {step}: unsplit {ref:.6f} pp x cp {loss:.6f} gnorm {e_full.grad_norm():.4f} "
                      f"{tr.engine.grad_norm():.4f}", flush=True)
        ev = tr.eval_sums(tok)
        with torch.no_grad():
            want = full(tok[:, :-1].contiguous(), tok[:, 1:].contiguous(), n_valid=1)
        ok &= abs(float(ev[0]) - float(want)) < 1e-3 * float(want) and int(ev[1]) == tok[:, 1:].numel()
    tiny = dict(n_layers=4, hidden=32, n_heads=4, n_kv_heads=2, head_dim=8, ffn_hidden=64, vocab_size=64, seq_len=32, dtype="fp32")
    out = run(dict(model=tiny, global_batch=2, micro_batch=1, train_iters=3, lr=5e-3, lr_warmup_iters=1, pipeline_parallel=2,
                   virtual_pipeline_parallel=v, context_parallel=2, context_parallel_mode="ring", eval_interval=3, eval_iters=1),
              device="cpu", stream=io.StringIO())
    t = torch.tensor(out["losses"], dtype=torch.float64)
    first = t.clone()
    dist.broadcast(first, src=0)
    ok &= out["steps"] == 3 and bool(torch.isfinite(t).all()) and bool((first - t).abs().max() < 1e-9)
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

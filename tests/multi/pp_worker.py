"""Worker: a 2-stage pipeline (1F1B, 4 micro-batches) must follow the unsplit model's loss curve."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec  # noqa: E402
from mlperf_training_b200.parallel.pipeline import GPTStage, PipelineRunner, pp_bucket_of  # noqa: E402


def main():
    backend = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = backend == "nccl"
    if gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if gpu else torch.device("cpu")
    dist.init_process_group(backend)
    mesh = Mesh(MeshSpec(pp=world))
    cfg = GPTConfig(n_layers=3, hidden=256 if gpu else 64, n_heads=4, n_kv_heads=2, head_dim=64 if gpu else 16,
                    ffn_hidden=512 if gpu else 128, vocab_size=512 if gpu else 256, seq_len=128 if gpu else 32,
                    dtype="bf16" if gpu else "fp32")
    full = GPT(cfg, device=device, seed=5)
    stage = GPTStage(cfg, mesh.index("pp"), world, device=device)
    stage.load_from_full(full)
    opt = OptimConfig(lr=2e-3, weight_decay=0.0, clip_grad=0.5)
    e_full = ZeroEngine(full, opt, group=mesh.group("dp"))
    e_st = ZeroEngine(stage, opt, group=mesh.group("dp"), bucket_of=pp_bucket_of, pp_group=mesh.group("pp"))
    prev, nxt = mesh.prev_next_stage()
    runner = PipelineRunner(stage, prev, nxt)
    M, ok = 4, True
    for step in range(4):
        g = torch.Generator().manual_seed(step)
        tok = torch.randint(0, cfg.vocab_size, (M, 2, cfg.seq_len + 1), generator=g).to(device)
        mbs = [(tok[i, :, :-1].contiguous(), tok[i, :, 1:].contiguous()) for i in range(M)]
        ref = 0.0
        for x, y in mbs:
            l = full(x, y)
            l.backward()
            ref += l.item()
        e_full.step(grad_scale=1.0 / M)
        tot = runner.run(mbs)
        e_st.step(grad_scale=1.0 / M)
        got = torch.tensor([tot.item() if tot is not None else 0.0], device=device)
        dist.all_reduce(got)
        tol = 3e-2 if gpu else 2e-4
        good = abs(got.item() - ref) < tol * max(1.0, abs(ref)) and abs(e_full.grad_norm() - e_st.grad_norm()) < 10 * tol
        ok &= good
        if rank == 0:
            print(f"step {step} full {ref / M:.5f} pp {got.item() / M:.5f} gnorm {e_full.grad_norm():.4f} {e_st.grad_norm():.4f}",
                  flush=True)
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

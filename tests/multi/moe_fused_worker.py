"""Worker (GPUs, NCCL): the peer-memory expert dispatcher must give the outputs and gradients of
the all-to-all dispatcher on the same routed tokens."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.ops import _lib  # noqa: E402
from mlperf_training_b200.ops import moe_ops as M  # noqa: E402
from mlperf_training_b200.parallel.expert import ExpertParallelDispatcher, FusedExpertDispatcher  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl")
    precision = sys.argv[1] if len(sys.argv) > 1 else "bf16"
    E, D, Fh, T, k = 4 * world, 256, 128, 512, 2
    L = E // world
    torch.manual_seed(10 + rank)
    x0 = torch.randn(T, D, device=dev).bfloat16()
    logits = torch.randn(T, E, device=dev)
    w1 = (torch.randn(L, 2 * Fh, D, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(L, D, Fh, device=dev) * 0.05).bfloat16()
    gy = torch.randn(T, D, device=dev).bfloat16()
    res = []
    for kind in ("nccl", "fused", "fused"):                     # the fused path twice: slabs are reused
        x = x0.clone().requires_grad_(True)
        a1, a2 = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        idx, w, counts = M.RouterFn.apply(logits.clone(), k)
        disp = ExpertParallelDispatcher(dist.group.WORLD, E) if kind == "nccl" else \
            FusedExpertDispatcher(dist.group.WORLD, E, D, T * k, dev, pad=M.pad_rows(precision))
        y = disp(x, idx, w, counts, a1, a2, precision)
        y.backward(gy)
        torch.cuda.synchronize()
        res.append((y.detach().float(), x.grad.float(), a1.grad.float(), a2.grad.float()))
        if kind == "fused":
            assert int(disp.dropped.item()) == 0
    _lib.check_status("moe fused")
    ok = True
    for other in res[1:]:
        for name, a, b in zip(("y", "dx", "dw1", "dw2"), res[0], other):
            err = (a - b).abs().max().item()
            tol = (2e-2 if precision == "bf16" else 6e-2) * max(a.abs().max().item(), 1e-3)   # block scales group other rows
            ok &= err <= tol
            if rank == 0:
                print(f"{name}: max diff {err:.4e} (tol {tol:.4e})", flush=True)
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

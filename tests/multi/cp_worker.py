"""Worker: context-parallel causal attention (sequence sharded over the ranks) equals attention
over the whole sequence, forward and backward.  argv: backend [ring]: with ``ring`` also the zig-zag ring form."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.ops.functional import attention  # noqa: E402
from mlperf_training_b200.parallel.context import (context_parallel_attention, ring_attention, ulysses_attention,  # noqa: E402
                                                   zigzag_chunk, zigzag_unchunk)


def main():
    backend = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = backend == "nccl"
    if gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device()) if gpu else torch.device("cpu")
    dist.init_process_group(backend)
    B, S, Hq, Hkv, D = 2, (256 if gpu else 32) * world, 4, 2, (64 if gpu else 16)
    dt = torch.bfloat16 if gpu else torch.float32
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, S, h, D, generator=g).to(dev).to(dt) for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, D, generator=g).to(dev).to(dt)
    ok = True
    for window in (0, 24 if not gpu else 128):
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = attention(qf, kf, vf, causal=True, window=window)
        ref.backward(do)
        s = S // world
        sl = slice(rank * s, (rank + 1) * s)
        ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
        out = context_parallel_attention(ql, kl, vl, dist.group.WORLD, window=window)
        out.backward(do[:, sl])
        tol = 3e-2 if gpu else 1e-5
        for name, a, b in (("o", out, ref[:, sl]), ("dq", ql.grad, qf.grad[:, sl]), ("dk", kl.grad, kf.grad[:, sl]),
                           ("dv", vl.grad, vf.grad[:, sl])):
            err = (a.float() - b.float()).abs().max().item()
            ok &= err <= tol * max(1.0, b.float().abs().max().item())
            if rank == 0:
                print(f"window {window} {name}: {err:.3e}", flush=True)
    # Ulysses exchange (sequence shards <-> head shards), non-causal and causal
    if Hkv % world == 0:
        for causal in (False, True):
            qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
            ref = attention(qf, kf, vf, causal=causal)
            ref.backward(do)
            s = S // world
            sl = slice(rank * s, (rank + 1) * s)
            ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
            out = ulysses_attention(ql, kl, vl, dist.group.WORLD, causal=causal)
            out.backward(do[:, sl])
            tol = 3e-2 if gpu else 1e-5
            for name, a, b in (("o", out, ref[:, sl]), ("dq", ql.grad, qf.grad[:, sl]), ("dk", kl.grad, kf.grad[:, sl]),
                               ("dv", vl.grad, vf.grad[:, sl])):
                err = (a.float() - b.float()).abs().max().item()
                ok &= err <= tol * max(1.0, b.float().abs().max().item())
                if rank == 0:
                    print(f"ulysses causal={causal} {name}: {err:.3e}", flush=True)
    if len(sys.argv) > 2 and sys.argv[2] == "ring":
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = attention(qf, kf, vf, causal=True)
        ref.backward(do)
        ql, kl, vl = (zigzag_chunk(t, world, rank).requires_grad_(True) for t in (q, k, v))
        out = ring_attention(ql, kl, vl, dist.group.WORLD)
        out.backward(zigzag_chunk(do, world, rank))
        tol = 3e-2 if gpu else 1e-5
        for name, a, b in (("o", out, ref), ("dq", ql.grad, qf.grad), ("dk", kl.grad, kf.grad), ("dv", vl.grad, vf.grad)):
            b = zigzag_chunk(b.detach(), world, rank)
            err = (a.float() - b.float()).abs().max().item()
            ok &= err <= tol * max(1.0, b.float().abs().max().item())
            if rank == 0:
                print(f"ring {name}: {err:.3e}", flush=True)
        pieces = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(pieces, out.detach().contiguous())
        ok &= bool((zigzag_unchunk(pieces) - ref.detach()).abs().max() <= tol)
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

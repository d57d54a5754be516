"""Worker: sharded embedding lookup + backward on W ranks must equal a single full table."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.parallel.embedding import ShardedEmbedding  # noqa: E402


def main():
    backend = sys.argv[1]
    comm = sys.argv[2] if len(sys.argv) > 2 else "nccl"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        device = torch.device("cuda", torch.cuda.current_device())
    else:
        device = torch.device("cpu")
    dist.init_process_group(backend)
    rows, dim = 1000, 64
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    tab = ShardedEmbedding(rows, dim, device=device, dtype=dtype, lr=0.1, comm=comm, max_requests=4096)
    # a replicated full copy, assembled from the shards
    shards = [torch.zeros(tab.rows_per_rank, dim, dtype=dtype, device=device) for _ in range(world)]
    dist.all_gather(shards, tab.weight.clone())
    full = torch.cat(shards)[:rows].float()
    full_state = torch.zeros(rows, device=device)
    ok = True
    for it in range(3):
        g = torch.Generator().manual_seed(100 * it + rank)
        ids = torch.randint(0, rows, (300,), generator=g).to(device)
        ids[:20] = ids[20:40]                                   # duplicates inside a rank
        w = torch.randn(300, dim, generator=g).to(device).to(dtype).float()
        out = tab.lookup(ids)
        ok &= bool(torch.allclose(out.float(), full[ids], atol=1e-2, rtol=1e-2))
        (out.float() * w).sum().backward()
        # reference update on the replicated copy: all ranks' gradients, summed per row
        all_ids = [torch.zeros_like(ids) for _ in range(world)]
        all_w = [torch.zeros_like(w) for _ in range(world)]
        dist.all_gather(all_ids, ids)
        dist.all_gather(all_w, w)
        gi, gw = torch.cat(all_ids), torch.cat(all_w)
        u, inv = torch.unique(gi, return_inverse=True)
        gsum = torch.zeros(u.numel(), dim, device=device).index_add_(0, inv, gw)
        full_state[u] += (gsum * gsum).mean(-1)
        full[u] -= 0.1 * gsum / (full_state[u].sqrt()[:, None] + tab.eps)
        if dtype == torch.bfloat16:
            full[u] = full[u].bfloat16().float()
    mine = full[tab.row_lo: tab.row_lo + tab.local_rows]
    err = (tab.weight.float() - mine).abs().max().item()
    ok &= err < (3e-2 if dtype == torch.bfloat16 else 1e-5)
    print(f"rank {rank} ok={ok} err={err:.3e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

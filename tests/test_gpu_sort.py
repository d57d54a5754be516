"""Bounded-key radix sort, run bookkeeping and the deterministic segment reduction against the CPU path."""
import pytest
import torch

from mlperf_training_b200.ops import _lib, sort
from mlperf_training_b200.parallel.embedding import ShardedEmbedding

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,rows", [(1, 10), (1000, 50), (200_003, 400_000_000), (65_536, 3)])
def test_sort_unique_and_segment_sum(n, rows):
    g = torch.Generator().manual_seed(n)
    ids = torch.randint(0, rows, (n,), generator=g)
    src = torch.randn(n, 64, generator=g).bfloat16()
    c = sort.sort_unique(ids, sort.key_bits_for(rows))
    d = sort.sort_unique(ids.cuda(), sort.key_bits_for(rows))
    torch.cuda.synchronize()
    _lib.check_status("sort")
    cnt = int(c.count)
    assert int(d.count.item()) == cnt
    assert torch.equal(d.keys.cpu(), c.keys) and torch.equal(d.perm.cpu(), c.perm)          # stable: same permutation
    assert torch.equal(d.uniq[:cnt].cpu(), c.uniq[:cnt]) and torch.equal(d.seg[:cnt + 1].cpu(), c.seg[:cnt + 1])
    assert torch.equal(d.inverse.cpu(), c.inverse) and bool((d.uniq[cnt:] == -1).all())
    for out_dtype in (torch.float32, torch.bfloat16):
        a = sort.segment_sum(src, c, out_dtype)[:cnt].float()
        b = sort.segment_sum(src.cuda(), d, out_dtype)[:cnt].float().cpu()
        assert (a - b).abs().max() <= 1e-2 * max(a.abs().max().item(), 1.0)
    b2 = sort.segment_sum(src.cuda(), d, torch.float32)
    assert torch.equal(b2, sort.segment_sum(src.cuda(), d, torch.float32))                  # run twice: bit-identical


def test_segment_sum_long_runs():
    """Skewed ids: runs longer than one warp's share (summed through per-block partial sums), runs that start in the
    middle of a block, a run of exactly the block size, next to ordinary short runs."""
    g = torch.Generator().manual_seed(5)
    ids = torch.cat([torch.full((1000,), 7), torch.full((65,), 3), torch.full((64,), 11), torch.full((129,), 2),
                     torch.randint(100, 5000, (3000,), generator=g), torch.full((300,), 99)])
    ids = ids[torch.randperm(ids.numel(), generator=g)]
    for D, dt in ((256, torch.bfloat16), (72, torch.float32)):
        src = torch.randn(ids.numel(), D, generator=g).to(dt)
        c = sort.sort_unique(ids, 13)
        d = sort.sort_unique(ids.cuda(), 13)
        cnt = int(c.count)
        a = sort.segment_sum(src, c, torch.float32)[:cnt]
        b = sort.segment_sum(src.cuda(), d, torch.float32)
        torch.cuda.synchronize()
        _lib.check_status("segment sum long runs")
        assert (a - b[:cnt].cpu()).abs().max() <= 2e-4 * max(a.abs().max().item(), 1.0)
        assert torch.equal(b, sort.segment_sum(src.cuda(), d, torch.float32))               # bit-identical when repeated


def test_embedding_backward_is_deterministic_and_matches_cpu():
    torch.manual_seed(0)
    ids = torch.randint(0, 500, (4000,))
    upstream = torch.randn(4000, 64)
    res = []
    for dev in ("cpu", "cuda", "cuda"):
        t = ShardedEmbedding(500, 64, device=dev, dtype=torch.float32, lr=0.1, seed=3)
        w0 = t.weight.clone()
        out = t.lookup(ids.to(dev))
        (out * upstream.to(dev)).sum().backward()
        res.append((t.weight - w0).cpu())
    torch.cuda.synchronize()
    assert torch.equal(res[1], res[2])
    assert (res[0] - res[1]).abs().max() < 1e-5

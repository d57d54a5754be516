"""Jagged HSTU attention kernels (forward / backward) against the eager fp32 oracle."""
import pytest
import torch

from mlperf_training_b200.ops import _lib
from mlperf_training_b200.ops.hstu_ops import hstu_attention, hstu_attention_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lengths,targets,ctx", [
    ([128], None, 0),
    ([17, 300, 1, 513], None, 0),
    ([64, 257, 130], [1, 1, 1], 0),
    ([200, 40, 384], [1, 3, 2], 8),
])
@pytest.mark.parametrize("via_uvqk", [False, True])
def test_hstu_attention_fwd_bwd(lengths, targets, ctx, via_uvqk):
    torch.manual_seed(sum(lengths))
    H, D, N = 4, 128, 1024
    L = sum(lengths)
    offs = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    nt = None if targets is None else torch.tensor(targets, dtype=torch.int32)
    if via_uvqk:
        uvqk = torch.randn(L, 4 * H * D, device="cuda").bfloat16()
        v = uvqk[:, H * D:2 * H * D].unflatten(-1, (H, D))
        q = uvqk[:, 2 * H * D:3 * H * D].unflatten(-1, (H, D))
        k = uvqk[:, 3 * H * D:].unflatten(-1, (H, D))
    else:
        q, k, v = (torch.randn(L, H, D, device="cuda").bfloat16() for _ in range(3))
    alpha = D ** -0.5
    qg, kg, vg = (t.detach().clone().contiguous().requires_grad_(True) if not via_uvqk else t.detach().requires_grad_(True)
                  for t in (q, k, v))
    out = hstu_attention(qg, kg, vg, offs.cuda(), N, alpha, None if nt is None else nt.cuda(), ctx)
    do = torch.randn_like(out)
    out.backward(do)
    torch.cuda.synchronize()
    _lib.check_status("hstu attention")
    qf, kf, vf = (t.detach().float().cpu().requires_grad_(True) for t in (q, k, v))
    ref = hstu_attention_reference(qf, kf, vf, offs, N, alpha, nt, ctx)
    ref.backward(do.float().cpu())
    sc = ref.abs().max().item() + 1e-9
    assert (out.float().cpu() - ref.detach()).abs().max().item() < 3e-2 * sc + 1e-4
    for name, got, want in (("dq", qg.grad, qf.grad), ("dk", kg.grad, kf.grad), ("dv", vg.grad, vf.grad)):
        g = got.float().cpu()
        s = want.abs().max().item() + 1e-9
        assert (g - want).abs().max().item() < 4e-2 * s + 1e-5, name

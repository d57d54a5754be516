"""tcgen05 flash attention forward / backward against eager fp32 softmax attention."""
import math

import pytest
import torch

from mlperf_training_b200.ops import _lib, kernels

pytestmark = pytest.mark.gpu

CASES = [
    # B, Sq, Skv, Hq, Hkv, D, causal, window, sink
    (1, 128, 128, 1, 1, 128, True, 0, False),
    (2, 256, 256, 4, 2, 128, True, 0, False),
    (1, 384, 384, 2, 1, 64, True, 0, False),
    (2, 200, 200, 2, 2, 128, True, 0, False),
    (1, 512, 512, 4, 1, 64, True, 128, True),
    (1, 640, 640, 2, 1, 128, True, 128, False),
    (2, 512, 512, 3, 3, 128, False, 0, False),
    (1, 1024, 1024, 8, 2, 128, True, 0, True),
]


def _mk(B, Sq, Skv, Hq, Hkv, D, seed):
    torch.manual_seed(seed)
    q = torch.randn(B, Sq, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, Skv, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, Skv, Hkv, D, device="cuda").bfloat16()
    return q, k, v


@pytest.mark.parametrize("B,Sq,Skv,Hq,Hkv,D,causal,window,sink", CASES)
def test_attention_fwd(B, Sq, Skv, Hq, Hkv, D, causal, window, sink):
    q, k, v = _mk(B, Sq, Skv, Hq, Hkv, D, Sq + D)
    sk = torch.randn(Hq, device="cuda") if sink else None
    scale = 1 / math.sqrt(D)
    o, lse = kernels.attention_fwd(q, k, v, scale=scale, causal=causal, window=window, sink=sk)
    torch.cuda.synchronize()
    _lib.check_status("attn fwd")
    o_ref, lse_ref = kernels.attention_reference(q, k, v, scale=scale, causal=causal, window=window, sink=sk)
    err = (o.float() - o_ref).abs().max().item()
    assert err < 2e-2, f"out err {err}"
    assert (lse - lse_ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("B,Sq,Skv,Hq,Hkv,D,causal,window,sink", CASES)
def test_attention_bwd(B, Sq, Skv, Hq, Hkv, D, causal, window, sink):
    q, k, v = _mk(B, Sq, Skv, Hq, Hkv, D, Sq + D + 1)
    sk = torch.randn(Hq, device="cuda") if sink else None
    scale = 1 / math.sqrt(D)
    do = torch.randn(B, Sq, Hq, D, device="cuda").bfloat16()
    o, lse = kernels.attention_fwd(q, k, v, scale=scale, causal=causal, window=window, sink=sk)
    dq, dk, dv, dsink = kernels.attention_bwd(do, q, k, v, o, lse, scale=scale, causal=causal, window=window, sink=sk)
    torch.cuda.synchronize()
    _lib.check_status("attn bwd")
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    sf = None if sk is None else sk.clone().requires_grad_(True)
    o_ref, _ = kernels.attention_reference(qf, kf, vf, scale=scale, causal=causal, window=window, sink=sf)
    o_ref.backward(do.float())
    for name, got, ref in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        err = (got.float() - ref).abs().max().item()
        sc = ref.abs().max().item()
        assert err < 3e-2 * max(sc, 1.0), f"{name}: err {err} scale {sc}"
    if sink:
        assert (dsink - sf.grad).abs().max().item() < 3e-2 * max(sf.grad.abs().max().item(), 1.0)


def test_attention_packed_qkv_views():
    """q/k/v as views into one [B*S, (Hq+2Hkv)*D] buffer, the layout the GPT block uses."""
    torch.manual_seed(9)
    B, S, Hq, Hkv, D = 2, 256, 4, 2, 128
    row = (Hq + 2 * Hkv) * D
    qkv = torch.randn(B * S, row, device="cuda").bfloat16()
    v4 = qkv.view(B, S, row)
    q = v4[:, :, :Hq * D].unflatten(-1, (Hq, D))
    k = v4[:, :, Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
    v = v4[:, :, (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
    o, lse = kernels.attention_fwd(q, k, v, causal=True)
    torch.cuda.synchronize()
    o_ref, _ = kernels.attention_reference(q, k, v, scale=1 / math.sqrt(D), causal=True)
    assert (o.float() - o_ref).abs().max().item() < 2e-2
    _lib.check_status("attn packed")

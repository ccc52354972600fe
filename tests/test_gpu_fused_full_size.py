"""The fused attention kernels at the benchmark's full sizes, where the CPU oracle cannot cover the whole problem:
parity on windows of rows that the oracle CAN afford (a window of queries sees its whole key prefix, which the operator
supports directly as Lq < Lk), plus properties that hold at any size (rows of P sum to one, landmark keys carry no value
weight, linearity in dO, independence of (batch, head) slices, bit-reproducibility)."""
import pytest
import torch

import landmark_attention_b200 as P
from landmark_attention_b200 import _lib as L
from oracle import landmark_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
BLK = 64


def rand(shape, seed, scale=0.5, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def grads(q, k, v, do):
    qc, kc, vc = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qc, kc, vc, None, path=P.PATH_TCGEN05)
    return (out.detach(), *torch.autograd.grad(out, [qc, kc, vc], do))


def test_headline_shape_forward_backward():
    # B=1, H=32, L=2048, D=128 bf16: oracle parity on three of the 32 heads, properties on all of them
    B, H, Lq, D = 1, 32, 2048, 128
    q, k, v, do = rand((B, H, Lq, D), 1), rand((B, H, Lq, D), 2), rand((B, H, Lq, D), 3), rand((B, H, Lq, D), 4, 1.0)
    out, dq, dk, dv = grads(q.to(DEV), k.to(DEV), v.to(DEV), do.to(DEV))
    assert L.device_status() == 0
    for h in (0, 13, 31):
        exp = O.landmark_attention_grads(q[:, h:h + 1].float(), k[:, h:h + 1].float(), v[:, h:h + 1].float(),
                                         do[:, h:h + 1].float(), BLK)
        for name, got, e in zip(("out", "dq", "dk", "dv"), (out, dq, dk, dv), exp):
            g = got[:, h:h + 1].float().cpu()
            assert (g - e).abs().max().item() < 2e-2, (name, h)
            assert ((g - e).norm() / e.norm()).item() < 1e-2, (name, h)
    assert dv[:, :, BLK - 1::BLK].abs().max().item() == 0.0             # landmark keys carry no value weight
    again = grads(q.to(DEV), k.to(DEV), v.to(DEV), do.to(DEV))
    for a, b in zip((out, dq, dk, dv), again):
        assert torch.equal(a, b)                                          # no atomics anywhere
    ones = P.fused_landmark_attention(q.to(DEV), k.to(DEV), torch.ones_like(v).to(DEV), None, path=P.PATH_TCGEN05)
    assert (ones.float() - 1).abs().max().item() < 1e-2                   # rows of P sum to one


@pytest.mark.parametrize("window", [(0, 256), (16384, 256), (32768 - 256, 256)])
def test_long_sequence_windows_against_oracle(window):
    # L = 32768 (the longest point of the sweep): a window of query rows against the oracle on its key prefix, and
    # the window computed on its own (Lq < Lk) against the same rows of the full call
    H, Lk, D = 2, 32768, 128
    r0, n = window
    q, k, v = rand((1, H, Lk, D), 5), rand((1, H, Lk, D), 6), rand((1, H, Lk, D), 7)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    full, l_full, m_full = P.attn_forward_with_stats(qd, kd, vd, BLK, path=P.PATH_TCGEN05)
    assert L.device_status() == 0
    hi = r0 + n
    exp, em, el = O.landmark_attention(q[:, :, r0:hi].float(), k[:, :, :hi].float(), v[:, :, :hi].float(), BLK,
                                       return_stats=True)
    got = full[:, :, r0:hi].float().cpu()
    assert (got - exp).abs().max().item() < 2e-2
    assert ((got - exp).norm() / exp.norm()).item() < 1e-2
    m_rows = m_full.view(1, H, Lk)[:, :, r0:hi].cpu()
    l_rows = l_full.view(1, H, Lk)[:, :, r0:hi].cpu()
    assert (m_rows - em.view_as(m_rows)).abs().max().item() < 2e-3
    assert ((l_rows - el.view_as(l_rows)).abs() / el.view_as(l_rows)).max().item() < 3e-3
    part = P.fused_landmark_attention(qd[:, :, r0:hi].contiguous(), kd[:, :, :hi], vd[:, :, :hi], None,
                                      path=P.PATH_TCGEN05)
    assert (part.float() - full[:, :, r0:hi].float()).abs().max().item() < 4e-3


def test_long_sequence_backward_by_linearity_in_dO():
    # All gradients are linear in dO.  With dO zero outside a window of query rows, dQ, dK and dV of the full call
    # (L = 16384, every key block streams 128 query tiles) must equal the oracle's gradients for that window alone.
    H, Lk, D = 1, 16384, 128
    q, k, v = rand((1, H, Lk, D), 8), rand((1, H, Lk, D), 9), rand((1, H, Lk, D), 10)
    for r0, n in ((Lk - 256, 256), (6144, 128)):
        hi = r0 + n
        do = torch.zeros(1, H, Lk, D, dtype=torch.bfloat16)
        do[:, :, r0:hi] = rand((1, H, n, D), 11, 1.0)
        out, dq, dk, dv = grads(q.to(DEV), k.to(DEV), v.to(DEV), do.to(DEV))
        assert L.device_status() == 0
        _, edq, edk, edv = O.landmark_attention_grads(q[:, :, r0:hi].float(), k[:, :, :hi].float(), v[:, :, :hi].float(),
                                                      do[:, :, r0:hi].float(), BLK)
        dq, dk, dv = dq.float().cpu(), dk.float().cpu(), dv.float().cpu()
        zero = lambda t: t.numel() == 0 or t.abs().max().item() == 0.0
        assert zero(dq[:, :, :r0]) and zero(dq[:, :, hi:])
        assert zero(dk[:, :, hi:]) and zero(dv[:, :, hi:])                                           # causality
        for name, got, e in (("dq", dq[:, :, r0:hi], edq), ("dk", dk[:, :, :hi], edk), ("dv", dv[:, :, :hi], edv)):
            assert (got - e).abs().max().item() < 2e-2, (name, r0)
            assert ((got - e).norm() / e.norm()).item() < 1.5e-2, (name, r0)


def test_batch_head_slices_are_independent():
    # B=8, H=32 (the sweep's batch): every (batch, head) slice equals the same slice computed on its own, bit for bit
    B, H, Lq, D = 8, 32, 1024, 128
    q, k, v, do = [rand((B, H, Lq, D), s).to(DEV) for s in (12, 13, 14, 15)]
    full = grads(q, k, v, do)
    assert L.device_status() == 0
    for b, h in ((0, 0), (3, 17), (7, 31)):
        one = grads(*[t[b:b + 1, h:h + 1].contiguous() for t in (q, k, v, do)])
        for a, f in zip(one, full):
            assert torch.equal(a, f[b:b + 1, h:h + 1])

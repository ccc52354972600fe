"""Parity of the general-path fused landmark attention kernels (through the C ABI) against the CPU oracle and the
golden fixtures recorded from the reference.  Tolerances: fp32 1e-4 max-abs; bf16 2e-2 max-abs and 1e-2 relative L2."""
import math

import pytest
import torch

import landmark_attention_b200 as P
from oracle import landmark_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run_ours(q, k, v, do, blk, path=P.PATH_GENERAL, scale=None):
    q, k, v = [t.to(DEV).detach().requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(q, k, v, None, sm_scale=scale, block_size=blk, path=path)
    dq, dk, dv = torch.autograd.grad(out, [q, k, v], do.to(DEV))
    return [t.detach().float().cpu() for t in (out, dq, dk, dv)]


def rel_l2(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-20)).item()


@pytest.mark.parametrize("name", ["fused_square", "fused_prefix", "fused_blk32", "fused_blk16_d128",
                                  "triton_square", "triton_prefix"])
def test_fp32_against_golden(golden, name):
    g = golden(name + ".pt")
    res = run_ours(g["q"], g["k"], g["v"], g["do"], g["blk"])
    for got, key in zip(res, ("out", "dq", "dk", "dv")):
        assert (got - g[key]).abs().max().item() < 1e-4, key


@pytest.mark.parametrize("name", ["triton_square", "triton_prefix"])
def test_saved_statistics_match_reference_kernel(golden, name):
    g = golden(name + ".pt")
    _, l, m = P.attn_forward_with_stats(g["q"].to(DEV), g["k"].to(DEV), g["v"].to(DEV), g["blk"],
                                        path=P.PATH_GENERAL)
    assert (m.cpu() - g["M"]).abs().max().item() < 1e-5
    assert ((l.cpu() - g["L"]).abs() / g["L"]).max().item() < 1e-5


def test_config1_fp32_against_oracle():
    # B=2, H=8, L=512, D=64, block 64, fp32, mask supplied
    torch.manual_seed(0)
    B, H, Lq, D, blk = 2, 8, 512, 64, 64
    q, k, v, do = [torch.randn(B, H, Lq, D) for _ in range(4)]
    is_mem = O.regular_is_mem(Lq, blk)
    qc, kc, vc = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qc, kc, vc, is_mem.to(DEV), block_size=blk, path=P.PATH_GENERAL)
    dq, dk, dv = torch.autograd.grad(out, [qc, kc, vc], do.to(DEV))
    eo, edq, edk, edv = O.landmark_attention_grads(q.double(), k.double(), v.double(), do.double(), blk)
    for got, exp in ((out, eo), (dq, edq), (dk, edk), (dv, edv)):
        assert (got.detach().cpu().double() - exp).abs().max().item() < 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 2, 256, 256, 128, 64), (2, 2, 64, 192, 64, 32), (1, 1, 96, 96, 32, 48)])
def test_16bit_general_against_oracle(dtype, shape):
    B, H, Lq, Lk, D, blk = shape
    torch.manual_seed(1)
    q = (torch.randn(B, H, Lq, D) * 0.5).to(dtype)
    k = (torch.randn(B, H, Lk, D) * 0.5).to(dtype)
    v = (torch.randn(B, H, Lk, D) * 0.5).to(dtype)
    do = torch.randn(B, H, Lq, D).to(dtype)
    res = run_ours(q, k, v, do, blk)
    exp = O.landmark_attention_grads(q.float(), k.float(), v.float(), do.float(), blk)
    for got, e in zip(res, exp):
        assert (got - e).abs().max().item() < 2e-2
        assert rel_l2(got, e) < 1e-2


def test_forward_ragged_last_block():
    # forward accepts a sequence that ends inside a block (reference kernel masks the tail, :44,:49)
    torch.manual_seed(2)
    B, H, Lq, D, blk = 1, 2, 100, 32, 32
    q, k, v = [torch.randn(B, H, Lq, D) for _ in range(3)]
    out = P.fused_landmark_attention(q.to(DEV), k.to(DEV), v.to(DEV), None, block_size=blk, path=P.PATH_GENERAL)
    # oracle on the sequence padded to whole blocks; rows beyond Lq dropped (causality makes padding invisible)
    pad = 128 - Lq
    qp, kp, vp = [torch.cat((t, torch.zeros(B, H, pad, D)), dim=2) for t in (q, k, v)]
    exp = O.landmark_attention(qp, kp, vp, blk)[:, :, :Lq]
    assert (out.cpu() - exp).abs().max().item() < 1e-4


def test_strided_inputs_are_read_in_place():
    # [B, L, H, D] projections viewed as [B, H, L, D], as the attention modules pass them (llama_mem.py:287-289)
    torch.manual_seed(3)
    B, H, L, D, blk = 2, 3, 128, 32, 32
    q, k, v = [torch.randn(B, L, H, D, device=DEV).transpose(1, 2) for _ in range(3)]
    out = P.fused_landmark_attention(q, k, v, None, block_size=blk, path=P.PATH_GENERAL)
    exp = O.landmark_attention(q.cpu().contiguous(), k.cpu().contiguous(), v.cpu().contiguous(), blk)
    assert (out.cpu() - exp).abs().max().item() < 1e-4


def test_known_answers():
    torch.manual_seed(4)
    B, H, L, D, blk = 1, 2, 256, 64, 64
    q, k = [torch.randn(B, H, L, D, device=DEV) for _ in range(2)]
    # rows of P sum to one: V = 1 gives O = 1
    ones = torch.ones(B, H, L, D, device=DEV)
    out = P.fused_landmark_attention(q, k, ones, None, block_size=blk, path=P.PATH_GENERAL)
    assert (out - 1).abs().max().item() < 1e-5
    # the first row attends to the first key only
    v = torch.randn(B, H, L, D, device=DEV)
    out = P.fused_landmark_attention(q, k, v, None, block_size=blk, path=P.PATH_GENERAL)
    assert (out[:, :, 0] - v[:, :, 0]).abs().max().item() < 1e-6
    # landmark keys carry no value weight: dV at landmark rows is exactly zero
    v.requires_grad_(True)
    out = P.fused_landmark_attention(q, k, v, None, block_size=blk, path=P.PATH_GENERAL)
    (dv,) = torch.autograd.grad(out.sum(), [v])
    assert dv[:, :, blk - 1::blk].abs().max().item() == 0.0
    # a single block is a plain causal softmax with the last key hidden and the last query shifted back by one
    q1, k1, v1 = [torch.randn(1, 1, blk, D, device=DEV) for _ in range(3)]
    out = P.fused_landmark_attention(q1, k1, v1, None, block_size=blk, path=P.PATH_GENERAL)
    s = (q1 @ k1.transpose(-1, -2)) / math.sqrt(D)
    pos = torch.arange(blk, device=DEV)
    pos_q = torch.where(pos == blk - 1, pos - 1, pos)
    s = s.masked_fill(~(pos_q[:, None] >= pos[None, :]), float("-inf"))
    assert (out - torch.softmax(s, -1) @ v1).abs().max().item() < 1e-5


def test_backward_is_bit_reproducible():
    torch.manual_seed(5)
    B, H, L, D, blk = 1, 2, 256, 64, 64
    q, k, v, do = [torch.randn(B, H, L, D) for _ in range(4)]
    a = run_ours(q, k, v, do, blk)
    b = run_ours(q, k, v, do, blk)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_reference_assertions_are_kept():
    q = torch.randn(1, 1, 64, 64, device=DEV)
    bad_mask = torch.zeros(64, dtype=torch.bool, device=DEV)
    with pytest.raises(AssertionError):
        P.fused_landmark_attention(q, q, q, bad_mask, block_size=64)
    with pytest.raises(AssertionError):
        P.fused_landmark_attention(q, q.half(), q, None, block_size=64)
    qr = torch.randn(1, 1, 96, 32, device=DEV, requires_grad=True)
    out = P.fused_landmark_attention(qr, qr, qr, None, block_size=64, path=P.PATH_GENERAL)   # ragged forward is fine
    with pytest.raises(AssertionError):
        out.sum().backward()                                                                 # backward is not

"""Fused landmark attention with arbitrary landmark positions (lmk_attn_mask_fwd / lmk_attn_mask_bwd, through the C ABI
via the registered operator) against the CPU oracle's lm_attention, which is pinned to the reference's
CausalSelfAttention.forward by tests/golden/lm_attn.pt.  bf16/fp16 tolerances: 2e-2 max-abs, 1e-2 relative L2."""
import pytest
import torch

import landmark_attention_b200 as P
from landmark_attention_b200 import _lib as L
from oracle import landmark_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_l2(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-20)).item()


def window_is_mem(B, T, g, block=51):
    """Landmark after every block-1 tokens of a long stream, windows cut at random offsets (optim/utils.py:21-26)."""
    im = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        off = int(torch.randint(0, block, (1,), generator=g))
        im[b] = (torch.arange(T) + off) % block == block - 1
    return im


def irregular_is_mem(B, T, g, lo=1, hi=9):
    im = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        p = int(torch.randint(0, hi, (1,), generator=g))
        while p < T:
            im[b, p] = True
            p += int(torch.randint(lo, hi, (1,), generator=g))
    return im


def make(B, H, T, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = [(torch.randn(B, H, T, 128, generator=g) * 0.5).to(dtype) for _ in range(3)]
    do = torch.randn(B, H, T, 128, generator=g).to(dtype)
    return g, q, k, v, do


def oracle(q, k, v, do, im):
    qf, kf, vf = [t.float().requires_grad_(True) for t in (q, k, v)]
    out = O.lm_attention(qf, kf, vf, im)
    grads = torch.autograd.grad(out, [qf, kf, vf], do.float())
    return (out.detach(), *grads)


def run(q, k, v, do, im, max_groups):
    qc, kc, vc = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.landmark_attention_masked(qc, kc, vc, im.to(DEV), max_groups=max_groups)
    grads = torch.autograd.grad(out, [qc, kc, vc], do.to(DEV))
    torch.cuda.synchronize()
    return [t.detach().float().cpu() for t in (out, *grads)]


def compare(got, exp, what):
    for name, a, e in zip(("out", "dq", "dk", "dv"), got, exp):
        assert torch.isfinite(a).all(), f"{what}: {name} not finite"
        tol = 2e-2 * max(1.0, e.abs().max().item())
        assert (a - e).abs().max().item() < tol, f"{what}: {name} max-abs {(a - e).abs().max().item()}"
        assert rel_l2(a, e) < 1e-2, f"{what}: {name} rel-L2 {rel_l2(a, e)}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,T", [(2, 2, 128), (2, 1, 256), (1, 2, 512)])
def test_training_windows_block_51(B, H, T, dtype):
    g, q, k, v, do = make(B, H, T, dtype, 100 + T)
    im = window_is_mem(B, T, g)
    compare(run(q, k, v, do, im, 16), oracle(q, k, v, do, im), f"T={T}")
    assert L.device_status() == 0


def test_irregular_and_adjacent_landmarks():
    # groups of 0..8 keys: adjacent landmarks (empty groups), a landmark on key 0, many groups per 64-key tile
    B, H, T = 3, 2, 256
    g, q, k, v, do = make(B, H, T, torch.bfloat16, 7)
    im = irregular_is_mem(B, T, g)
    im[0, 0] = True
    im[1, 10:13] = True
    n_groups = int(im.sum(-1).max())
    assert n_groups <= 64
    compare(run(q, k, v, do, im, 64), oracle(q, k, v, do, im), "irregular")
    assert L.device_status() == 0


def test_no_landmarks_is_plain_causal_attention():
    B, H, T = 1, 2, 256
    g, q, k, v, do = make(B, H, T, torch.bfloat16, 9)
    im = torch.zeros(B, T, dtype=torch.bool)
    got = run(q, k, v, do, im, 4)
    qf, kf, vf = [t.float().requires_grad_(True) for t in (q, k, v)]
    ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True)
    grads = torch.autograd.grad(ref, [qf, kf, vf], do.float())
    compare(got, (ref.detach(), *grads), "no landmarks")


def test_regular_pattern_matches_fused_fast_path():
    # with a landmark at the end of every 64-key block the general kernels and the regular-pattern kernels agree
    B, H, T = 1, 2, 512
    g, q, k, v, do = make(B, H, T, torch.bfloat16, 11)
    im = (torch.arange(T) % 64 == 63).view(1, T).expand(B, T).contiguous()
    got = run(q, k, v, do, im, 16)
    qc, kc, vc = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qc, kc, vc, None, block_size=64)
    grads = torch.autograd.grad(out, [qc, kc, vc], do.to(DEV))
    for a, e in zip(got, (out, *grads)):
        e = e.detach().float().cpu()
        assert (a - e).abs().max().item() < 2e-2 * max(1.0, e.abs().max().item())


def test_lm_benchmark_training_shape():
    # B=16, H=8, T=512, D=128, landmark every 51 tokens at seeded random window offsets; the oracle runs on two heads
    B, H, T = 16, 8, 512
    g, q, k, v, do = make(B, H, T, torch.bfloat16, 3)
    im = window_is_mem(B, T, g)
    got = run(q, k, v, do, im, 16)
    exp = oracle(q[:, 2:4], k[:, 2:4], v[:, 2:4], do[:, 2:4], im)
    compare([t[:, 2:4] for t in got], exp, "training shape")
    # bitwise reproducible (no atomics anywhere)
    again = run(q, k, v, do, im, 16)
    for a, b in zip(got, again):
        assert torch.equal(a, b)
    assert L.device_status() == 0


def test_call_site_uses_the_fused_operator_and_compiles():
    B, H, T = 2, 2, 256
    g, q, k, v, do = make(B, H, T, torch.bfloat16, 5)
    im = window_is_mem(B, T, g).to(DEV)

    class Attn(torch.nn.Module):
        def forward(self, q, k, v, im):
            return P.lm_landmark_attention(q, k, v, im, max_groups=16)

    qc, kc, vc = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    eager = Attn()(qc, kc, vc, im)
    ge = torch.autograd.grad(eager, [qc, kc, vc], do.to(DEV))
    compiled = torch.compile(Attn(), fullgraph=True)
    out = compiled(qc, kc, vc, im)
    gc = torch.autograd.grad(out, [qc, kc, vc], do.to(DEV))
    assert torch.equal(out, eager)
    for a, b in zip(gc, ge):
        assert torch.equal(a, b)


def test_too_many_landmarks_is_reported_not_hidden():
    B, H, T = 1, 1, 128
    g, q, k, v, do = make(B, H, T, torch.bfloat16, 6)
    im = torch.zeros(B, T, dtype=torch.bool)
    im[0, ::4] = True                       # 32 landmarks, statistics for 8
    L.device_status()
    P.landmark_attention_masked(q.to(DEV), k.to(DEV), v.to(DEV), im.to(DEV), max_groups=8)
    assert L.device_status() == 431
    with pytest.raises(NotImplementedError):
        P.landmark_attention_masked(q.to(DEV), k.to(DEV), v.to(DEV), im.to(DEV), max_groups=65)


@pytest.mark.parametrize("B,H,Lq,Lk,blk", [(1, 2, 512, 512, 32), (2, 2, 256, 384, 16), (1, 2, 1024, 1024, 128),
                                           (1, 1, 2048, 2048, 32)])
def test_fused_entry_with_other_block_sizes_runs_on_these_kernels(B, H, Lq, Lk, blk):
    # fused_landmark_attention(block_size != 64) routes 16-bit head-dim-128 problems to the arbitrary-landmark
    # tensor-core kernels (regular flags); result against the oracle of the fused operator, with history keys
    g = torch.Generator().manual_seed(Lk + blk)
    q = (torch.randn(B, H, Lq, 128, generator=g) * 0.5).to(torch.bfloat16)
    k, v = [(torch.randn(B, H, Lk, 128, generator=g) * 0.5).to(torch.bfloat16) for _ in range(2)]
    do = torch.randn(B, H, Lq, 128, generator=g).to(torch.bfloat16)
    eo, edq, edk, edv = O.landmark_attention_grads(q.float(), k.float(), v.float(), do.float(), blk)
    qd, kd, vd = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qd, kd, vd, None, block_size=blk)
    assert "FusedLandmarkAttention" not in type(out.grad_fn).__name__      # not the block-64 / general entry
    dq, dk, dv = torch.autograd.grad(out, [qd, kd, vd], do.to(DEV))
    for got, exp in ((out, eo), (dq, edq), (dk, edk), (dv, edv)):
        got = got.float().cpu()
        assert torch.isfinite(got).all()
        assert (got - exp).abs().max().item() < 3e-2 and rel_l2(got, exp) < 1e-2
    assert L.device_status() == 0


@pytest.mark.parametrize("D,blk,Lq,Lk", [(64, 64, 256, 384), (64, 32, 256, 256), (96, 64, 128, 128), (32, 16, 128, 192)])
def test_fused_entry_with_smaller_head_dims_runs_on_tensor_cores(D, blk, Lq, Lk):
    # 16-bit head dims below 128 are zero-padded to 128 and run on the tensor-core kernels (block 64: lmk_attn_fwd/bwd,
    # other blocks: the arbitrary-landmark kernels); the default scale stays 1/sqrt(D) of the real head dim
    g = torch.Generator().manual_seed(D + blk)
    B, H = 2, 2
    q = (torch.randn(B, H, Lq, D, generator=g) * 0.5).to(torch.bfloat16)
    k, v = [(torch.randn(B, H, Lk, D, generator=g) * 0.5).to(torch.bfloat16) for _ in range(2)]
    do = torch.randn(B, H, Lq, D, generator=g).to(torch.bfloat16)
    eo, edq, edk, edv = O.landmark_attention_grads(q.float(), k.float(), v.float(), do.float(), blk)
    qd, kd, vd = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qd, kd, vd, None, block_size=blk)
    assert out.shape == (B, H, Lq, D)
    assert "FusedLandmarkAttention" not in type(out.grad_fn).__name__          # a slice of the padded problem's output
    dq, dk, dv = torch.autograd.grad(out, [qd, kd, vd], do.to(DEV))
    general = P.fused_landmark_attention(qd, kd, vd, None, block_size=blk, path=P.PATH_GENERAL)
    assert (out.float() - general.float()).abs().max().item() < 2e-2
    for got, exp in ((out, eo), (dq, edq), (dk, edk), (dv, edv)):
        got = got.float().cpu()
        assert got.shape == exp.shape and torch.isfinite(got).all()
        assert (got - exp).abs().max().item() < 3e-2 and rel_l2(got, exp) < 1e-2
    assert L.device_status() == 0


@pytest.mark.parametrize("D,blk,Lq,Lk", [(128, 64, 200, 200), (128, 64, 130, 258), (64, 64, 1000, 1000), (128, 32, 100, 164)])
def test_fused_entry_with_ragged_lengths_runs_on_tensor_cores(D, blk, Lq, Lk):
    # 16-bit problems whose lengths are not whole tiles are padded with zero rows at the end (hidden by causality) and
    # run on the tensor-core kernels; forward and backward against the oracle on the unpadded problem
    g = torch.Generator().manual_seed(Lq + Lk)
    B, H = 1, 2
    q = (torch.randn(B, H, Lq, D, generator=g) * 0.5).to(torch.bfloat16)
    k, v = [(torch.randn(B, H, Lk, D, generator=g) * 0.5).to(torch.bfloat16) for _ in range(2)]
    do = torch.randn(B, H, Lq, D, generator=g).to(torch.bfloat16)
    pad = -Lk % blk                                   # the oracle works on whole blocks: same trick, on its side
    kf, vf = [torch.nn.functional.pad(t.float(), (0, 0, 0, pad)) for t in (k, v)]
    qf, dof = [torch.nn.functional.pad(t.float(), (0, 0, 0, pad)) for t in (q, do)]
    eo, edq, edk, edv = O.landmark_attention_grads(qf, kf, vf, dof, blk)
    eo, edq, edk, edv = eo[:, :, :Lq], edq[:, :, :Lq], edk[:, :, :Lk], edv[:, :, :Lk]
    qd, kd, vd = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qd, kd, vd, None, block_size=blk)
    assert out.shape == (B, H, Lq, D) and "FusedLandmarkAttention" not in type(out.grad_fn).__name__
    dq, dk, dv = torch.autograd.grad(out, [qd, kd, vd], do.to(DEV))
    for got, exp in ((out, eo), (dq, edq), (dk, edk), (dv, edv)):
        got = got.float().cpu()
        assert got.shape == exp.shape and torch.isfinite(got).all()
        assert (got - exp).abs().max().item() < 3e-2 and rel_l2(got, exp) < 1e-2
    assert L.device_status() == 0

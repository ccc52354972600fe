"""Kernel-level timing of the fused attention entry points through the C ABI (no autograd, no allocation in the loop).

    python kernel_bench.py --L 2048 --B 1 --H 32 [--path 2] [--iters 30] [--only fwd|bwd]

Prints one line with the average device time of lmk_attn_fwd and lmk_attn_bwd (CUDA events around back-to-back
calls) and the algorithmic TFLOP/s (2*B*H*L^2*D forward, 5*B*H*L^2*D backward).  This is the command the ncu
summaries under profiles/ were captured with.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from landmark_attention_b200 import _lib as L  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--L", type=int, default=2048)
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--D", type=int, default=128)
    ap.add_argument("--block", type=int, default=64)
    ap.add_argument("--path", type=int, default=L.PATH_AUTO)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--only", default="both", choices=["both", "fwd", "bwd"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--masked", action="store_true",
                    help="time the arbitrary-landmark fused attention (lmk_attn_mask_fwd / _bwd) instead: a landmark after "
                         "every block-1 tokens at a different random window offset per batch row")
    ap.add_argument("--grouped-softmax", action="store_true",
                    help="time the stand-alone grouped softmax (forward and backward) on [B,H,L,L] fp32 logits instead")
    a = ap.parse_args()
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    dev = torch.device("cuda")
    if a.grouped_softmax:
        return grouped_softmax_bench(a, dev)
    if a.masked:
        return masked_bench(a, dt, dev)
    g = torch.Generator().manual_seed(0)
    B, H, Lq, D = a.B, a.H, a.L, a.D
    q, k, v = [(torch.randn(B, H, Lq, D, generator=g) * 0.5).to(dt).to(dev) for _ in range(3)]
    do = torch.randn(B, H, Lq, D, generator=g).to(dt).to(dev)
    o = torch.empty_like(q)
    l = torch.empty(B * H, Lq, device=dev)
    m = torch.empty(B * H, Lq, device=dev)
    dq, dk, dv = [torch.empty_like(q) for _ in range(3)]
    lib = L.lib()
    code = L.dtype_code(q)
    need = lib.lmk_attn_bwd_workspace(B, H, Lq, Lq, D, a.block, code, a.path)
    ws = torch.empty(max(int(need), 256), dtype=torch.uint8, device=dev)
    st, s3 = L.stream_ptr(dev), L.strides3(q)
    scale = D ** -0.5

    def fwd():
        L.check(lib.lmk_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(l), L.ptr(m), B, H, Lq, Lq, D, s3, s3, s3,
                                 a.block, scale, code, a.path, st), "lmk_attn_fwd")

    def bwd():
        L.check(lib.lmk_attn_bwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(do), L.ptr(l), L.ptr(m), L.ptr(dq),
                                 L.ptr(dk), L.ptr(dv), L.ptr(ws), ws.numel(), B, H, Lq, Lq, D, s3, s3, s3, a.block,
                                 scale, code, a.path, st), "lmk_attn_bwd")

    def timeit(f):
        for _ in range(a.warmup):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters * 1e3

    fwd()
    fl = B * H * Lq * Lq * D
    parts = [f"B={B} H={H} L={Lq} D={D} {a.dtype}"]
    if a.only in ("both", "fwd"):
        t = timeit(fwd)
        parts.append(f"fwd {t:.1f} us ({2 * fl / t / 1e6:.0f} TFLOP/s)")
    if a.only in ("both", "bwd"):
        t = timeit(bwd)
        parts.append(f"bwd {t:.1f} us ({5 * fl / t / 1e6:.0f} TFLOP/s)")
    parts.append(f"status {L.device_status()}")
    print("  ".join(parts))


def masked_bench(a, dt, dev):
    """Forward and backward of the arbitrary-landmark operator through its registered ops (one C-ABI call each)."""
    from landmark_attention_b200.masked import _bwd, _fwd
    B, H, T, D = a.B, a.H, a.L, a.D
    g = torch.Generator().manual_seed(0)
    q, k, v = [(torch.randn(B, H, T, D, generator=g) * 0.5).to(dt).to(dev) for _ in range(3)]
    do = torch.randn(B, H, T, D, generator=g).to(dt).to(dev)
    offs = torch.randint(0, a.block, (B,), generator=g)
    im = ((torch.arange(T).view(1, T) + offs.view(B, 1)) % a.block == a.block - 1).to(dev)
    groups = min(64, T // a.block + 2)
    scale = D ** -0.5
    o, R, A = _fwd(q, k, v, im, scale, groups)

    def timeit(f):
        for _ in range(a.warmup):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters * 1e3

    fl = B * H * T * T * D
    t_f = timeit(lambda: _fwd(q, k, v, im, scale, groups))
    t_b = timeit(lambda: _bwd(q, k, v, im, o, do, R, A, scale, groups))
    print(f"masked B={B} H={H} T={T} D={D} landmark every {a.block} {a.dtype}  fwd {t_f:.1f} us ({2 * fl / t_f / 1e6:.0f} TFLOP/s)  "
          f"bwd {t_b:.1f} us ({5 * fl / t_b / 1e6:.0f} TFLOP/s)  status {L.device_status()}")


def grouped_softmax_bench(a, dev):
    """Training-shaped call of the lm_benchmark flavour through the C ABI: causal mask, a landmark after every
    `block - 1` tokens, fp32 logits [B,H,L,L]; reports achieved GB/s of algorithmic bytes (forward: read x, write probs;
    backward: read x and grad, write grad; masks are broadcast views of [1,1,L,L] bytes)."""
    from landmark_attention_b200.grouped_softmax import _prep, prepare_landmark_masks
    B, H, Lq = a.B, a.H, a.L
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B, H, Lq, Lq, generator=g).to(dev)
    is_mem_row = (torch.arange(Lq, device=dev) % a.block == a.block - 1).view(1, Lq)
    hidden = torch.ones(Lq, Lq, dtype=torch.bool, device=dev).triu(1)
    mask, is_mem, last = prepare_landmark_masks(is_mem_row, hidden)
    x.masked_fill_(mask, float("-inf"))            # as the call site does (lm_benchmark/models/landmark.py:224)
    grad = torch.randn(B, H, Lq, Lq, generator=g).to(dev)
    probs, gx = torch.empty_like(x), torch.empty_like(x)
    max_groups = Lq // a.block + 2
    x, ((m8, ms), (l8, ls), (h8, hs)) = _prep(x, is_mem, last, mask)
    lib, st = L.lib(), L.stream_ptr(dev)

    def fwd():
        L.check(lib.lmk_grouped_softmax_fwd(L.ptr(x), L.strides3(x), L.ptr(m8), ms, L.ptr(l8), ls, L.ptr(h8), hs,
                                            L.ptr(probs), None, 0, B, H, Lq, Lq, L.dtype_code(x), 1, max_groups, st),
                "lmk_grouped_softmax_fwd")

    def bwd():
        L.check(lib.lmk_grouped_softmax_bwd(L.ptr(x), L.strides3(x), L.ptr(m8), ms, L.ptr(l8), ls, L.ptr(h8), hs,
                                            L.ptr(grad), L.ptr(gx), B, H, Lq, Lq, L.dtype_code(x), 1, max_groups, st),
                "lmk_grouped_softmax_bwd")

    def timeit(f):
        for _ in range(a.warmup):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters * 1e3

    t_f, t_b = timeit(fwd), timeit(bwd)
    nbytes = x.numel() * 4
    print(f"grouped softmax B={B} H={H} L={Lq} block={a.block} fp32  fwd {t_f:.1f} us ({2 * nbytes / t_f / 1e3:.0f} GB/s)  "
          f"bwd {t_b:.1f} us ({3 * nbytes / t_b / 1e3:.0f} GB/s)")


if __name__ == "__main__":
    main()

"""Time the reference's own GPU code (staged under oracle/_ref/, see make_ref.py) on this machine's GPU.
TEST INFRASTRUCTURE ONLY: it runs none of this repository's kernels.

    python oracle/time_ref_gpu.py [--out ref_gpu.json] [--sweep]

What is timed (CUDA events, seeded inputs of the benchmark's shapes):
  * the reference's Triton kernels through its public `fused_landmark_attention` (forward, forward+backward) at the
    headline shape B=1 H=32 L=2048 D=128 bf16, with parity against its own high-level path in fp32;
  * the reference's high-level PyTorch path on the GPU at the same shape (bf16), and
    torch.nn.functional.scaled_dot_product_attention(is_causal=True) as context;
  * with --sweep, the Triton kernels at L = 4096 and 8192 with B*H = 32 (the reference's backward kernel runs one
    program per (batch, head), so longer sequences or more heads take minutes per call and are left out).
Every section is wrapped: a compile or launch error is recorded as text instead of stopping the run.
"""
import argparse
import json
import os
import sys
import time
import traceback

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import ref_runner as R  # noqa: E402


def cuda_time(fn, warm, iters):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return dict(ms_min=ts[0], ms_median=ts[len(ts) // 2])


def flops(B, H, L, D):
    return 2 * B * H * L * L * D, 7 * B * H * L * L * D


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="ref_gpu.json", help="where the JSON record goes (default: the working directory)")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--retrieval", action="store_true",
                    help="also time the reference's own LlamaAttention.forward cache branch (llama/llama_mem.py:318-430) for "
                         "one layer at the long-context shape: 32 heads of 128, cache 32768 tokens in blocks of 32, chunk 258, top-4")
    ap.add_argument("--config3", action="store_true",
                    help="also time one optimizer step of the reference's own lm_benchmark GPT (models/landmark.py GPTBase) "
                         "at 12 layers, n_embd 1024, 8 heads, seq 512, batch 16, bf16 autocast, on one GPU")
    a = ap.parse_args()
    res = {"env": dict(torch=torch.__version__, gpu=torch.cuda.get_device_name(0), staged=R.available())}
    try:
        import triton
        res["env"]["triton"] = triton.__version__
    except Exception as e:      # noqa: BLE001
        res["env"]["triton"] = repr(e)

    def save():
        if os.path.dirname(a.out):
            os.makedirs(os.path.dirname(a.out), exist_ok=True)
        with open(a.out, "w") as f:
            json.dump(res, f, indent=1, default=str)

    if not R.available():
        res["error"] = "oracle/_ref is not staged"
        save()
        print(json.dumps(res))
        return
    dev = "cuda"
    fla = R.triton_kernels()

    def case(B, H, L, D, blk, iters, with_highlevel):
        out = {}
        g = torch.Generator(device=dev).manual_seed(0)
        q, k, v = [(torch.randn(B, H, L, D, device=dev, generator=g) * 0.5).to(torch.bfloat16).requires_grad_(True)
                   for _ in range(3)]
        do = torch.randn(B, H, L, D, device=dev, generator=g).to(torch.bfloat16)
        is_mem = torch.arange(L, device=dev) % blk == blk - 1
        ff, ft = flops(B, H, L, D)

        def t_fwd():
            with torch.no_grad():
                return fla.fused_landmark_attention(q, k, v, is_mem, block_size=blk)

        def t_fb():
            o = fla.fused_landmark_attention(q, k, v, is_mem, block_size=blk)
            return torch.autograd.grad(o, [q, k, v], do)

        try:
            t0 = time.perf_counter()
            o = fla.fused_landmark_attention(q, k, v, is_mem, block_size=blk)
            gr = torch.autograd.grad(o, [q, k, v], do)
            torch.cuda.synchronize()
            out["first_call_s"] = time.perf_counter() - t0
            if with_highlevel:
                qf, kf, vf = [t.detach().float() for t in (q, k, v)]
                exp = R.highlevel_fwd_bwd(qf[:, :4], kf[:, :4], vf[:, :4], do.float()[:, :4], blk)
                got = (o[:, :4], gr[0][:, :4], gr[1][:, :4], gr[2][:, :4])
                out["triton_bf16_vs_highlevel_fp32_max_abs_4_heads"] = {
                    n: (x.float() - e).abs().max().item() for n, x, e in zip(("out", "dq", "dk", "dv"), got, exp)}
            r = cuda_time(t_fwd, 3, iters)
            r["tflops_at_median"] = ff / (r["ms_median"] * 1e-3) / 1e12
            out["triton_fwd"] = r
            r = cuda_time(t_fb, 3, iters)
            r["tflops_at_median"] = ft / (r["ms_median"] * 1e-3) / 1e12
            out["triton_fwd_bwd"] = r
        except Exception:       # noqa: BLE001
            out["triton_error"] = traceback.format_exc()[-2000:]
        if with_highlevel:
            try:
                def t_hi():
                    o = R.highlevel_attention(q, k, v, blk)
                    return torch.autograd.grad(o, [q, k, v], do)
                r = cuda_time(t_hi, 2, 5)
                r["tflops_at_median"] = ft / (r["ms_median"] * 1e-3) / 1e12
                out["highlevel_bf16_gpu_fwd_bwd"] = r
            except Exception:   # noqa: BLE001
                out["highlevel_error"] = traceback.format_exc()[-2000:]
            try:
                def t_sdpa():
                    o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
                    return torch.autograd.grad(o, [q, k, v], do)
                r = cuda_time(t_sdpa, 3, iters)
                r["tflops_at_median"] = ft / (r["ms_median"] * 1e-3) / 1e12
                out["torch_sdpa_causal_fwd_bwd"] = r
            except Exception:   # noqa: BLE001
                out["sdpa_error"] = traceback.format_exc()[-2000:]
        return out

    res["B1_H32_L2048_D128_bf16"] = case(1, 32, 2048, 128, 64, 10, True)
    save()
    print(json.dumps(res["B1_H32_L2048_D128_bf16"]), flush=True)
    if a.sweep:
        for L in (4096, 8192):
            res[f"B1_H32_L{L}_D128_bf16"] = case(1, 32, L, 128, 64, 3, False)
            save()
            print(L, json.dumps(res[f"B1_H32_L{L}_D128_bf16"]), flush=True)
    if a.retrieval:
        try:
            res["retrieval_reference_layer"] = retrieval_layer(dev)
        except Exception:       # noqa: BLE001
            res["retrieval_reference_layer"] = traceback.format_exc()[-2000:]
        print(json.dumps(res["retrieval_reference_layer"]), flush=True)
        save()
    if a.config3:
        try:
            res["config3_reference_gpt"] = config3(dev)
        except Exception:       # noqa: BLE001
            res["config3_reference_gpt"] = traceback.format_exc()[-2000:]
        print(json.dumps(res["config3_reference_gpt"]), flush=True)
    save()


def retrieval_layer(dev):
    """One LlamaAttention layer of the reference with a filled cache, driven the way LlamaModel.forward drives it
    (mask construction of llama/llama_mem.py:36-50 and :804-815, then LlamaAttention.forward with cache_top_k / mem_freq)."""
    lm = R.llama_mem()
    from llama_landmark_config import LlamaLandmarkConfig
    H, D, C, T, blk, top_k = 32, 128, 32768, 258, 32, 4
    cfg = LlamaLandmarkConfig(hidden_size=H * D, num_attention_heads=H, num_hidden_layers=1, intermediate_size=11008,
                              max_position_embeddings=C + T + 8, vocab_size=32001, mem_freq=blk - 1)
    torch.manual_seed(0)
    attn = lm.LlamaAttention(cfg).to(dev).to(torch.bfloat16).eval()
    g = torch.Generator(device=dev).manual_seed(7)
    pk = torch.randn(1, H, C, D, generator=g, device=dev).to(torch.bfloat16)
    pv = torch.randn(1, H, C, D, generator=g, device=dev).to(torch.bfloat16)
    hidden = torch.randn(1, T, H * D, generator=g, device=dev).to(torch.bfloat16)
    position_ids = torch.arange(C, C + T, device=dev).view(1, T)
    is_mem_row = (position_ids % blk == blk - 1)
    fmin = torch.finfo(torch.bfloat16).min

    def masks():
        mask = torch.full((T, T), fmin, device=dev, dtype=torch.bfloat16).triu(1)
        mask = torch.cat([torch.zeros(T, C, dtype=torch.bfloat16, device=dev), mask], dim=-1)[None, None]
        is_mem = is_mem_row.unsqueeze(1).unsqueeze(2)
        mem_ids = torch.where(mask[..., -T:] < -1, 0, torch.cumsum(is_mem, -1) - is_mem.int())
        last = torch.amax(mem_ids, -1, keepdim=True) == mem_ids
        mask = mask.clone()
        mask[..., -T:].masked_fill_(last & is_mem, fmin)
        last = last.logical_and(mask[..., -T:] > -1)
        is_mem = is_mem.logical_and(mask[..., -T:] > -1)
        return mask, is_mem, last

    def layer():
        with torch.no_grad():
            mask, is_mem, last = masks()
            return attn(hidden, attention_mask=mask, position_ids=position_ids, past_key_value=(pk, pv), use_cache=True,
                        is_mem=is_mem, last_section_mask=last, cache_top_k=top_k, mem_freq=blk - 1)[0]

    out = layer()
    r = cuda_time(layer, 2, 5)
    r["tok_per_s_32_layers"] = 250.0 / (32 * r["ms_median"] * 1e-3)
    r["what"] = ("reference LlamaAttention.forward, cache branch, one layer incl. its q/k/v/o projections and mask "
                 "preparation, bf16, H=32 D=128 cache 32768 block 32 chunk 258 top-4 per (head, token)")
    r["finite"] = bool(torch.isfinite(out.float()).all())
    return r


def config3(dev):
    """The reference's GPTBase with its own attention (score matrix, mask block, grouped softmax), same data, optimizer
    and step loop as bench.py's config 3 entry."""
    import types
    import bench_lm
    lm = R.lm_landmark()
    c = bench_lm.CONFIG
    cfg = types.SimpleNamespace(vocab_size=c["vocab_size"], n_embd=c["n_embd"], n_head=c["n_head"], n_layer=c["n_layer"],
                                sequence_length=c["sequence_length"], dropout=0.0, bias=False, positional_encoder="rotary",
                                softmax_func="mem_opt", lm_cache="none", postpone_lm_cache=True,
                                max_groups_for_softmax=c["max_groups_for_softmax"], group_dropout=None,
                                enable_rem_score=False, landmark_id=bench_lm.LANDMARK_ID, mem_freq=c["mem_freq"],
                                mem_cache_freq=None)
    torch.manual_seed(5)
    ref = lm.GPTBase(cfg).to(dev)

    class Wrap(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, x, y):
            return self.m(x, targets=y)["loss"]

    out = bench_lm.train_step_bench(Wrap(ref), c, 1, 0, torch.device(dev), 5, 2, lambda w: None, lambda x, w, d: x)
    return {"what": "reference GPTBase (lm_benchmark/models/landmark.py) training step, eager (no torch.compile), 1 GPU",
            "tokens_per_s": out["tokens_per_s"], "ms_per_step": out["ms_per_step"], "loss_first": out["loss_first"],
            "loss_last": out["loss_last"]}


if __name__ == "__main__":
    main()

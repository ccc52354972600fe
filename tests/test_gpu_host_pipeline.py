"""The host-memory pipeline (chunked heads, copies overlapped with kernels) gives exactly what the device-resident call gives."""
import pytest
import torch

import landmark_attention_b200 as P

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunks", [1, 2, 4])
def test_host_pipeline_matches_device_call(chunks):
    g = torch.Generator().manual_seed(21)
    B, H, L, D = 1, 8, 256, 128
    host = [(torch.randn(B, H, L, D, generator=g) * 0.5).to(torch.bfloat16).pin_memory() for _ in range(3)]
    host.append(torch.randn(B, H, L, D, generator=g).to(torch.bfloat16).pin_memory())
    outs = [torch.empty(B, H, L, D, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    pipe = P.HostAttentionPipeline(B, H, L, L, D, torch.bfloat16, 64, chunks=chunks)
    for _ in range(2):                                   # second run reuses the device buffers
        pipe.run(*host, *outs)
        torch.cuda.synchronize()
    q, k, v = [t.cuda().requires_grad_(True) for t in host[:3]]
    o = P.fused_landmark_attention(q, k, v, None)
    grads = torch.autograd.grad(o, [q, k, v], host[3].cuda())
    for got, exp in zip(outs, (o, *grads)):
        assert torch.equal(got, exp.detach().cpu())


@pytest.mark.parametrize("chunks", [1, 2, 4])
def test_overlapped_steps_keep_their_problems_apart(chunks):
    # run(wait=False): consecutive steps share the rotating device buffers through events; five different problems in a
    # row, each with its own pinned outputs, must all come out as the device-resident call computes them
    g = torch.Generator().manual_seed(22)
    B, H, L, D, n = 1, 8, 256, 128, 5
    pipe = P.HostAttentionPipeline(B, H, L, L, D, torch.bfloat16, 64, chunks=chunks)
    problems, results = [], []
    for _ in range(n):
        problems.append([(torch.randn(B, H, L, D, generator=g) * 0.5).to(torch.bfloat16).pin_memory() for _ in range(4)])
        results.append([torch.zeros(B, H, L, D, dtype=torch.bfloat16).pin_memory() for _ in range(4)])
    last = None
    for host, outs in zip(problems, results):
        last = pipe.run(*host, *outs, wait=False)
    last.synchronize()                                   # the copies leave in order: the last one covers them all
    for host, outs in zip(problems, results):
        q, k, v = [t.cuda().requires_grad_(True) for t in host[:3]]
        o = P.fused_landmark_attention(q, k, v, None)
        grads = torch.autograd.grad(o, [q, k, v], host[3].cuda())
        for got, exp in zip(outs, (o, *grads)):
            assert torch.equal(got, exp.detach().cpu())

"""Training step of the lm_benchmark landmark GPT (BASELINE config 3) for bench.py: data-parallel over the ranks with
NCCL gradient all-reduce (torch DistributedDataParallel, as lm_benchmark/distributed/ddp.py:48-55 does).

The model below has the architecture, initialisation and loss of the reference's GPTBase
(lm_benchmark/models/landmark.py:276-392: 12 layers, n_embd 1024, 8 heads of 128, rotary positions, bias-free linears,
tied embedding / output weights, dropout 0) and differs in ONE place: the attention inside each block is this
package's fused operator (`lm_landmark_attention` -> `lmk::masked_attention`) instead of the reference's
score matrix + mask block + grouped softmax + att @ v (landmark.py:196-236).  It exists to measure that operator where
the reference uses it; it is a benchmark harness, not a model library.

Data: PG19 is not available offline; token ids are uniform random with the landmark id 50260 inserted after every
50 tokens of a long stream, and windows are cut at seeded random offsets exactly as get_batch does
(lm_benchmark/optim/utils.py:21-29, including the target shift over landmarks and the -1 targets at landmarks).
"""
import math
import time

import torch
import torch.nn as nn
from torch.nn import functional as F

LANDMARK_ID = 50260
EOT_ID = 50256
CONFIG = dict(vocab_size=50304, n_embd=1024, n_head=8, n_layer=12, sequence_length=512, mem_freq=50, batch_size=16,
              max_groups_for_softmax=16, lr=2e-3, weight_decay=1e-3, beta1=0.9, beta2=0.95)


def synthetic_stream(n_tokens, mem_freq, seed):
    """Uniform random ids (never the landmark or end-of-text id) with a landmark after every mem_freq tokens."""
    g = torch.Generator().manual_seed(seed)
    raw = torch.randint(0, 50256, (n_tokens,), generator=g)
    n_blocks = n_tokens // mem_freq
    blocks = raw[: n_blocks * mem_freq].view(n_blocks, mem_freq)
    lm = torch.full((n_blocks, 1), LANDMARK_ID, dtype=raw.dtype)
    return torch.cat((blocks, lm), dim=1).reshape(-1)


def get_batch(stream, seq_length, batch_size, generator):
    """Same sampling and target construction as lm_benchmark/optim/utils.py:21-26."""
    ix = torch.randint(len(stream) - seq_length - 1, (batch_size,), generator=generator)
    x = torch.stack([stream[i:i + seq_length] for i in ix])
    y = torch.stack([stream[i + 1:i + 1 + seq_length + 1] for i in ix])
    y = torch.where(y[:, :-1] == LANDMARK_ID, y[:, 1:], y[:, :-1])
    y = torch.where((x == LANDMARK_ID) | (x == EOT_ID), -1, y)
    return x, y


def rotary_cos_sin(T, hs, device):
    """lm_benchmark's rotary tables (positional_encoders/rotary.py:24-55): interleaved pairs, freqs 10^(-4 i / hs)."""
    freqs = 10 ** (-4 * torch.arange(0, hs, 2, device=device)[: hs // 2].float() / hs)
    ang = (torch.arange(T, device=device, dtype=torch.float32).unsqueeze(-1) * freqs.view(1, -1))
    ang = ang.unsqueeze(-1).expand(T, hs // 2, 2).reshape(T, hs)
    return ang.cos(), ang.sin()


def apply_rotary(x, cos, sin):
    """t * cos + rotate_half(t) * sin with pairs (2i, 2i+1) (positional_encoders/rotary_utils.py:17-31)."""
    xr = x.view(*x.shape[:-1], -1, 2)
    rot = torch.stack((-xr[..., 1], xr[..., 0]), dim=-1).view(x.shape)
    return x * cos.to(x) + rot * sin.to(x)


class Attention(nn.Module):
    def __init__(self, n_embd, n_head, max_groups, attention_fn, rotary_fn=None):
        super().__init__()
        self.c_attn = nn.Linear(n_embd, 3 * n_embd, bias=False)
        self.c_proj = nn.Linear(n_embd, n_embd, bias=False)
        self.n_head, self.n_embd, self.max_groups, self.attention_fn = n_head, n_embd, max_groups, attention_fn
        self.rotary_fn = rotary_fn

    def forward(self, x, is_mem, cos, sin):
        B, T, C = x.size()
        q, k, v = self.c_attn(x).split(self.n_embd, dim=2)
        q, k, v = [t.view(B, T, self.n_head, C // self.n_head).transpose(1, 2) for t in (q, k, v)]
        if self.rotary_fn is not None and q.is_cuda:
            q, k = self.rotary_fn(q, k, cos.to(q.dtype), sin.to(q.dtype))
        else:
            q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)
        y = self.attention_fn(q, k, v, is_mem, max_groups=self.max_groups)
        return self.c_proj(y.transpose(1, 2).contiguous().view(B, T, C))


class Block(nn.Module):
    def __init__(self, n_embd, n_head, max_groups, attention_fn, rotary_fn=None):
        super().__init__()
        self.ln_1 = nn.LayerNorm(n_embd, bias=False)
        self.attn = Attention(n_embd, n_head, max_groups, attention_fn, rotary_fn)
        self.ln_2 = nn.LayerNorm(n_embd, bias=False)
        self.c_fc = nn.Linear(n_embd, 4 * n_embd, bias=False)
        self.c_proj = nn.Linear(4 * n_embd, n_embd, bias=False)

    def forward(self, x, is_mem, cos, sin):
        x = x + self.attn(self.ln_1(x), is_mem, cos, sin)
        return x + self.c_proj(F.gelu(self.c_fc(self.ln_2(x))))


class LandmarkGPT(nn.Module):
    def __init__(self, cfg, attention_fn, rotary_fn=None):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg["vocab_size"], cfg["n_embd"])
        self.h = nn.ModuleList([Block(cfg["n_embd"], cfg["n_head"], cfg["max_groups_for_softmax"], attention_fn,
                                      rotary_fn) for _ in range(cfg["n_layer"])])
        self.ln_f = nn.LayerNorm(cfg["n_embd"], bias=False)
        self.lm_head = nn.Linear(cfg["n_embd"], cfg["vocab_size"], bias=False)
        self.wte.weight = self.lm_head.weight
        self.apply(self._init)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                torch.nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * cfg["n_layer"]))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            torch.nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def forward(self, idx, targets):
        B, T = idx.shape
        is_mem = idx == LANDMARK_ID
        cos, sin = rotary_cos_sin(T, self.cfg["n_embd"] // self.cfg["n_head"], idx.device)
        x = self.wte(idx)
        for blk in self.h:
            x = blk(x, is_mem, cos, sin)
        logits = self.lm_head(self.ln_f(x))
        return F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1), ignore_index=-1)


def train_step_bench(model, cfg, world, rank, device, steps, warmup, barrier, max_over_ranks):
    """Times `steps` optimizer steps (forward, backward with gradient all-reduce, AdamW) after `warmup` untimed ones.
    Each step's batch comes from pinned host memory inside the timed region and its loss goes back to the host.
    Returns dict(tokens_per_s, ms_per_step, loss_first, loss_last)."""
    stream = synthetic_stream(2_000_000, cfg["mem_freq"], seed=17)
    g = torch.Generator().manual_seed(1000 + rank)
    T, B = cfg["sequence_length"], cfg["batch_size"]
    batches = [tuple(t.pin_memory() for t in get_batch(stream, T, B, g)) for _ in range(warmup + steps)]
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=cfg["lr"], betas=(cfg["beta1"], cfg["beta2"]), weight_decay=cfg["weight_decay"],
                            fused=True)
    losses = []

    def step(i):
        x, y = [t.to(device, non_blocking=True) for t in batches[i]]
        with torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
            loss = model(x, y)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    model.train()
    for i in range(warmup):
        step(i)
    barrier(world)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for i in range(warmup, warmup + steps):
        losses.append(step(i).detach().float().cpu())       # device -> host read of the step's result
    b.record()
    torch.cuda.synchronize()
    barrier(world)
    wall = time.perf_counter() - t0
    ms = max_over_ranks(a.elapsed_time(b) / steps, world, device)
    return dict(tokens_per_s=world * B * T / (ms * 1e-3), ms_per_step=ms, wall_s=wall,
                loss_first=float(losses[0]), loss_last=float(losses[-1]),
                h2d_bytes_per_step=2 * B * T * 8, d2h_bytes_per_step=4)

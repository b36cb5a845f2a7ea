"""Library baseline of the headline benchmark: the same GPT-2 small training step written with stock PyTorch
pieces only, on the same shapes and with the same timing rules as ``bench.py``.

    attention  F.scaled_dot_product_attention (cuDNN / flash backend picked by torch)
    GEMMs      cuBLAS through torch.matmul under bf16 autocast, fp32 master weights
    optimizer  torch.optim.AdamW(fused=True) after clip_grad_norm_
    N > 1      DistributedDataParallel over NCCL (bucketed all-reduce overlapped with backward)

Nothing of this framework's kernels or engine is on that path; it is the "NCCL + library" row of the results
table. Prints one JSON line on rank 0 (tokens/s of the whole job, CUDA events, max over ranks).

    python scripts/bench_gpt2_torch_baseline.py --steps 20 --warmup 5
    torchrun --nproc-per-node 8 scripts/bench_gpt2_torch_baseline.py
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.h = h
        self.ln1, self.ln2 = nn.LayerNorm(d, eps=1e-5), nn.LayerNorm(d, eps=1e-5)
        self.attn, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc, self.out = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)

    def forward(self, x):
        B, T, d = x.shape
        q, k, v = self.attn(self.ln1(x)).view(B, T, 3, self.h, d // self.h).permute(2, 0, 3, 1, 4)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, d)
        x = x + self.proj(y)
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, vocab=50257, ctx=1024, d=768, h=12, layers=12):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(ctx, d)
        self.blocks = nn.ModuleList(Block(d, h) for _ in range(layers))
        self.ln_f = nn.LayerNorm(d, eps=1e-5)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear):
                nn.init.zeros_(m.bias)
        for b in self.blocks:
            nn.init.normal_(b.proj.weight, std=0.02 / math.sqrt(2 * layers))
            nn.init.normal_(b.out.weight, std=0.02 / math.sqrt(2 * layers))

    def forward(self, idx, targets):
        T = idx.shape[1]
        x = self.wte(idx) + self.wpe.weight[:T]
        for b in self.blocks:
            x = b(x)
        logits = self.ln_f(x) @ self.wte.weight.t()
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=1024)
    args = ap.parse_args()
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    model = GPT2().to(dev)
    step_model = nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    decay = [p for n, p in model.named_parameters() if p.dim() >= 2 and "wte" not in n and "wpe" not in n]
    rest = [p for n, p in model.named_parameters() if not (p.dim() >= 2 and "wte" not in n and "wpe" not in n)]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}],
                            lr=6e-4, betas=(0.9, 0.95), eps=1e-8, fused=True)
    B, T = args.micro_batch, args.seq_len
    g = torch.Generator().manual_seed(1234 + rank)
    data = [torch.randint(0, 50257, (B, T + 1), generator=g).to(dev) for _ in range(args.steps + args.warmup)]

    def step(t):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = step_model(t[:, :-1], t[:, 1:])
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for i in range(args.warmup):
        step(data[i])
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(args.steps):
        loss = step(data[args.warmup + i])
    b.record()
    barrier()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    if rank == 0:
        print(json.dumps({"impl": "pytorch SDPA + cuBLAS + fused AdamW" + (" + DDP/NCCL" if world > 1 else ""),
                          "metric": "train tokens/s/box", "value": B * T * world * args.steps / (ms / 1e3),
                          "ms_per_step": ms / args.steps, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "dtype": "bf16 autocast, fp32 master weights", "final_loss": float(loss)}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

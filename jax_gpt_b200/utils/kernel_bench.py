"""Per-kernel micro-benchmarks with CUDA-event timing and roofline fractions.

    python -m jax_gpt_b200.utils.kernel_bench --op gemm --M 8192 --N 8192 --K 8192
    python -m jax_gpt_b200.utils.kernel_bench --op attn_fwd --B 16 --T 1024 --H 12 --D 64
    python -m jax_gpt_b200.utils.kernel_bench --op attn_bwd | norm_fwd | norm_bwd | adamw | ce
    python -m jax_gpt_b200.utils.kernel_bench --op mla_decode --B 32 --T 2304 --H 16
    python -m jax_gpt_b200.utils.kernel_bench --op gdn_prep_fwd | gdn_prep_bwd | gdn_prefill --B 1 --T 4096

Each run does ``--warmup`` untimed launches, then times ``--iters`` launches with CUDA events on
the launching stream (synchronised on both sides) and prints one JSON line with the achieved
rate and its fraction of the measured peak (cuBLAS bf16 burst for FLOP-bound kernels, the copy
bandwidth for byte-bound ones). Working sets are sized above the 126 MB L2 by default where the
op is bandwidth-bound. The same commands are the ones run under ``ncu`` for profiles.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import roofline as R


def _time(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main(argv=None):
    from .. import _ext
    from ..ops import attention as A
    from ..ops import gemm as G
    from ..ops import misc, norm
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", required=True)
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--N", type=int, default=8192)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--H", type=int, default=12)
    ap.add_argument("--D", type=int, default=64)
    ap.add_argument("--Dv", type=int, default=0, help="attention: v head width when it differs from --D")
    ap.add_argument("--Hkv", type=int, default=0, help="attention: kv heads (default: --H)")
    ap.add_argument("--splits", type=int, default=0, help="mla_decode: KV splits per sequence (0 = fill the SMs)")
    ap.add_argument("--graph", action="store_true", help="time CUDA-graph replays (excludes host launch overhead)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    peaks = R.load_peaks()
    flops = bytes_ = 0.0
    if args.op == "gemm":
        M, N, K = args.M, args.N, args.K
        a = torch.randn((K, M) if args.a_mn else (M, K), device=dev).to(torch.bfloat16)
        b = torch.randn((K, N) if args.b_mn else (N, K), device=dev).to(torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fn = lambda: G.gemm(a, b, a_mn_major=args.a_mn, b_mn_major=args.b_mn, out=out)
        flops, bytes_ = 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    elif args.op in ("attn_fwd", "attn_bwd"):
        B, T, H, D = args.B, args.T, args.H, args.D
        Hkv, Dv = args.Hkv or H, args.Dv or D
        if Hkv == H and Dv == D:
            qkv = torch.randn(B, T, 3 * H * D, device=dev).to(torch.bfloat16)
            q, k, v = [qkv[..., i * H * D:(i + 1) * H * D].unflatten(-1, (H, D)) for i in range(3)]
        else:
            q = torch.randn(B, T, H, D, device=dev).to(torch.bfloat16)
            k = torch.randn(B, T, Hkv, D, device=dev).to(torch.bfloat16)
            v = torch.randn(B, T, Hkv, Dv, device=dev).to(torch.bfloat16)
        out, lse = A.attn_fwd(q, k, v)
        base = 2.0 * B * H * T * T * (D + Dv) / 2          # causal: S = Q K^T and O = P V
        if args.op == "attn_fwd":
            fn = lambda: A.attn_fwd(q, k, v, out=out, lse=lse)
            flops = base
        else:
            dout = torch.randn_like(out)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            acc = torch.zeros(B * T, H * D, device=dev)
            delta = torch.empty(B, H, T, device=dev)

            def fn():
                acc.zero_()
                A.attn_bwd(q, k, v, out, dout, lse, dq=dq, dk=dk, dv=dv, dq_accum=acc, delta=delta)
            flops = 2.0 * B * H * T * T * (3 * D + 2 * Dv) / 2  # S, dP, dV, dK, dQ
        bytes_ = 2.0 * B * T * (2 * H * D + 2 * Hkv * D + 2 * Hkv * Dv + 2 * H * Dv)
    elif args.op == "attn_decode":
        B, T, H, D = args.B, args.T, args.H, args.D
        Hkv = args.Hkv or H
        ck = torch.randn(B, Hkv, T, D, device=dev).to(torch.bfloat16)
        cv = torch.randn(B, Hkv, T, D, device=dev).to(torch.bfloat16)
        q = torch.randn(B, H, D, device=dev).to(torch.bfloat16)
        S = args.splits or A.decode_splits(B, Hkv, T)
        scratch = (torch.empty(B, H, S, D, device=dev), torch.empty(B, H, S, 2, device=dev))
        out = torch.empty(B, H * D, device=dev, dtype=torch.bfloat16)
        fn = lambda: A.attention_decode(q, ck, cv, kv_len=T, scratch=scratch, out=out)
        flops = 4.0 * B * H * T * D
        bytes_ = 2.0 * 2 * B * Hkv * T * D
    elif args.op in ("norm_fwd", "norm_bwd"):
        M, D = args.M, args.N if args.N <= 8192 else 768
        x = torch.randn(M, D, device=dev).to(torch.bfloat16)
        g = torch.ones(D, device=dev, dtype=torch.bfloat16)
        bta = torch.zeros(D, device=dev, dtype=torch.bfloat16)
        y, mean, rstd = norm.norm_fwd(norm.LAYERNORM, x, g, bta, 1e-5)
        if args.op == "norm_fwd":
            fn = lambda: norm.norm_fwd(norm.LAYERNORM, x, g, bta, 1e-5, y=y, mean=mean, rstd=rstd)
            bytes_ = 2.0 * 2 * M * D
        else:
            dy = torch.randn_like(x)
            dx = torch.empty_like(x)
            dg = torch.zeros(D, device=dev)
            db = torch.zeros(D, device=dev)
            fn = lambda: norm.norm_bwd(norm.LAYERNORM, dy, x, g, mean, rstd, dg, db, dx=dx)
            bytes_ = 2.0 * 3 * M * D
    elif args.op == "adamw":
        n = args.M * args.N
        p, g, m, v = [torch.randn(n, device=dev) for _ in range(4)]
        v.abs_()
        pb = torch.empty(n, device=dev, dtype=torch.bfloat16)
        hp = torch.tensor([1e-3, 0.1, 0.05, 1.0], device=dev)
        fn = lambda: misc.adamw(p, g, m, v, hp, None, wd=0.1, p_bf16=pb)
        bytes_ = n * (16.0 + 18.0)
    elif args.op == "ce":
        M, V = args.M, args.N
        logits = torch.randn(M, (V + 63) // 64 * 64, device=dev).to(torch.bfloat16)
        tg = torch.randint(0, V, (M,), device=dev, dtype=torch.int32)
        loss = torch.empty(M, device=dev)
        fn = lambda: misc.cross_entropy_fwd_bwd(logits, tg, V, 1.0 / M, loss=loss)
        bytes_ = 2.0 * 2 * M * V
    elif args.op == "gemm_mxfp8":
        from ..ops import fp8 as Q
        M, N, K = args.M, args.N, args.K
        xq, xs = Q.fp8_quant_1x128(torch.randn(M, K, device=dev).to(torch.bfloat16), pow2=True)
        wq, ws = Q.fp8_quant_128x128(torch.randn(N, K, device=dev).to(torch.bfloat16), pow2=True)
        sfa, sfb = Q.pack_scales_ue8m0(xs, M, True), Q.pack_scales_ue8m0(ws, N, False)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fn = lambda: _ext.ops().gemm_mxfp8(xq, sfa, wq, sfb, out)
        flops, bytes_ = 2.0 * M * N * K, 1.0 * (M * K + N * K) + 2.0 * M * N
    elif args.op == "gdn_scan":
        # --B (batch x heads) sequences of --T tokens: the inter-chunk scan of the gated delta rule
        BH, N = args.B, args.T // 64
        bf = torch.bfloat16
        kq = (torch.randn(BH, N, 128, 128, device=dev) * 0.05).to(bf)
        intra = (torch.randn(BH, N, 64, 64, device=dev) * 0.05).to(bf)
        kdec = (torch.randn(BH, N, 64, 128, device=dev) * 0.05).to(bf)
        veff = torch.randn(BH, N, 64, 128, device=dev).to(bf)
        e = torch.full((BH, N), 0.9, device=dev)
        o = torch.empty(BH, N, 64, 128, device=dev, dtype=bf)
        s_out = torch.empty(BH, 128, 128, device=dev)
        fn = lambda: _ext.ops().gdn_scan(kq, intra, kdec, veff, e, None, o, s_out)
        bytes_ = 2.0 * BH * N * (128 * 128 + 64 * 64 + 64 * 128 * 3)
        flops = 2.0 * BH * N * (128 * 128 * 128 + 64 * 64 * 128 + 128 * 64 * 128)
    elif args.op in ("gdn_prep_fwd", "gdn_prep_bwd", "gdn_prefill"):
        # the Gated-DeltaNet prefill between the input and the output projection: --B sequences of --T tokens,
        # --Hkv q/k heads and --H value heads of width 128 (defaults 16 / 32). gdn_prep_*: the chunk-preparation
        # kernel alone; gdn_prefill: preparation + scan + gated norm, forward and backward through autograd
        from ..models.qwen35 import deltanet as DN
        B, T, Hv = args.B, args.T, args.H if args.H != 12 else 32
        Hqk = args.Hkv or Hv // 2
        N = (T + 63) // 64
        bf = torch.bfloat16
        mixed = torch.nn.functional.silu(torch.randn(B, T, (2 * Hqk + Hv) * 128, device=dev)).to(bf)
        bg, ag = torch.randn(B, T, Hv, device=dev).to(bf), torch.randn(B, T, Hv, device=dev).to(bf)
        A_log = torch.log(torch.rand(Hv, device=dev) * 15.9 + 0.1)
        dtb = torch.ones(Hv, device=dev)
        BH = B * Hv
        kq = torch.empty(BH, N, 128, 128, device=dev, dtype=bf)
        intra = torch.empty(BH, N, 64, 64, device=dev, dtype=bf)
        kdec, veff = torch.empty(BH, N, 64, 128, device=dev, dtype=bf), torch.empty(BH, N, 64, 128, device=dev, dtype=bf)
        e = torch.empty(BH, N, device=dev)
        if args.op == "gdn_prep_fwd":
            fn = lambda: _ext.ops().gdn_chunk_prep(mixed, bg, ag, A_log, dtb, kq, intra, kdec, veff, e, Hqk, Hv)
            bytes_ = 2.0 * (mixed.numel() + kq.numel() + intra.numel() + kdec.numel() + veff.numel())
        elif args.op == "gdn_prep_bwd":
            _ext.ops().gdn_chunk_prep(mixed, bg, ag, A_log, dtb, kq, intra, kdec, veff, e, Hqk, Hv)
            dm = torch.empty_like(mixed)
            db, da = torch.empty(B, T, Hv, device=dev), torch.empty(B, T, Hv, device=dev)
            dal, ddt = torch.zeros(Hv, device=dev), torch.zeros(Hv, device=dev)
            fn = lambda: _ext.ops().gdn_chunk_prep_bwd(mixed, bg, ag, A_log, dtb, kq, intra, kdec, veff, e, dm, db, da,
                                                       dal, ddt, Hqk, Hv)
            bytes_ = 2.0 * (2 * mixed.numel() + kq.numel() + intra.numel() + kdec.numel() + veff.numel())
        else:
            leaves = [t.requires_grad_() for t in (mixed, bg, ag, A_log, dtb)]
            z = torch.randn(B, T, Hv * 128, device=dev).to(bf).requires_grad_()
            w = torch.ones(128, device=dev, requires_grad=True)
            dy = torch.randn(B, T, Hv * 128, device=dev).to(bf)

            def fn():
                o, _ = DN.gated_delta_prefill_cuda(*leaves, Hqk, Hv, head_major=True)
                DN._GdnGatedNormFn.apply(o, z, w, Hv, 1e-6).backward(dy)
            flops = 0.0
            bytes_ = 0.0
    elif args.op == "mla_decode":
        # --B sequences of --T cached tokens each, --H heads (16 = DeepSeek-V3 with 8-way head sharding)
        from ..cache.paged import PagedCache
        from ..ops.mla_decode import mla_paged_decode
        B, T, H = args.B, args.T, args.H
        pages = (T + 63) // 64
        cache = PagedCache(1, 576, n_pages=B * pages, page_size=64, max_seqs=B, max_pages_per_seq=pages, device=dev)
        cache.pool.normal_()
        ids = list(range(B))
        cache._tab.reserve(ids, [T] * B)
        cache.commit(ids, T)
        q = (torch.randn(B, H, 576, device=dev) * 0.3).to(torch.bfloat16)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        ns = args.splits or max(1, min(sms // (B * (1 if H <= 16 else (H + 31) // 32)), (T + 127) // 128, 32))
        part_out = torch.empty(2 * B * ns * H * 512, device=dev)
        part_lse = torch.empty(2 * B * ns * H, device=dev)
        out = torch.empty(B, H, 512, device=dev, dtype=torch.bfloat16)
        idt = cache.seq_id_tensor(ids)
        pool0 = cache.pool[0]
        fn = lambda: _ext.ops().mla_paged_decode(q, pool0, cache.block_table, cache.seq_lens, idt, 192 ** -0.5, ns,
                                                 part_out, part_lse, out)
        bytes_ = 2.0 * B * T * 576
        flops = 2.0 * B * H * T * (576 + 512)
    else:
        raise SystemExit(f"unknown op {args.op}")
    if args.graph:
        # launch-bound ops: replay `--iters` launches from one CUDA graph so that host time is excluded
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(args.iters):
                fn()
        inner = args.iters
        ms = _time(graph.replay, args.warmup, 3) / inner
    else:
        ms = _time(fn, args.warmup, args.iters)
    _ext.check_status(dev)
    res = {"op": args.op, "ms": ms, "args": {k: v for k, v in vars(args).items() if k not in ("op",)}}
    if flops:
        res["tflops"] = flops / ms / 1e9
        res["frac_of_measured_bf16_peak"] = res["tflops"] / peaks["bf16_tflops"]
    if bytes_:
        res["gbs"] = bytes_ / ms / 1e6
        res["frac_of_measured_hbm"] = res["gbs"] / peaks["hbm_gbs"]
    res["denominators"] = peaks["source"]
    print(json.dumps(res))


if __name__ == "__main__":
    main()

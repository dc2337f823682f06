#!/usr/bin/env python
"""Single-GPU micro-benchmarks of the hand-written sm_100a kernels against the vendor library.

    python benchmarks/kernels.py gemm        # tcgen05 GEMMs vs cuBLAS on the Llama-3-8B layer shapes
    python benchmarks/kernels.py attention   # tcgen05 flash attention forward vs the library SDPA
    python benchmarks/kernels.py fused       # bandwidth of the fused elementwise / norm / loss / optimizer kernels
    python benchmarks/kernels.py one-gemm [fwd|dx|dw] [M N K]   # a few launches of one GEMM (small case for a profiler)
    python benchmarks/kernels.py one-attention [B S Hq Hkv]     # a few launches of the attention forward and backward
    python benchmarks/kernels.py one-fused                      # a few launches of every fused bandwidth-bound kernel

Timing: CUDA events on the launching stream, 3 warm-up iterations, then `--iters` timed ones.
Variants of one op are interleaved round-robin and the median over rounds is reported, because
on a power-capped part the clock drifts over seconds and back-to-back blocks are not comparable.
Operands of every case are larger than L2 or the case rotates over several operand sets.
"""

import argparse
import json
import os
import statistics
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elf_b200.ops import _ext, fused, gemm as G  # noqa: E402

PEAKS_FILE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")


def measured_peaks():
    """(hbm GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained) with the stated fallbacks."""
    try:
        with open(PEAKS_FILE) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    except Exception:
        return 6650.0, 1590.0, 1400.0, "fallback"


def event_time(fn, iters):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters  # ms


def interleaved(fns: dict, iters=10, rounds=5):
    """Median ms per call of every entry of `fns`, measured round-robin."""
    for fn in fns.values():
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    samples = {k: [] for k in fns}
    for _ in range(rounds):
        for k, fn in fns.items():
            samples[k].append(event_time(fn, iters))
    return {k: statistics.median(v) for k, v in samples.items()}


LAYER_SHAPES = [  # (name, M tokens, N out features, K in features)
    ("wqkv", 4096, 6144, 4096),
    ("wo", 4096, 4096, 4096),
    ("w_gate_up", 4096, 28672, 4096),
    ("w_down", 4096, 4096, 14336),
]


def bench_gemm(args):
    _, burst, sustained, src = measured_peaks()
    dev = torch.device("cuda")
    print(f"# bf16 GEMM TFLOP/s, median of {args.rounds} interleaved rounds x {args.iters} launches; cuBLAS bf16 peak {burst:.0f} burst / {sustained:.0f} sustained ({src})")
    print("| matrix (M x N x K) | mode | ours 1-CTA | ours CTA pair | ours pair, no K-split | cuBLAS | pair / cuBLAS | pair / peak (burst) |")
    print("|---|---|---|---|---|---|---|---|")
    for name, M, N, K in LAYER_SHAPES + [("square", 8192, 8192, 8192)]:
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        g = torch.zeros(N, K, device=dev, dtype=torch.bfloat16)
        flops = 2.0 * M * N * K

        def with_variant(v, split, fn):
            def run():
                G.set_variant(v, split)
                fn()
            return run

        modes = {
            "forward": (lambda: G.linear_forward(x, w), lambda: F.linear(x, w)),
            "input-grad": (lambda: G.linear_input_grad(dy, w), lambda: dy @ w),
            "weight-grad (+=)": (lambda: G.linear_weight_grad(dy, x, out=g), lambda: g.addmm_(dy.t(), x)),
        }
        for mode, (ours, lib) in modes.items():
            t = interleaved(
                {
                    "one": with_variant(0, True, ours),
                    "pair": with_variant(1, True, ours),
                    "pair_nosplit": with_variant(1, False, ours),
                    "lib": lib,
                },
                args.iters,
                args.rounds,
            )
            tf = {k: flops / (v * 1e-3) / 1e12 for k, v in t.items()}
            print(f"| {name} {M}x{N}x{K} | {mode} | {tf['one']:.0f} | {tf['pair']:.0f} | {tf['pair_nosplit']:.0f} | {tf['lib']:.0f} | {tf['pair'] / tf['lib']:.2f} | {tf['pair'] / burst:.2f} |", flush=True)
        del x, w, dy, g
    G.set_variant(1, True)
    G.check_status(dev)


def bench_attention(args):
    from elf_b200.ops import attention_native as A

    dev = torch.device("cuda")
    _, burst, _, src = measured_peaks()
    print(f"# causal GQA attention forward, head_dim 128, bf16; TFLOP/s counts 4*B*H*S^2*D/2; cuBLAS bf16 peak {burst:.0f} ({src})")
    print("| B | S | Hq | Hkv | ours us | ours TFLOP/s | library us | library TFLOP/s | ours / library |")
    print("|---|---|---|---|---|---|---|---|---|")
    for B, S, hq, hkv in [(4, 1024, 32, 8), (2, 2048, 32, 8), (1, 4096, 32, 8), (1, 8192, 32, 8), (1, 4096, 32, 32)]:
        qkv = torch.randn(B, S, hq + 2 * hkv, 128, device=dev).bfloat16()
        q = qkv[:, :, :hq].transpose(1, 2)
        k = qkv[:, :, hq : hq + hkv].transpose(1, 2)
        v = qkv[:, :, hq + hkv :].transpose(1, 2)
        t = interleaved(
            {
                "ours": lambda: A.forward_packed(qkv, hq, hkv),
                "lib": lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=hq != hkv),
            },
            args.iters,
            args.rounds,
        )
        flops = 4.0 * B * hq * S * S * 128 / 2
        print(f"| {B} | {S} | {hq} | {hkv} | {t['ours'] * 1e3:.1f} | {flops / t['ours'] / 1e9:.0f} | {t['lib'] * 1e3:.1f} | {flops / t['lib'] / 1e9:.0f} | {t['lib'] / t['ours']:.2f} |", flush=True)
    G.check_status(dev)


def bench_fused(args):
    hbm, _, _, src = measured_peaks()
    dev = torch.device("cuda")
    T, D, FF, V = 4096, 4096, 14336, 128256
    sets = 8  # rotate over operand sets so that every launch reads from HBM, not L2
    print(f"# fused kernels on Llama-3-8B shapes (T={T} tokens); bytes = algorithmic reads + writes; HBM copy peak {hbm:.0f} GB/s ({src})")
    print("| kernel | bytes per launch | us | GB/s | fraction of peak |")
    print("|---|---|---|---|---|")

    def report(name, nbytes, fn_list):
        i = [0]

        def run():
            fn_list[i[0] % len(fn_list)]()
            i[0] += 1

        t = interleaved({"k": run}, args.iters, args.rounds)["k"]
        gbs = nbytes / (t * 1e-3) / 1e9
        print(f"| {name} | {nbytes / 1e6:.1f} MB | {t * 1e3:.1f} | {gbs:.0f} | {gbs / hbm:.2f} |", flush=True)

    xs = [torch.randn(T, D, device=dev, dtype=torch.bfloat16) for _ in range(sets)]
    wn = torch.ones(D, device=dev, dtype=torch.bfloat16)
    report("rms_norm forward", 2 * T * D * 2, [lambda x=x: fused.rms_norm(x, wn, 1e-5) for x in xs])
    res = [torch.randn(T, D, device=dev, dtype=torch.bfloat16) for _ in range(sets)]
    report("add + rms_norm forward", 4 * T * D * 2, [lambda x=x, r=r: fused.add_rms_norm(x, r, wn, 1e-5) for x, r in zip(xs, res)])
    gu = [torch.randn(T, 2 * FF, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    report("swiglu forward", 3 * T * FF * 2, [lambda t=t: fused.swiglu(t) for t in gu])
    logits = [torch.randn(T, V, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    tgt = torch.randint(0, V, (T,), device=dev)
    report("cross_entropy forward (loss + lse)", T * V * 2, [lambda l=l: fused.cross_entropy(l, tgt) for l in logits])
    n = 256 * 1024 * 1024
    p = torch.randn(n, device=dev, dtype=torch.bfloat16)
    g = torch.randn(n, device=dev, dtype=torch.bfloat16)
    master = p.float()
    m = torch.zeros(n, device=dev, dtype=torch.float32)
    v = torch.zeros(n, device=dev, dtype=torch.float32)
    step = [0]

    def adam():
        step[0] += 1
        _ext.get().adamw(p, g, master, m, v, 1e-4, 0.9, 0.95, 1e-8, 0.1, step[0], 1.0)

    # reads grad (2 B) + master, m, v (12 B); writes param (2 B) + master, m, v (12 B)
    report("fused AdamW (bf16 param/grad, fp32 master + moments)", n * 28, [adam])
    G.check_status(dev)


def one_gemm(args):
    dev = torch.device("cuda")
    mode = args.rest[0] if args.rest else "fwd"
    M, N, K = (int(a) for a in args.rest[1:4]) if len(args.rest) >= 4 else (4096, 6144, 4096)
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    g = torch.zeros(N, K, device=dev, dtype=torch.bfloat16)
    fn = {"fwd": lambda: G.linear_forward(x, w), "dx": lambda: G.linear_input_grad(dy, w), "dw": lambda: G.linear_weight_grad(dy, x, out=g),
          "cublas": lambda: F.linear(x, w)}[mode]
    for _ in range(4):
        fn()
    torch.cuda.synchronize()
    G.check_status(dev)
    print("done", mode, M, N, K)


def one_attention(args):
    from elf_b200.ops import attention_native as A

    B, S, hq, hkv = (int(a) for a in args.rest[:4]) if len(args.rest) >= 4 else (1, 4096, 32, 8)
    qkv = torch.randn(B, S, hq + 2 * hkv, 128, device="cuda").bfloat16()
    g = torch.randn(B, S, hq, 128, device="cuda").bfloat16()
    for _ in range(4):
        out, lse = A.forward_packed(qkv, hq, hkv)
    for _ in range(3):
        A.backward_packed(g, qkv, out, lse, hq, hkv)
    torch.cuda.synchronize()
    G.check_status(torch.device("cuda"))
    print("done attention", B, S, hq, hkv)


def one_fused(args):
    """Three launches of every fused kernel on the Llama-3-8B layer shapes (operands larger than L2 where the op allows)."""
    dev = torch.device("cuda")
    T, D, FF, V = 4096, 4096, 14336, 32064
    x = torch.randn(T, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
    w = torch.ones(D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    gu = torch.randn(T, 2 * FF, device=dev, dtype=torch.bfloat16, requires_grad=True)
    logits = torch.randn(T, V, device=dev, dtype=torch.bfloat16, requires_grad=True)
    tgt = torch.randint(0, V, (T,), device=dev)
    table = torch.randn(V, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (1, T), device=dev)
    qkv = torch.randn(T, 48 * 128, device=dev, dtype=torch.bfloat16)
    cos, sin = fused.rope_tables(T, 128, 500000.0, dev)
    n = 64 * 1024 * 1024
    p = torch.randn(n, device=dev, dtype=torch.bfloat16)
    gr = torch.randn(n, device=dev, dtype=torch.bfloat16)
    master, m, v = p.float(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    for step in range(1, 4):
        h, s2 = fused.add_rms_norm(x, r, w, 1e-5)
        (h.float().sum() + s2.float().sum()).backward()
        fused.rms_norm(x, w, 1e-5).float().sum().backward()
        fused.swiglu(gu).float().sum().backward()
        fused.cross_entropy(logits.clone(), tgt).backward()
        fused.embedding(table, ids, into_grad=True).float().sum().backward()
        fused.rope_(qkv, cos, sin, 40, 128, T)
        ext = _ext.get()
        ext.residual_add(r, x.detach())
        q4 = qkv.view(1, T, 48, 128)
        ext.pack_qkv_grad(q4[:, :, :32], q4[:, :, 32:40], q4[:, :, 40:], cos, sin)
        ext.adamw(p, gr, master, m, v, 1e-4, 0.9, 0.95, 1e-8, 0.1, step, 1.0)
    torch.cuda.synchronize()
    print("done fused")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["gemm", "attention", "fused", "one-gemm", "one-attention", "one-fused"])
    ap.add_argument("rest", nargs="*")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--rounds", type=int, default=5)
    args = ap.parse_args()
    _ext.require_on_gpu()
    {"gemm": bench_gemm, "attention": bench_attention, "fused": bench_fused, "one-gemm": one_gemm, "one-attention": one_attention, "one-fused": one_fused}[args.what](args)


if __name__ == "__main__":
    main()

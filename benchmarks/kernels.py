"""Single-GPU micro-benchmark of the hand-written kernels against the measured rooflines.

    python benchmarks/kernels.py [--case NAME ...] [--iters N] [--small]

Each case is timed with CUDA events on the launching stream after 3 warm-up runs, with a write of
a 256 MB buffer between iterations (L2 flush) and a synchronize on both sides.  The achieved
fraction is algorithmic FLOPs (tensor-core kernels) or algorithmic bytes (the rest) per second
over the measured peaks of ``MEASURED_PEAKS.json`` (fallback 1590 TFLOP/s / 6650 GB/s).
``--small`` shrinks the shapes (used for profiler captures).  One JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from hyper_parallel_b200.ops import attention, fp8, native  # noqa: E402
from hyper_parallel_b200.ops import functional as Fn  # noqa: E402
from hyper_parallel_b200.ops import moe  # noqa: E402
from hyper_parallel_b200.ops.grouped import grouped_linear  # noqa: E402


def peaks():
    try:
        d = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    except (OSError, KeyError):
        return 1590.0, 6650.0, "fallback"


def timed(fn, iters, reps=1):
    """Mean device time of one call.  ``reps`` back-to-back calls share one event pair so that the
    host-side launch cost (tens of microseconds through the Python wrappers) does not dominate the
    short memory-bound kernels; their working sets are larger than L2."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1) / reps
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", nargs="*", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--bwd-group", type=int, default=None,
                    help="attention backward: (batch, head) pairs scheduled together (0 = all, key-tile major)")
    ap.add_argument("--mla-probe", type=int, default=0,
                    help="timing probe of the MLA backward (wrong results): 1 = no dQ reduce, 2 = no exponentials, "
                         "4 / 8 / 16 = without the dQ / dK, dV / score products")
    args = ap.parse_args()
    if args.mla_probe:
        native.lib().hpb_mla_attn_set_probe(args.mla_probe)
    if args.bwd_group is not None:
        native.lib().hpb_flash_attn_set_head_group(args.bwd_group)
        native.lib().hpb_mla_attn_set_head_group(args.bwd_group)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tf, gbs, src = peaks()
    bf = torch.bfloat16
    T = 2048 if args.small else 8192
    TB = 2048 if args.small else 32768          # rows of the memory-bound cases (working set > L2)
    cases = {}

    def gemm_case(M, N, K, pair):
        a, b = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)

        def run():
            Fn.set_gemm_pair_mode("1" if pair else "0")
            Fn.gemm(a, b, out=out)
            Fn.set_gemm_pair_mode("auto")
        return run, 2.0 * M * N * K, None

    cases["gemm_128x256"] = lambda: gemm_case(T, 8192, 4096, False)
    cases["gemm_pair_256x256"] = lambda: gemm_case(T, 8192, 4096, True)

    def fp8_case():
        M, N, K = T, 7168, 2048 if args.small else 7168
        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf) * 0.05
        aq, sa = fp8.quantize_act_1x128(x)
        bq, sb = fp8.quantize_weight_128x128(w)
        return (lambda: fp8.gemm_fp8(aq, sa, bq, sb)), 2.0 * M * N * K, None
    cases["gemm_fp8_blockscale"] = fp8_case

    def quant_case():
        M, K = TB, 7168
        x = torch.randn(M, K, device=dev, dtype=bf)
        return (lambda: fp8.quantize_act_1x128(x)), None, M * K * 3 + M * K // 128 * 4
    cases["quant_act_1x128"] = quant_case

    def attn_case(bwd):
        B, S, H, Hkv = (1, 2048, 16, 4) if args.small else (2, 4096, 32, 8)
        q = torch.randn(B, S, H, 128, device=dev, dtype=bf)
        k, v = torch.randn(B, S, Hkv, 128, device=dev, dtype=bf), torch.randn(B, S, Hkv, 128, device=dev, dtype=bf)
        do = torch.randn_like(q)
        o, lse = attention.flash_attention_forward(q, k, v)
        fl = 4.0 * B * H * S * S * 128 / 2
        if bwd:
            return (lambda: attention.flash_attention_backward(q, k, v, o, lse, do)), 2.5 * fl, None
        return (lambda: attention.flash_attention_forward(q, k, v)), fl, None
    cases["flash_attn_fwd"] = lambda: attn_case(False)
    cases["flash_attn_bwd"] = lambda: attn_case(True)

    def mla_case(bwd, lib=False):
        """192 / 128 latent attention; ``lib``: the expanded form through the cuDNN graph (what the
        model ran before the kernels existed), including its two concatenations."""
        from hyper_parallel_b200.ops import mla_attention as mla
        B, S, H = (1, 2048, 16) if args.small else (2, 4096, 32)
        q = torch.randn(B, S, H, 192, device=dev, dtype=bf)
        kv = torch.randn(B, S, H, 256, device=dev, dtype=bf)
        kr = torch.randn(B, S, 64, device=dev, dtype=bf)
        do = torch.randn(B, S, H, 128, device=dev, dtype=bf)
        fl = 2.0 * B * H * S * S * (192 + 128) / 2
        if lib:
            import torch.nn.functional as F
            from torch.nn.attention import SDPBackend, sdpa_kernel

            def run():
                qa, kva, kra = [t.detach().requires_grad_(bwd) for t in (q, kv, kr)]
                kh = torch.cat([kva[..., :128], kra.view(B, S, 1, 64).expand(B, S, H, 64)], dim=-1)
                with sdpa_kernel([SDPBackend.CUDNN_ATTENTION]):
                    o = F.scaled_dot_product_attention(qa.transpose(1, 2), kh.transpose(1, 2),
                                                       kva[..., 128:].transpose(1, 2), is_causal=True)
                if bwd:
                    o.backward(do.transpose(1, 2))
            return run, (3.5 if bwd else 1.0) * fl, None
        o, lse = mla.mla_forward(q, kv, kr)
        if bwd:
            return (lambda: mla.mla_backward(q, kv, kr, o, lse, do)), 2.5 * fl, None
        return (lambda: mla.mla_forward(q, kv, kr)), fl, None
    cases["mla_attn_fwd"] = lambda: mla_case(False)
    cases["mla_attn_bwd"] = lambda: mla_case(True)
    cases["mla_attn_fwd_cudnn_expanded"] = lambda: mla_case(False, lib=True)
    cases["mla_attn_fwd_bwd_cudnn_expanded"] = lambda: mla_case(True, lib=True)

    def rms_case():
        x, w = torch.randn(TB, 4096, device=dev, dtype=bf), torch.ones(4096, device=dev, dtype=bf)
        r = torch.randn_like(x)
        return (lambda: Fn.add_rmsnorm(x, r, w, 1e-5)), None, TB * 4096 * 2 * 4
    cases["add_rmsnorm_fwd"] = rms_case

    def swiglu_case():
        gu = torch.randn(T, 2 * 14336, device=dev, dtype=bf)
        return (lambda: Fn.swiglu(gu)), None, T * 14336 * 2 * 3
    cases["swiglu_fwd"] = swiglu_case

    def rope_case():
        x = torch.randn(TB, 40, 128, device=dev, dtype=bf)
        return (lambda: Fn.rope_(x, min(TB, 4096), 5e5)), None, TB * 40 * 128 * 2 * 2
    cases["rope_inplace"] = rope_case

    def ce_case():
        V = 32064 if args.small else 128256
        logits = torch.randn(T, V, device=dev, dtype=bf)
        tgt = torch.randint(0, V, (T,), device=dev)
        return (lambda: Fn.cross_entropy_fwd_bwd(logits, tgt, 1.0 / T)), None, T * V * 2 * 2
    cases["cross_entropy_fwd_bwd"] = ce_case

    def adamw_case():
        n = (32 if args.small else 218) * 1000 * 1000
        p = torch.zeros(n, device=dev, dtype=bf)
        m, a, b = (torch.zeros(n, device=dev) for _ in range(3))
        g = torch.randn(n, device=dev, dtype=bf)
        return (lambda: Fn.adamw_step_(p, m, a, b, g, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                       step=1)), None, n * (2 + 24 + 2)
    cases["adamw_fp32_master"] = adamw_case

    def router_case():
        Tt, E = (T, 256)
        logits = torch.randn(Tt, E, device=dev)
        bias = torch.zeros(E, device=dev)
        return (lambda: moe._RouteKernel.apply(logits, bias, 8, 8, 4, 2.5)), None, Tt * E * 4 + Tt * 8 * 12
    cases["moe_router_topk"] = router_case

    def grouped_case():
        E, Hh, Fh = 32, 7168, 2048
        per = 256 if args.small else 1024
        counts = [per] * E
        x = torch.randn(per * E, Hh, device=dev, dtype=bf)
        w = torch.randn(E, 2 * Fh, Hh, device=dev, dtype=bf) * 0.02
        return (lambda: grouped_linear(x, w, counts)), 2.0 * per * E * 2 * Fh * Hh, None
    cases["grouped_gemm_32_experts"] = grouped_case

    for name in (args.case or list(cases)):
        fn, flops, nbytes = cases[name]()
        ms = timed(fn, args.iters, reps=1 if (flops is not None or args.small) else 4)
        native.check_status()
        rec = {"case": name, "ms": round(ms, 4), "peaks": src, "small": args.small}
        if flops is not None:
            rec["tflops"] = round(flops / ms / 1e9, 1)
            peak = tf * (2.0 if "fp8" in name else 1.0)
            rec["fraction_of_peak"] = round(flops / ms / 1e9 / peak, 3)
            rec["peak_tflops_used"] = peak
        else:
            rec["gbs"] = round(nbytes / ms / 1e6, 1)
            rec["fraction_of_hbm"] = round(nbytes / ms / 1e6 / gbs, 3)
        print(json.dumps(rec))


if __name__ == "__main__":
    main()

"""Per-kernel timing of the fused compute+collective paths against their rooflines.

Run with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 benchmarks/fused_paths.py

Every number is device time (CUDA events on the launching stream, barrier + synchronize on both
sides, L2 flushed between iterations), max over ranks.  For each path the unfused sequence
(NCCL collective + the same tcgen05 GEMM) is timed the same way.  Roofline of a fused path = the
slower of FLOPs / measured GEMM peak and NVLink bytes / measured link bandwidth per direction.
Rank 0 prints one JSON line per path.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from hyper_parallel_b200.collectives import cc  # noqa: E402
from hyper_parallel_b200.ops import functional as Fn  # noqa: E402
from hyper_parallel_b200.ops import native  # noqa: E402
from hyper_parallel_b200.parallel.tp_fused import TPWorkspace  # noqa: E402

LINK_GBS = 770.0          # measured peer copy, per direction per GPU


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops", 1590.0)), float(d.get("hbm_gbs", 6650.0)), "measured"
    except OSError:
        return 1590.0, 6650.0, "fallback"


def timed(fn, iters=10, warmup=3):
    dev = torch.device("cuda", torch.cuda.current_device())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(warmup):
        fn()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    t = torch.tensor([total / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    group = dist.group.WORLD
    peak_tf, hbm_gbs, src = _peaks()
    n = world
    out = []

    # ---- tensor parallel: all-gather -> GEMM and GEMM -> reduce-scatter (Llama-2-13B, TP = n) ----
    T, H, F = 8192, 5120, 13824
    for name, (k_dim, n_dim) in {"qkv": (H, 3 * H // n), "gate_up": (H, 2 * F // n)}.items():
        Ms = T // n
        x = torch.randn(Ms, k_dim, device=dev, dtype=torch.bfloat16)
        w = torch.randn(n_dim, k_dim, device=dev, dtype=torch.bfloat16) * 0.02
        ws = TPWorkspace.get(group, Ms * k_dim * 2, T * max(H, 1) * 2)
        full = torch.empty(T, k_dim, device=dev, dtype=torch.bfloat16)
        y = torch.empty(T, n_dim, device=dev, dtype=torch.bfloat16)

        def unfused():
            dist.all_gather_into_tensor(full, x)
            Fn.gemm(full, w, out=y)

        t_f = timed(lambda: ws.ag_gemm(x, w, out=y))
        t_u = timed(unfused)
        flops = 2.0 * T * n_dim * k_dim
        roof = max(flops / (peak_tf * 1e12), (n - 1) * Ms * k_dim * 2 / (LINK_GBS * 1e9)) * 1e3
        out.append({"path": f"ag_gemm[{name}]", "n_gpus": n, "M": T, "N": n_dim, "K": k_dim, "fused_ms": t_f,
                    "nccl_plus_gemm_ms": t_u, "roofline_ms": roof, "fraction_of_roofline": roof / t_f,
                    "peaks": src})
    for name, (k_dim, n_dim) in {"out_proj": (H // n, H), "down": (F // n, H)}.items():
        a = torch.randn(T, k_dim, device=dev, dtype=torch.bfloat16)
        w = torch.randn(n_dim, k_dim, device=dev, dtype=torch.bfloat16) * 0.02
        ws = TPWorkspace.get(group, (T // n) * H * 2, T * n_dim * 2)
        part = torch.empty(T, n_dim, device=dev, dtype=torch.bfloat16)
        red = torch.empty(T // n, n_dim, device=dev, dtype=torch.bfloat16)

        def unfused():
            Fn.gemm(a, w, out=part)
            dist.reduce_scatter_tensor(red, part)

        t_f = timed(lambda: ws.gemm_rs(a, w))
        t_u = timed(unfused)
        flops = 2.0 * T * n_dim * k_dim
        roof = max(flops / (peak_tf * 1e12), (n - 1) * (T // n) * n_dim * 2 / (LINK_GBS * 1e9)) * 1e3
        out.append({"path": f"gemm_rs[{name}]", "n_gpus": n, "M": T, "N": n_dim, "K": k_dim, "fused_ms": t_f,
                    "nccl_plus_gemm_ms": t_u, "roofline_ms": roof, "fraction_of_roofline": roof / t_f,
                    "peaks": src})
    native.check_status(dev)

    # ---- HSDP: weight all-gather fused into the consumer GEMM, P2P all-gather, fused reduce-scatter + AdamW
    # (one Llama-3-8B layer: 218 M params) ----
    import ctypes
    from hyper_parallel_b200.parallel import fused_hsdp as fh
    from hyper_parallel_b200.parallel.symm import DEFAULT_WAIT_NS, SLOT_SHARD_VERSION, SymmetricMemory
    lib = fh._bind(native.lib())
    stream = native.stream(dev)
    status = native.status_word(dev)
    T = 8192
    for name, (rows, cols, w_mn) in {"gate_up fwd": (28672, 4096, False), "qkv fwd": (6144, 4096, False),
                                      "down fwd": (4096, 14336, False), "gate_up dgrad": (28672, 4096, True),
                                      "down dgrad": (4096, 14336, True)}.items():
        shard_rows = rows // n
        sm = SymmetricMemory(group, shard_rows * cols * 2, dev)
        w_shard = sm.tensor(torch.bfloat16, shard_rows * cols, 0).view(shard_rows, cols)
        w_shard.normal_(0, 0.02)
        staging = torch.empty(rows, cols, device=dev, dtype=torch.bfloat16)
        cnt = torch.zeros((rows + 127) // 128 + 2, dtype=torch.int32, device=dev)
        K, N = (rows, cols) if w_mn else (cols, rows)
        a = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        y = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
        seq = [0]
        torch.cuda.synchronize()
        dist.barrier()

        def fused():
            seq[0] += 1
            native.check(lib.hpb_gemm2_agw(a.data_ptr(), a.stride(0), sm.ptrs, staging.data_ptr(), int(w_mn), rows,
                                           cols, y.data_ptr(), y.stride(0), T, n, rank, cnt.data_ptr(), seq[0], sm.pad_ptrs[rank],
                                           SLOT_SHARD_VERSION, 0, DEFAULT_WAIT_NS, status.data_ptr(),
                                           native.sm_count(dev), stream), "hpb_gemm2_agw")

        def unfused():
            dist.all_gather_into_tensor(staging.view(-1), w_shard.view(-1))
            Fn.gemm(a, staging, b_mn=w_mn, out=y)

        t_f = timed(fused)
        t_u = timed(unfused)
        t_g = timed(lambda: Fn.gemm(a, staging, b_mn=w_mn, out=y))
        flops = 2.0 * T * N * K
        roof = max(flops / (peak_tf * 1e12), (n - 1) * shard_rows * cols * 2 / (LINK_GBS * 1e9)) * 1e3
        out.append({"path": f"hsdp_allgather_gemm[{name}]", "n_gpus": n, "M": T, "N": N, "K": K, "fused_ms": t_f,
                    "nccl_plus_gemm_ms": t_u, "gemm_alone_ms": t_g, "roofline_ms": roof,
                    "fraction_of_roofline": roof / t_f, "peaks": src})
        native.check_status(dev)
        del staging, a, y
        sm.close()

    numel = 218_112_000 // (8 * n) * (8 * n)
    shard = numel // n
    symm = SymmetricMemory(group, shard * 2 + 256 + numel * 2, dev, multicast=True)
    goff = (shard * 2 + 255) // 256 * 256
    full = torch.empty(numel, dtype=torch.bfloat16, device=dev)
    segs = torch.tensor([[0, 0, shard, 0]], dtype=torch.int64, device=dev)
    sptr, gptr = symm.ptr_table(0), symm.ptr_table(goff)
    symm.tensor(torch.bfloat16, numel, goff).normal_()
    master = torch.zeros(shard, dtype=torch.float32, device=dev)
    m1, m2 = torch.zeros_like(master), torch.zeros_like(master)
    hyper = (ctypes.c_float * 5)(1e-4, 0.9, 0.95, 1e-8, 0.1)
    ver = [0]

    def ag():
        native.check(lib.hpb_p2p_allgather(sptr, symm.pad_ptrs, segs.data_ptr(), 1, full.data_ptr(), rank, n,
                                           symm.next_epoch(), DEFAULT_WAIT_NS, status.data_ptr(),
                                           symm.done_counter.data_ptr(), fh._NUM_COMM_CTAS, stream), "ag")

    def rs(mc):
        ver[0] += 1
        native.check(lib.hpb_fused_rs_adamw(gptr, mc, symm.pad_ptrs, segs.data_ptr(), 1, master.data_ptr(),
                                            m1.data_ptr(), m2.data_ptr(),
                                            symm.tensor(torch.bfloat16, shard, 0).data_ptr(), hyper, 1, 1, 1.0, rank,
                                            n, symm.next_epoch(), ver[0], DEFAULT_WAIT_NS, status.data_ptr(),
                                            symm.done_counter.data_ptr() + 8, fh._NUM_RS_CTAS, stream), "rs")

    shard_t = torch.empty(shard, dtype=torch.bfloat16, device=dev)
    grad_full = torch.randn(numel, dtype=torch.bfloat16, device=dev)
    grad_shard = torch.empty(shard, dtype=torch.bfloat16, device=dev)

    def ag_nccl():
        dist.all_gather_into_tensor(full, shard_t)

    def rs_nccl():
        dist.reduce_scatter_tensor(grad_shard, grad_full)
        g32 = grad_shard.float()
        torch._fused_adamw_([master], [g32], [m1], [m2], [], [torch.tensor(1.0, device=dev)], lr=1e-4, beta1=0.9,
                            beta2=0.95, weight_decay=0.1, eps=1e-8, amsgrad=False, maximize=False)
        shard_t.copy_(master)

    t = timed(ag)
    roof = max((n - 1) * shard * 2 / (LINK_GBS * 1e9), numel * 2 / (hbm_gbs * 1e9)) * 1e3
    out.append({"path": "hsdp_p2p_allgather", "n_gpus": n, "params": numel, "fused_ms": t, "nccl_ms": timed(ag_nccl),
                "roofline_ms": roof, "fraction_of_roofline": roof / t, "peaks": src})
    # bytes: (n-1) peer shards of bf16 gradients over NVLink (egress; with the in-switch reduction the
    # ingress is one shard); local: own gradient shard 2 B, master/m/v read + write 24 B, bf16
    # parameter write 2 B per owned element
    roof = max((n - 1) * shard * 2 / (LINK_GBS * 1e9), shard * 28 / (hbm_gbs * 1e9)) * 1e3
    t_nccl = timed(rs_nccl)
    t = timed(lambda: rs(None))
    out.append({"path": "hsdp_fused_rs_adamw[peer loads]", "n_gpus": n, "params": numel, "fused_ms": t,
                "nccl_rs_plus_adamw_ms": t_nccl, "roofline_ms": roof, "fraction_of_roofline": roof / t,
                "peaks": src})
    if symm.mc_base is not None:
        t = timed(lambda: rs(symm.mc_base + goff))
        out.append({"path": "hsdp_fused_rs_adamw[multimem.ld_reduce]", "n_gpus": n, "params": numel, "fused_ms": t,
                    "nccl_rs_plus_adamw_ms": t_nccl, "roofline_ms": roof, "fraction_of_roofline": roof / t,
                    "peaks": src})
    else:
        out.append({"path": "hsdp_fused_rs_adamw[multimem.ld_reduce]", "n_gpus": n,
                    "unavailable": f"no multicast mapping (transport {symm.transport})"})
    # ---- (4) expert-parallel dispatch / combine: DeepSeek-V3 shapes, uniform random routing ------------------
    from hyper_parallel_b200.parallel.ep_fused import EPWorkspace
    T, k, H = 4096, 8, 7168
    E = min(256, 64 * n)                      # the kernels hold at most 64 local experts per rank
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, generator=g)
    topk_idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(64)]).repeat(T // 64, 1)
    topk_idx = topk_idx[torch.randperm(T, device=dev, generator=g)].contiguous()
    flat_e = topk_idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    sorted_token = (order // k).to(torch.int32)
    counts = torch.bincount(flat_e, minlength=E).to(torch.int32)
    sorted_pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    sorted_pos[order] = torch.arange(T * k, dtype=torch.int32, device=dev)
    w = torch.rand(T, k, device=dev)
    ws = EPWorkspace.get(dist.group.WORLD, T, k, H, E, 2.0)
    ws.dispatch(x, sorted_token, counts)
    ws.out.normal_()
    rows_remote = T * k * (n - 1) / n
    roof = max(rows_remote * H * 2 / (LINK_GBS * 1e9), (T * k * H * 2 * 2) / (hbm_gbs * 1e9)) * 1e3
    send = torch.empty(T * k, H, device=dev, dtype=torch.bfloat16)
    recv_nccl = torch.empty_like(send)

    def a2a():
        dist.all_to_all_single(recv_nccl, send)

    t_a2a = timed(a2a)
    t = timed(lambda: ws.dispatch(x, sorted_token, counts))
    out.append({"path": "ep_dispatch", "n_gpus": n, "tokens": T, "top_k": k, "hidden": H, "experts": E, "fused_ms": t,
                "nccl_all_to_all_ms": t_a2a, "roofline_ms": roof, "fraction_of_roofline": roof / t, "peaks": src,
                "note": "fused = stage + peer pull into the padded expert layout + grouped-GEMM tables; NCCL = one "
                        "all_to_all_single of the same rows (equal splits, no permutation, no tables)"})
    t = timed(lambda: ws.combine(topk_idx, sorted_pos, w, save_rows=False))
    out.append({"path": "ep_combine", "n_gpus": n, "tokens": T, "top_k": k, "hidden": H, "experts": E, "fused_ms": t,
                "nccl_all_to_all_ms": t_a2a, "roofline_ms": roof, "fraction_of_roofline": roof / t, "peaks": src,
                "note": "fused = peer pull of the k expert rows of every token + weighted sum"})
    native.check_status(dev)
    if rank == 0:
        for o in out:
            print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in o.items()}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

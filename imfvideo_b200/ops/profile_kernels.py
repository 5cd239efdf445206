"""Launch one kernel of the library a few times on a chosen shape, for use
under ``ncu`` (or for a quick CUDA-event timing without it).

    python -m imfvideo_b200.ops.profile_kernels attn_fwd  --L 9472
    python -m imfvideo_b200.ops.profile_kernels attn_jvp  --L 9472
    python -m imfvideo_b200.ops.profile_kernels attn_bwd  --L 4736
    python -m imfvideo_b200.ops.profile_kernels attn_jvp  --L 32780 --H 12 --hd 128
    python -m imfvideo_b200.ops.profile_kernels gemm      --M 58280 --N 528 --K 256
    python -m imfvideo_b200.ops.profile_kernels gemm_fp8  --M 65560 --N 4096 --K 1024   # e4m3 operands
    python -m imfvideo_b200.ops.profile_kernels sparse    --L 9472
    python -m imfvideo_b200.ops.profile_kernels resnorm   --rows 29140
    python -m imfvideo_b200.ops.profile_kernels resnorm_bwd --rows 29140 --D 256
    python -m imfvideo_b200.ops.profile_kernels lin       --L 29140      # linear-branch kernels, one line each
    python -m imfvideo_b200.ops.profile_kernels route     --L 29140      # block means, top-k, INT8 quantiser
    python -m imfvideo_b200.ops.profile_kernels ns --B 24 --M 1024 --K 1024  # Newton-Schulz, 5 iterations
    IMF_NS_SYM=0 python -m imfvideo_b200.ops.profile_kernels ns --B 24 --M 1024 --K 1024   # full products
    python -m imfvideo_b200.ops.profile_kernels qkprep_bwd --rows 29140 --H 4   # q/k preparation backward

Prints the CUDA-event time per launch (after warm-up, inputs larger than L2
or L2 flushed between launches) and the achieved fraction of the measured
peaks in MEASURED_PEAKS.json when that file is present.
"""

from __future__ import annotations

import argparse
import json
import os

import torch


def _time(fn, iters: int, flush) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["attn_fwd", "attn_jvp", "attn_bwd", "gemm", "gemm_fp8", "sparse",
                                       "sparse_jvp", "resnorm", "resnorm_bwd", "lin", "route", "ns",
                                       "qkprep_bwd"])
    ap.add_argument("--L", type=int, default=9472)
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--H", type=int, default=4)
    ap.add_argument("--hd", type=int, default=64, help="head dimension of the attention kernels")
    ap.add_argument("--M", type=int, default=58280)
    ap.add_argument("--N", type=int, default=528)
    ap.add_argument("--K", type=int, default=256)
    ap.add_argument("--rows", type=int, default=29140)
    ap.add_argument("--D", type=int, default=256)
    ap.add_argument("--snaps", type=int, default=3)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    from . import cuda as cu

    assert cu.available()
    from . import kernels as K

    dev = torch.device("cuda")
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: flush_buf.fill_(0)
    B, L, H = args.B, args.L, args.H
    mk = lambda: torch.randn(B, L, H, 64, device=dev).bfloat16()
    flops = bytes_ = None
    if args.kernel in ("attn_fwd", "attn_jvp", "attn_bwd"):
        mkd = lambda: torch.randn(B, L, H, args.hd, device=dev).bfloat16()
        q, k, v, dq, dk, dv = (mkd() for _ in range(6))
        base = 4.0 * B * H * L * L * args.hd
        if args.kernel == "attn_fwd":
            fn, flops = (lambda: K.attn_fwd(q, k, v)), base
        elif args.kernel == "attn_jvp":
            fn, flops = (lambda: K.attn_fwd(q, k, v, dq, dk, dv)), 3 * base
        else:
            o, _, lse = K.attn_fwd(q, k, v)
            fn, flops = (lambda: K.attn_bwd(q, k, v, o, lse, dq)), 2.5 * base
    elif args.kernel == "gemm":
        a = torch.randn(args.M, args.K, device=dev).bfloat16()
        b = torch.randn(args.N, args.K, device=dev).bfloat16()
        fn, flops = (lambda: K.gemm(a, b)), 2.0 * args.M * args.N * args.K
        bytes_ = 2.0 * (args.M * args.K + args.N * args.K + args.M * args.N)
    elif args.kernel == "gemm_fp8":
        a = torch.randn(args.M, args.K, device=dev).bfloat16()
        b = torch.randn(args.N, args.K, device=dev).bfloat16()
        a8, sa = K.quantize_fp8(a)
        b8, sb = K.quantize_fp8(b)
        fn, flops = (lambda: K.gemm_fp8(a8, sa, b8, sb)), 2.0 * args.M * args.N * args.K
        bytes_ = 1.0 * (args.M * args.K + args.N * args.K) + 2.0 * args.M * args.N
    elif args.kernel == "qkprep_bwd":
        # backward of the q / k preparation (per-head RMSNorm + partial RoPE + shared rope key):
        # --rows tokens, --H heads, --hd 64 | 128 (half of each head takes the rope)
        from . import rowops as R

        rows, hd = args.rows, args.hd
        dn = dr = hd // 2
        dv = hd
        rn = lambda *sh: torch.randn(*sh, device=dev).bfloat16()
        qb, kvb = rn(rows, H * hd), rn(rows, H * (dn + dv))
        ang = torch.rand(rows, dr // 2, device=dev) * 6
        cos, sin = torch.cos(ang), torch.sin(ang)
        qg, kg = torch.rand(dn, device=dev) + 0.5, torch.rand(dn, device=dev) + 0.5
        gq, gk = rn(rows, H * hd), rn(rows, H * hd)
        g_qb, g_kvb = torch.empty_like(qb), torch.zeros_like(kvb)
        na = 256 + dr
        g_a = torch.zeros(rows, na, device=dev, dtype=torch.bfloat16)
        fn = lambda: R.qkprep_bwd(qb, kvb, cos, sin, qg, kg, gq, gk, g_qb, g_kvb, g_a[:, 256:], rows,
                                  rows, H, dn, dr, dv, na, 1e-5, raw=True)
        # reads gq, gk, q_b, the k half of kv_b; writes g_qb, the k half of g_kvb, g_k_rope
        bytes_ = 2.0 * rows * (2 * H * hd + H * hd + H * dn + H * hd + H * dn + dr)
    elif args.kernel == "ns":
        # Newton-Schulz on a batch of B matrices of M x K (5 iterations, 3 launches each)
        G = torch.randn(B, args.M, args.K, device=dev)
        co = (3.4445, -4.7750, 2.0315)
        fn = lambda: K.newton_schulz(G, co, steps=5)
        g_, o_ = min(args.M, args.K), max(args.M, args.K)
        flops = 5 * B * (2.0 * g_ * g_ * o_ + 2.0 * g_ ** 3 + 2.0 * g_ * g_ * o_)
    elif args.kernel in ("sparse", "sparse_jvp"):
        from . import sparse as SP

        q, k, v, dq, dk, dv = (mk() for _ in range(6))
        Mb, Nb = -(-L // 64), -(-L // 64)
        T = max(1, Nb // 10)
        sel = torch.stack([torch.stack([torch.randperm(Nb, device=dev)[:T] for _ in range(Mb)])
                           for _ in range(H)]).unsqueeze(0).expand(B, -1, -1, -1).contiguous()
        lut, flags = SP.build_tile_lut(sel, 64)
        tang = args.kernel == "sparse_jvp"
        fn = lambda: SP.sparse_fwd(q, k, v, dq if tang else None, dk if tang else None,
                                   dv if tang else None, lut, flags, 64, True, True)
    elif args.kernel in ("lin", "route"):
        from . import linattn as LA
        from . import sparse as SP

        q, k, v, o_s, go = (mk() for _ in range(5))
        Mb = Nb = -(-L // 64)
        T = max(1, Nb // 10)
        qh, kh = q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3)
        if args.kernel == "route":
            qb, kb = SP.pool_blocks(qh, 64), SP.pool_blocks(kh, 64)
            eye = torch.eye(64, device=dev)
            for name, f in (("pool_blocks", lambda: SP.pool_blocks(qh, 64)),
                            ("route_topk", lambda: SP.route_topk(qb, kb, T, eye, eye)),
                            ("quantize_blocks", lambda: SP.quantize_blocks(q, 64, want_fq=True))):
                print(json.dumps({"kernel": name, "ms": _time(f, args.iters, flush)}))
            K.check_status()
            return
        sel = SP.route_topk(SP.pool_blocks(qh, 64), SP.pool_blocks(kh, 64), T)
        a_rows = torch.full((H, L), 0.9, device=dev)
        S2, _ = LA.states(k, None, v, None, None, 64, L)
        cm2 = LA.comp_mask(sel, Mb, Nb)
        o, _, C = LA.forward(q, k, v, None, None, None, o_s, None, sel, a_rows, 64, 64, None)
        gq, gnum, gden, ga, g_os = LA.backward_rows(q, o_s, go, C, a_rows, 64)
        steps = (
            ("lin_states", lambda: LA.states(k, None, v, None, None, 64, L)),
            ("comp_mask (torch)", lambda: LA.comp_mask(sel, Mb, Nb)),
            ("mask gemm", lambda: K.gemm_batched(cm2, S2, b_mn=True, out_dtype=torch.float32)),
            ("forward (states + mask + gemm + apply)",
             lambda: LA.forward(q, k, v, None, None, None, o_s, None, sel, a_rows, 64, 64, None)),
            ("lin_bwd_rows", lambda: LA.backward_rows(q, o_s, go, C, a_rows, 64)),
            ("backward_kv (states + mask + gemm + kv)",
             lambda: LA.backward_kv(q, k, v, gnum, gden, sel, g_os, g_os, 64, 64, None)),
        )
        for name, f in steps:
            print(json.dumps({"kernel": name, "ms": _time(f, args.iters, flush)}))
        K.check_status()
        return
    elif args.kernel == "resnorm_bwd":
        from . import rowops as R

        rows, D, ns = args.rows, args.D, args.snaps
        res = torch.randn(rows, D, device=dev)
        y = torch.randn(rows, D, device=dev).bfloat16()
        gn = torch.randn(rows, D, device=dev).bfloat16()
        gext = torch.randn(rows, D, device=dev)
        snaps = [torch.randn(rows, D, device=dev) for _ in range(ns)]
        gate, w, gain = (torch.randn(D, device=dev) for _ in range(3))
        fn = lambda: R.resnorm_bwd(res, y, gate, snaps, w, gain, 1e-5, gn, gext)
        # reads: res, y, gn, g_pfx_ext, snaps; writes: g_res, g_y, g_snaps
        bytes_ = rows * D * (4 + 2 + 2 + 4 + 4 * ns + 4 + 2 + 4 * ns)
    else:
        from . import rowops as R

        rows, D, ns = args.rows, args.D, args.snaps
        res = torch.randn(rows, D, device=dev)
        y = torch.randn(rows, D, device=dev).bfloat16()
        snaps = [torch.randn(rows, D, device=dev) for _ in range(ns)]
        gate, w, gain = (torch.randn(D, device=dev) for _ in range(3))
        n, pf = torch.empty(rows, D, dtype=torch.bfloat16, device=dev), torch.empty(rows, D, device=dev)
        fn = lambda: R.resnorm_fwd(res, None, y, None, gate, snaps, [None] * ns, w, gain, 1e-5, n,
                                   None, pf, None)
        bytes_ = rows * D * (4 * (2 + ns) + 2 + 2)
    ms = _time(fn, args.iters, flush)
    K.check_status()
    line = {"kernel": args.kernel, "ms": ms}
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                         "MEASURED_PEAKS.json")
    pk = json.load(open(peaks)) if os.path.exists(peaks) else {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}
    if flops:
        line["tflops"] = flops / ms / 1e9
        line["frac_of_measured_bf16"] = line["tflops"] / pk["bf16_tflops"]
    if bytes_:
        line["gbs"] = bytes_ / ms / 1e6
        line["frac_of_measured_hbm"] = line["gbs"] / pk["hbm_gbs"]
    print(json.dumps(line))


if __name__ == "__main__":
    main()

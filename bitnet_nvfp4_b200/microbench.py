"""Single-kernel micro-benchmarks of libbnf4 (CUDA-event timing; also the small cases used for ncu captures).

    python -m bitnet_nvfp4_b200.microbench gemm  [--m 65536] [--variants plain,lora,direct,gelu,gelufp4,aid<N>] [--iters 5]
    python -m bitnet_nvfp4_b200.microbench efla  [--seqs 2048] [--iters 3] [--mma 0|1]
    python -m bitnet_nvfp4_b200.microbench rowquant [--rows 65536] [--iters 5]
    python -m bitnet_nvfp4_b200.microbench sweep            # perturbed-GEMM sweep M x (K = N) with FP4 utilisation

Inputs are seeded random tensors of the shapes the default model uses (K = 512, heads of 64).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np
import torch

from . import host as H
from . import lib

ROOT = Path(__file__).resolve().parent.parent


def _time(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1400.0, "fallback"


def _operands(m, n, k, rank, R, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.clamp(torch.round(torch.randn(m, k, device="cuda", generator=g) * 40), -127, 127).to(torch.int8)
    w = torch.randint(-1, 2, (n, k), device="cuda", generator=g, dtype=torch.int8)
    a, sfa = H.nvfp4_quantize_a(x)
    b, sfb = H.nvfp4_quantize_b(w)
    pairs = max(1, m // R // 2)
    A = torch.randint(-4, 5, (pairs, n, max(rank, 1)), device="cuda", generator=g, dtype=torch.int8)
    t = torch.randint(-1000, 1000, (m, max(rank, 1)), device="cuda", generator=g, dtype=torch.int32)
    return a, sfa, b, sfb, A, t, pairs


def bench_gemm(m, variants, iters, n_arg=0, k_arg=0):
    k, R = (k_arg or 512), 4096
    for v in variants:
        n = n_arg or (1024 if v.startswith("gelu") else 512)
        a, sfa, b, sfb, A, t, pairs = _operands(m, n, k, 1, R)
        alpha = float(1 / np.sqrt(k))
        ldd = (n + 31) & ~31
        d = torch.empty((m, ldd), dtype=torch.float32, device="cuda")
        d8 = torch.empty((m, n), dtype=torch.int8, device="cuda")
        codes = torch.zeros(m * n // 2, dtype=torch.uint8, device="cuda")
        sf = torch.zeros(H.sf_bytes(m, n), dtype=torch.uint8, device="cuda")
        nt = torch.zeros((m, 1), dtype=torch.int32, device="cuda")
        tv = torch.randint(-4, 5, (pairs, 1, n), device="cuda", dtype=torch.int8)
        lora = dict(rank=1, rows_per_member=R, lora_t=t, t_stride=1, lora_A=A, lora_A_pair_stride=n, lora_scale=0.01)
        base = dict(a=a, b=b, sfa=sfa, sfb=sfb, m=m, n=n, k=k, alpha=alpha)

        def run():
            if v == "plain":
                H.gemm_nvfp4_ex(**base, d=d, ldd=ldd, epilogue=H.EPI_F32)
            elif v == "direct":
                lib.load().bnf4_set_option(b"gemm_tma_store", 0)
                H.gemm_nvfp4_ex(**base, d=d, ldd=n, epilogue=H.EPI_F32)
                lib.load().bnf4_set_option(b"gemm_tma_store", 1)
            elif v.startswith("aid"):  # aid<store mode + 4 * timing-aid bits>, e.g. aid15 = no A/B loads, no store
                lib.load().bnf4_set_option(b"gemm_tma_store", int(v[3:]))
                H.gemm_nvfp4_ex(**base, d=d, ldd=n, epilogue=H.EPI_F32)
                lib.load().bnf4_set_option(b"gemm_tma_store", 1)
            elif v == "lora":
                H.gemm_nvfp4_ex(**base, d=d, ldd=ldd, epilogue=H.EPI_F32, **lora)
            elif v == "addi8":  # the product added into an int8 residual stream (the ff2 form)
                H.gemm_nvfp4_ex(**base, epilogue=H.EPI_ADD_I8, resid=d8, ld_resid=n, add_scale=0.0625, **lora)
            elif v == "gelu":
                H.gemm_nvfp4_ex(**base, epilogue=H.EPI_GELU_I8, act_scale=1.0, d_i8=d8, ld_i8=n)
            elif v == "gelufp4":
                H.gemm_nvfp4_ex(**base, epilogue=H.EPI_GELU_FP4, act_scale=1.0, d_codes=codes, d_sf=sf, **lora, next_tvec=tv,
                                next_tvec_pair_stride=n, next_nvec=1, next_t=nt)
            else:
                raise SystemExit(f"unknown variant {v}")

        ms = _time(run, iters)
        out_bytes = m * n * (4 if v in ("plain", "direct", "lora") or v.startswith("aid") else (1 if v in ("gelu", "addi8") else 0.5625))
        print(f"gemm {v:8s} M={m} N={n} K={k}: {ms:.4f} ms  {2 * m * n * k / ms / 1e9:8.1f} TFLOP/s  output {out_bytes / ms / 1e6:7.1f} GB/s")
    assert H.device_error() == 0


def bench_sweep(iters):
    hbm, bf16, src = _peaks()
    fp4_peak = 4 * bf16
    print(f"FP4 dense peak taken as 4 x {bf16:.0f} TFLOP/s ({src} sustained bf16 GEMM) = {fp4_peak:.0f} TFLOP/s; nominal 9000")
    for kn in (512, 1024, 2048, 4096):
        for m in (4096, 8192, 16384):
            a, sfa, b, sfb, A, t, pairs = _operands(m, kn, kn, 1, 4096)
            d = torch.empty((m, kn), dtype=torch.float32, device="cuda")
            alpha = float(1 / np.sqrt(kn))

            def run():
                H.gemm_nvfp4_ex(a=a, b=b, sfa=sfa, sfb=sfb, m=m, n=kn, k=kn, alpha=alpha, d=d, ldd=kn, epilogue=H.EPI_F32, rank=1,
                                rows_per_member=4096, lora_t=t, t_stride=1, lora_A=A, lora_A_pair_stride=kn, lora_scale=0.01)

            ms = _time(run, iters)
            tf = (2 * m * kn * kn + 2 * m * (kn + kn)) / ms / 1e9
            print(f"perturbed gemm M={m:6d} K=N={kn:5d}: {ms:.4f} ms  {tf:8.1f} TFLOP/s  {100 * tf / fp4_peak:5.1f} % of FP4 peak "
                  f"({100 * tf / 9000:4.1f} % of nominal)")
    assert H.device_error() == 0


def bench_efla(seqs, iters, mma=2):
    T, hidden, heads, fc = 128, 512, 8, 1568
    lib.load().bnf4_set_option(b"efla_mma", mma)
    qkv = torch.randn(seqs * T, fc, device="cuda") * 0.3
    out = torch.empty(seqs * T, hidden, device="cuda")
    bb = torch.full((seqs // 32 + 1,), -2.0, device="cuda")

    def run():
        H.efla_scan(state=None, state_fp16=1, q=qkv, k=qkv[:, hidden:], v=qkv[:, 2 * hidden:], beta_raw=qkv[:, 3 * hidden:], ld_qkv=fc,
                    ld_beta=fc, beta_bias_seq=bb, seqs_per_bias=32, hidden=hidden, heads=heads, seqs=seqs, T=T, method=1, eps=1e-6,
                    out=out, ld_out=hidden)

    ms = _time(run, iters, warm=2)
    rows = seqs * T
    print(f"efla_scan ({('multiply-add', 'tensor-core fp32 rank-1', 'tensor-core fp16 accumulators')[mma]} kernel) seqs={seqs} T={T} heads={heads}x64: {ms:.4f} ms  {rows * ((3 * hidden + 1) * 4 + 4 * hidden) / ms / 1e6:7.1f} GB/s algorithmic  "
          f"{rows * heads / ms / 1e3:7.1f} M head-steps/s")


def bench_rowquant(rows, iters, fe="add"):
    hid = 512
    x = torch.randint(-127, 128, (rows, hid), dtype=torch.int8, device="cuda")
    y = torch.randn(rows, hid, device="cuda") * 20
    tv = torch.randint(-4, 5, (rows // 8192 + 1, 4, hid), dtype=torch.int8, device="cuda")
    codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
    t = torch.zeros(rows, 4, dtype=torch.int32, device="cuda")

    def run_norm():
        H.rowquant(H.FE_ABSMEAN, rows=rows, cols_in=hid, cols_out=hid, rows_per_member=4096, in_i8=x, ld_in=hid, norm_scale=1.0,
                   out_codes=codes, out_sf=sf, tvec=tv, tvec_pair_stride=4 * hid, nvec=4, t_out=t)

    if fe == "norm":  # int8 rows in (the quantiser after the residual-add GEMM epilogue)
        ms = _time(run_norm, iters)
        print(f"rowquant int8 absmean+quant rows={rows}: {ms:.4f} ms  {rows * (hid + hid // 2 + hid // 16 + 16) / ms / 1e6:7.1f} GB/s algorithmic")
        return

    def run():
        H.rowquant(H.FE_ADD_ABSMEAN, rows=rows, cols_in=hid, cols_out=hid, rows_per_member=4096, sigma=0.125, inout_i8=x, in_f32=y,
                   ld_in=hid, add_scale=1.0, norm_scale=1.0, out_codes=codes, out_sf=sf, tvec=tv, tvec_pair_stride=4 * hid, nvec=4, t_out=t)

    ms = _time(run, iters)
    print(f"rowquant add+absmean+quant rows={rows}: {ms:.4f} ms  {rows * (4 * hid + hid + hid + hid // 2 + hid // 16 + 16) / ms / 1e6:7.1f} GB/s algorithmic")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "efla", "rowquant", "sweep"])
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=0, help="gemm: output columns (default 512, 1024 for the GELU variants)")
    ap.add_argument("--k", type=int, default=0, help="gemm: reduction length (default 512)")
    ap.add_argument("--variants", default="plain,lora,direct,gelu,gelufp4")
    ap.add_argument("--seqs", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--fe", default="add", choices=["add", "norm"], help="rowquant: residual add + abs-mean norm (fp32 in) or abs-mean norm of int8 rows")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--mma", type=int, default=2, help="efla scan kernel: 2 = tensor cores with fp16 accumulators, 1 = tensor cores with an fp32 rank-1 term, 0 = multiply-add")
    a = ap.parse_args()
    if a.what == "gemm":
        bench_gemm(a.m, a.variants.split(","), a.iters, a.n, a.k)
    elif a.what == "sweep":
        bench_sweep(a.iters)
    elif a.what == "efla":
        bench_efla(a.seqs, a.iters, a.mma)
    else:
        bench_rowquant(a.rows, a.iters, a.fe)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the population-evaluation ES step (BASELINE.json metric: population tokens/s per ES step).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--pop P] [--stress] [--exact-scan]
    python bench.py --sweep                      # perturbed-NVFP4 GEMM sweep M x (K = N) with FP4 utilisation, one JSON line
    python bench.py --kernel efla|gemm|rowquant  # one kernel on a small case larger than L2 (the unit the ncu summaries profile)

One step = derive the step's noise, evaluate every antithetic pair of the population on synthetic Zipf byte
tokens, gather the per-member losses, shape the fitness and apply the ES update (including re-quantising the
base weights). With N > 1 (torchrun, one rank per GPU) the population is sharded over ranks, the per-member
losses are all-gathered with NCCL and every rank applies the identical update; the total work is fixed, so
scaling is "strong". Prints one JSON line on rank 0.

--impl reference times the CPU restatement of the reference's math (oracle/, all host threads) on a bounded
sample of the same workload: the reference's own NVFP4 path is CUDA-only, sm_120-only and cannot run here.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_HBM_GBS = 8000.0
DTYPE = "nvfp4 (e2m1 x ue4m3) with fp32 accumulation"
# DRAM bytes (read + write) per row of one launch, from ncu captures of smaller launches of the same kernels (traffic
# grows in proportion to rows); None where no capture of the current kernel exists
NCU_DRAM_BYTES_PER_ROW = {"gemm_ff1_gelu_fp4": 21.81e6 / 65536, "efla_scan": 247.71e6 / 65536, "gemm_qkv": 166.76e6 / 65536}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU port of the reference math
def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def oracle_model(cfg, weights):
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_lib as orc
    orc.lib().orc_set_num_threads(host_threads())  # launchers export OMP_NUM_THREADS=1 to their workers
    ocfg = dict(vocab=cfg.vocab, hidden=cfg.hidden, layers=cfg.layers, mlp_mult=cfg.mlp_mult, seq=cfg.seq, batch=cfg.batch,
                heads=cfg.heads, rank=cfg.rank, sigma_shift=cfg.sigma_shift, use_clt=cfg.use_clt, clt_k=cfg.clt_k, method=cfg.method,
                act_scale=cfg.act_scale, mlp_act_scale=cfg.mlp_act_scale, ln_scale=cfg.ln_scale, residual_scale=cfg.residual_scale,
                mlp_residual_scale=cfg.mlp_residual_scale, eps=cfg.eps)
    return orc, orc.OracleModel(ocfg, weights)


def oracle_pairs_seconds(orc, om, tok, tgt, pairs: int) -> float:
    """Seconds the CPU oracle needs for `pairs` antithetic pairs (forward + loss of both members) of the benchmark model."""
    t0 = time.perf_counter()
    for p in range(pairs):
        ps = orc.mix(1, orc.mix(0, p))
        om.forward(tok, tgt, ps, 1)
        om.forward(tok, tgt, ps, -1)
    return time.perf_counter() - t0


def algorithmic_work(cfg, members: int, dedup_input: bool, half_io: bool):
    """Per kernel class: (bound, bytes or flops, launches per wave) for ONE launch over a wave of `members` members.
    half_io: q | k | v and the scan's output travel as IEEE halves (heads of 64 with the chunked scan)."""
    H, F, V, T, B, L, r = cfg.hidden, cfg.hidden * cfg.mlp_mult, cfg.vocab, cfg.seq, cfg.batch, cfg.layers, cfg.rank
    rows = members * B * T
    erows = members * V if dedup_input else rows  # the embedding and its projection run once per (member, distinct token)
    fp4 = lambda k: k / 2 + k / 16  # codes + scale bytes per row
    return {
        "embed_quant": ("hbm", erows * (1 + fp4(H) + 4 * r), 1),
        "gemm_win": ("tensor", 2.0 * erows * H * H + 2.0 * erows * r * H, 1),
        "pos_gelu_norm_quant": ("hbm", rows * (4 * H + H + fp4(H) + 16 * r), 1),
        "gemm_qkv": ("tensor", 2.0 * rows * (3 * H + 1) * H + 2.0 * rows * r * (3 * H + 1), L),
        "efla_scan": ("hbm", rows * ((3 * H * 2 + 4 + 2 * H) if half_io else ((3 * H + 1) * 4 + 4 * H)), L),
        "add_norm_quant": ("hbm", rows * ((2 if half_io else 4) * H + H + H + fp4(H) + 4 * r), L),
        "norm_quant": ("hbm", rows * (H + fp4(H) + 16 * r), L),
        "gemm_ff1_gelu_fp4": ("tensor", 2.0 * rows * F * H + 2.0 * rows * r * F, L),
        "gemm_ff2": ("tensor", 2.0 * rows * H * F + 2.0 * rows * r * H, L),
        "gemm_head": ("tensor", 2.0 * rows * V * H + 2.0 * rows * r * V, 1),
        "cross_entropy": ("hbm", rows * (4 * V + 1), 1),
    }


# ------------------------------------------------------------------------------------------------ single kernels and the GEMM sweep
def _event_ms(fn, iters: int, warm: int = 3, flush=None) -> float:
    """Mean CUDA-event time of fn() over `iters` launches; flush() (outside the events) runs before every timed launch."""
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _gemm_operands(H, m, n, k, rank, rows_per_member, seed=0):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.clamp(torch.round(torch.randn(m, k, device="cuda", generator=g) * 40), -127, 127).to(torch.int8)
    w = torch.randint(-1, 2, (n, k), device="cuda", generator=g, dtype=torch.int8)
    a, sfa = H.nvfp4_quantize_a(x)
    b, sfb = H.nvfp4_quantize_b(w)
    pairs = max(1, (m + 2 * rows_per_member - 1) // (2 * rows_per_member))
    A = torch.randint(-4, 5, (pairs, n, max(rank, 1)), device="cuda", generator=g, dtype=torch.int8)
    t = torch.randint(-1000, 1000, (m, max(rank, 1)), device="cuda", generator=g, dtype=torch.int32)
    return a, sfa, b, sfb, A, t, pairs


def run_sweep(args):
    """BASELINE config 4's standalone sweep: D = alpha A B^T + rank-r term, fp32 out, M x (K = N)."""
    import numpy as np
    import torch
    from bitnet_nvfp4_b200 import host as H
    peaks, src = load_peaks()
    fp4_peak = 4.0 * peaks["bf16_tflops_sustained"]
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rank = args.rank
    points = []
    for kn in (512, 1024, 2048, 4096):
        for m in (4096, 8192, 16384):
            a, sfa, b, sfb, A, t, _ = _gemm_operands(H, m, kn, kn, rank, 4096)
            d = torch.empty((m, kn), dtype=torch.float32, device="cuda")
            alpha = float(1 / np.sqrt(kn))

            def run():
                H.gemm_nvfp4_ex(a=a, b=b, sfa=sfa, sfb=sfb, m=m, n=kn, k=kn, alpha=alpha, d=d, ldd=kn, epilogue=H.EPI_F32, rank=rank,
                                rows_per_member=4096, lora_t=t, t_stride=rank, lora_A=A, lora_A_pair_stride=kn * rank, lora_scale=0.01)

            ms = _event_ms(run, args.iters, flush=lambda: flush_buf.fill_(1))
            tf = (2.0 * m * kn * kn + 2.0 * m * rank * (kn + kn)) / ms / 1e9
            points.append({"m": m, "n": kn, "k": kn, "ms": round(ms, 5), "tflops": round(tf, 1), "frac_measured": round(tf / fp4_peak, 4),
                           "frac_nominal": round(tf / NOMINAL_FP4_TFLOPS, 4)})
    assert H.device_error() == 0
    best = max(points, key=lambda e: e["tflops"])
    print(json.dumps({"metric": "NVFP4 GEMM % of FP4 tensor peak", "value": 100.0 * best["frac_measured"], "unit": "% of 4 x sustained bf16 GEMM rate",
                      "best_point": best, "points": points, "rank": rank, "dtype": DTYPE, "data": "synthetic",
                      "peak_tflops": fp4_peak, "peak_source": f"{src}: FP4 dense peak taken as 4 x the sustained bf16 GEMM rate; nominal dense FP4 {NOMINAL_FP4_TFLOPS:.0f}",
                      "config": {"workload": f"perturbed NVFP4 GEMM sweep, M in {{4096, 8192, 16384}} x K = N in {{512, 1024, 2048, 4096}}, rank-{rank} epilogue, fp32 output",
                                 "l2": "a 256 MB buffer is written between timed launches"}}))


def run_kernel(args):
    """One kernel of the step on a small case whose inputs exceed L2; prints its CUDA-event time."""
    import numpy as np
    import torch
    from bitnet_nvfp4_b200 import host as H
    peaks, src = load_peaks()
    out = {"kernel": args.kernel, "peak_source": src}
    if args.kernel == "efla":
        T, hidden, heads, fc = 128, 512, 8, 1568
        seqs = args.seqs
        bb = torch.full((seqs // 32 + 1,), -2.0, device="cuda")
        if args.half:   # q | k | v and the output as IEEE halves, beta_raw fp32: what the batched driver feeds the chunked kernel
            qkv = (torch.randn(seqs * T, 3 * hidden, device="cuda") * 0.3).half()
            beta = torch.randn(seqs * T, device="cuda")
            y = torch.empty(seqs * T, hidden, device="cuda", dtype=torch.float16)
            kw = dict(q=qkv, k=qkv[:, hidden:], v=qkv[:, 2 * hidden:], beta_raw=beta, ld_qkv=3 * hidden, ld_beta=1, qkv_f16=1, out_f16=1)
            row_bytes = 3 * hidden * 2 + 4 + 2 * hidden
        else:
            qkv = torch.randn(seqs * T, fc, device="cuda") * 0.3
            y = torch.empty(seqs * T, hidden, device="cuda")
            kw = dict(q=qkv, k=qkv[:, hidden:], v=qkv[:, 2 * hidden:], beta_raw=qkv[:, 3 * hidden:], ld_qkv=fc, ld_beta=fc)
            row_bytes = (3 * hidden + 1) * 4 + 4 * hidden

        def run():
            H.efla_scan(state=None, state_fp16=1, beta_bias_seq=bb, seqs_per_bias=32, hidden=hidden, heads=heads, seqs=seqs, T=T, method=1,
                        eps=1e-6, out=y, ld_out=hidden, variant=args.variant, **kw)

        ms = _event_ms(run, args.iters)
        gbs = seqs * T * row_bytes / ms / 1e6
        out.update(case=f"seqs={seqs} T={T} heads={heads}x64 variant={args.variant} half_io={int(args.half)}", ms=ms, achieved=gbs, unit="GB/s",
                   frac=gbs / peaks["hbm_gbs"], algorithmic_bytes=seqs * T * row_bytes)
    elif args.kernel == "gemm":
        m, n, k, R = args.m, args.n, args.k, 4096
        a, sfa, b, sfb, A, t, pairs = _gemm_operands(H, m, n, k, args.rank, R)
        alpha = float(1 / np.sqrt(k))
        lora = dict(rank=args.rank, rows_per_member=R, lora_t=t, t_stride=max(args.rank, 1), lora_A=A, lora_A_pair_stride=n * max(args.rank, 1),
                    lora_scale=0.01) if args.rank > 0 else {}
        base = dict(a=a, b=b, sfa=sfa, sfb=sfb, m=m, n=n, k=k, alpha=alpha)
        d = torch.empty((m, n), dtype=torch.float32, device="cuda") if args.epilogue == "f32" else None
        n16 = (n - 1) // 32 * 32 if n % 32 else n   # f16 epilogue: leading multiple of 32 as halves, the rest (e.g. beta_raw) fp32
        d16 = torch.empty((m, n16), dtype=torch.float16, device="cuda") if args.epilogue == "f16" else None
        dtail = torch.empty((m, max(n - n16, 1)), dtype=torch.float32, device="cuda")
        d8 = torch.zeros((m, n), dtype=torch.int8, device="cuda")
        codes = torch.zeros(m * n // 2, dtype=torch.uint8, device="cuda")
        sf = torch.zeros(H.sf_bytes(m, n), dtype=torch.uint8, device="cuda")
        nt = torch.zeros((m, max(args.rank, 1)), dtype=torch.int32, device="cuda")
        tv = torch.randint(-4, 5, (pairs, max(args.rank, 1), n), device="cuda", dtype=torch.int8)

        def run():
            if args.epilogue == "f32":
                H.gemm_nvfp4_ex(**base, d=d, ldd=n, epilogue=H.EPI_F32, **lora)
            elif args.epilogue == "f16":
                H.gemm_nvfp4_ex(**base, d_f16=d16, ld_f16=n16, n_f16=n16, d=dtail, ldd=max(n - n16, 1), epilogue=H.EPI_F16, **lora)
            elif args.epilogue == "add_i8":
                H.gemm_nvfp4_ex(**base, epilogue=H.EPI_ADD_I8, resid=d8, ld_resid=n, add_scale=0.0625, **lora)
            elif args.epilogue == "gelu_i8":
                H.gemm_nvfp4_ex(**base, epilogue=H.EPI_GELU_I8, act_scale=1.0, d_i8=d8, ld_i8=n, **lora)
            else:
                nxt = dict(next_tvec=tv, next_tvec_pair_stride=n * args.rank, next_nvec=args.rank, next_t=nt) if args.rank > 0 else {}
                H.gemm_nvfp4_ex(**base, epilogue=H.EPI_GELU_FP4, act_scale=1.0, d_codes=codes, d_sf=sf, **lora, **nxt)

        ms = _event_ms(run, args.iters)
        tf = 2.0 * m * n * k / ms / 1e9
        out.update(case=f"M={m} N={n} K={k} epilogue={args.epilogue} rank={args.rank}", ms=ms, achieved=tf, unit="TFLOP/s",
                   frac=tf / (4.0 * peaks["bf16_tflops_sustained"]))
    else:
        rows, hid = args.rows, 512
        x = torch.randint(-127, 128, (rows, hid), dtype=torch.int8, device="cuda")
        yv = torch.randn(rows, hid, device="cuda") * 20
        tv = torch.randint(-4, 5, (rows // 8192 + 1, 4, hid), dtype=torch.int8, device="cuda")
        codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
        sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
        t = torch.zeros(rows, 4, dtype=torch.int32, device="cuda")
        nvec = 4 if args.fe == "norm" else (1 if args.half else 4)   # the step's: 4 fused q | k | v | beta projections; 1 for ff1
        common = dict(rows=rows, cols_in=hid, cols_out=hid, rows_per_member=4096, ld_in=hid, norm_scale=1.0, out_codes=codes, out_sf=sf,
                      tvec=tv, tvec_pair_stride=4 * hid, nvec=nvec, t_out=t)
        if args.fe == "norm":   # abs-mean norm of int8 rows (after the residual-add GEMM epilogue)
            run = lambda: H.rowquant(H.FE_ABSMEAN, in_i8=x, **common)
            nbytes = rows * (hid + hid // 2 + hid // 16 + 16)
        elif args.half:         # residual add of a branch travelling as IEEE halves (the scan's output in the step) + abs-mean norm
            yh = (yv * 0.01).half()
            run = lambda: H.rowquant(H.FE_ADD_ABSMEAN, sigma=0.125, inout_i8=x, in_f32=yh, in_f16=1, add_scale=100.0, **common)
            nbytes = rows * (2 * hid + hid + hid + hid // 2 + hid // 16 + 4)
        else:                   # residual add of an fp32 branch + abs-mean norm
            run = lambda: H.rowquant(H.FE_ADD_ABSMEAN, sigma=0.125, inout_i8=x, in_f32=yv, add_scale=1.0, **common)
            nbytes = rows * (4 * hid + hid + hid + hid // 2 + hid // 16 + 16)
        ms = _event_ms(run, args.iters)
        out.update(case=f"rows={rows} hidden={hid} front-end={args.fe}" + (" half branch" if args.half and args.fe == "add" else ""), ms=ms, achieved=nbytes / ms / 1e6, unit="GB/s", frac=nbytes / ms / 1e6 / peaks["hbm_gbs"])
    assert H.device_error() == 0
    print(json.dumps(out))


# ------------------------------------------------------------------------------------------------ the ES step
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--pop", type=int, default=0, help="population (default 2048; 128 with --stress)")
    ap.add_argument("--stress", action="store_true",
                    help="the scaled-up stress widths instead of the default model: hidden 2048, 12 layers, 32 heads of 64, MLP 8192, seq 512, "
                         "batch 16, rank-4 perturbations")
    ap.add_argument("--wave", type=int, default=0, help="members per wave (0 = library default)")
    ap.add_argument("--exact-scan", action="store_true", help="per-token EFLA kernel (fp16 state rounding after every token) instead of the chunked one")
    ap.add_argument("--graph", action="store_true", help="replay every wave of the evaluation as one CUDA graph (the reference's --cuda_graph)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-pairs", type=int, default=6, help="largest CPU sample, in antithetic pairs (about 2 s of CPU work each on 16 threads)")
    ap.add_argument("--cpu-seconds", type=float, default=20.0, help="CPU work per sample the reference arm / CPU baseline aims for")
    ap.add_argument("--sweep", action="store_true", help="perturbed-GEMM sweep instead of the ES step")
    ap.add_argument("--kernel", choices=["efla", "gemm", "rowquant"], help="time one kernel on a small case instead of the ES step")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--seqs", type=int, default=512, help="--kernel efla: sequences")
    ap.add_argument("--variant", type=int, default=0, help="--kernel efla: 0 library default, 2 per-token, 3 chunked")
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=512)
    ap.add_argument("--k", type=int, default=512)
    ap.add_argument("--rank", type=int, default=-1, help="--kernel gemm / --sweep: rank of the perturbation term (defaults 1 / 4)")
    ap.add_argument("--epilogue", default="f32", choices=["f32", "f16", "gelu_i8", "gelu_fp4", "add_i8"])
    ap.add_argument("--half", action="store_true", help="--kernel efla: q | k | v and the output as IEEE halves; --kernel rowquant --fe add: the branch as halves")
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--fe", default="add", choices=["add", "norm"])
    ap.add_argument("--train", action="store_true",
                    help="the reference driver's epoch loop instead of the timed step: a fresh batch per epoch, ES step, loss of the updated "
                         "model on the training batch, periodic validation loss; reports the reference's tok/s_eval and tok/s_total")
    ap.add_argument("--epochs", type=int, default=5)
    ap.add_argument("--val-every", type=int, default=1)
    ap.add_argument("--corpus", default="", help="--train: a byte corpus file (e.g. Tiny Shakespeare); default: the seeded synthetic Zipf corpus")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.sweep or args.kernel:
        if rank != 0:
            return
        import torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: libbnf4 has no CPU fallback")
        torch.cuda.set_device(local_rank)
        if args.rank < 0:
            args.rank = 4 if args.sweep else 1
        return run_sweep(args) if args.sweep else run_kernel(args)

    from bitnet_nvfp4_b200 import population, synth  # noqa: E402  (imports torch)
    if args.pop <= 0:
        args.pop = 128 if args.stress else 2048
    if args.stress:
        cfg = population.Config(hidden=2048, layers=12, mlp_mult=4, seq=512, batch=16, heads=32, rank=4, max_pairs=args.pop // 2,
                                wave_members=args.wave)
        args.no_cpu_baseline = True
    else:
        cfg = population.Config(max_pairs=args.pop // 2, wave_members=args.wave)
    tokens_per_step = args.pop * cfg.batch * cfg.seq
    workload = (f"{'stress-width' if args.stress else 'default'} ES step: pop={args.pop} (antithetic pairs), batch={cfg.batch}, seq={cfg.seq}, hidden={cfg.hidden}, "
                f"layers={cfg.layers}, mlp_mult={cfg.mlp_mult}, heads={cfg.heads}x{cfg.hidden // cfg.heads}, rank-{cfg.rank} "
                f"perturbation, sigma=2^-{cfg.sigma_shift}, lr=0.8, thresh=0.008, centered-rank fitness")
    config = {"workload": workload, "pop": args.pop, "global_batch_tokens": tokens_per_step,
              "parallelism": f"population sharded over {world} GPU(s), NCCL all-gather of {args.pop} fp32 losses",
              "l2": "inputs larger than L2 (every wave streams GBs of activations)"}

    weights = synth.init_weights(cfg)
    corpus = synth.zipf_corpus(1 << 20, 1.1, 123)
    tok, tgt = synth.sample_batch(corpus, cfg.batch, cfg.seq, 123)

    # ------------------------------------------------------------------ reference arm (CPU port of the reference math)
    if args.impl == "reference":
        if rank != 0:
            return
        if args.stress:
            print(json.dumps({"impl": "reference", "unavailable": "the CPU port is timed on the default model only (one member of the stress widths takes minutes)"}))
            return
        orc, om = oracle_model(cfg, weights)
        threads = orc.lib().orc_num_threads()
        pair_s = oracle_pairs_seconds(orc, om, tok, tgt, 1)                  # warm-up, and the measure that sizes the sample
        pairs = max(1, min(args.cpu_pairs, int(args.cpu_seconds / max(pair_s, 1e-3))))
        for _ in range(max(0, min(args.warmup, 3) - 1)):
            oracle_pairs_seconds(orc, om, tok, tgt, 1)
        times = [oracle_pairs_seconds(orc, om, tok, tgt, pairs) for _ in range(args.steps)]
        sec = sum(times) / len(times)
        val = 2 * pairs * cfg.batch * cfg.seq / sec
        sample = f"{pairs} antithetic pair(s) = {2 * pairs} members x {cfg.batch * cfg.seq} tokens per step (forward + loss only), {sec:.1f} s of CPU work per step"
        print(json.dumps({
            "impl": "reference", "metric": "population tokens/s per ES step", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ------------------------------------------------------------------ our arm
    import torch
    import torch.distributed as dist
    from bitnet_nvfp4_b200 import host as bhost
    from bitnet_nvfp4_b200 import lib as blib
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libbnf4 has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = blib.load()
    if args.exact_scan:
        blib.check(L.bnf4_set_option(b"efla_chunked", 0))

    pairs_total = args.pop // 2
    assert pairs_total % world == 0, "population pairs must divide evenly over ranks"
    my_pairs = pairs_total // world

    model = population.PopulationModel(cfg)
    model.set_weights(weights)
    if args.graph:
        model.set_graph(True)
    if args.train:
        # the reference's per-epoch log (src/train_efla_lm.cpp:5733-5800) for `--epochs` epochs, then one JSON line with the
        # throughput definitions of :5786-5792 averaged over the epochs after the first
        from bitnet_nvfp4_b200 import trainer
        data = synth.load_corpus(args.corpus) if args.corpus else corpus
        tc = trainer.TrainConfig(epochs=args.epochs, pairs=pairs_total, seed=1, val_every=args.val_every)
        recs = trainer.train(model, data, tc, rank=rank, world=world, log=lambda line: print(line, file=sys.stderr))
        code = bhost.device_error()
        if code != 0:
            raise SystemExit(f"a bounded wait expired inside a kernel (code {code}): results invalid")
        if rank == 0:
            tail = recs[1:] if len(recs) > 1 else recs
            mean = lambda k: sum(r[k] for r in tail) / len(tail)
            print(json.dumps({
                "metric": "tok/s_total of the training loop (population evaluation + update + train/val evaluation, per epoch wall time)",
                "value": mean("tok_s_total"), "unit": "tokens/s", "tok_s_eval": mean("tok_s_eval"), "n_gpus": world, "epochs": args.epochs,
                "higher_is_better": True, "dtype": DTYPE, "data": args.corpus or "synthetic", "config": config,
                "train_loss_first": recs[0]["train_loss"], "train_loss_last": recs[-1]["train_loss"],
                "val_loss_last": next((r["val_loss"] for r in reversed(recs) if "val_loss" in r), None),
                "epoch_wall_ms": mean("wall_s") * 1e3, "eval_ms": mean("eval_s") * 1e3, "update_ms": mean("update_s") * 1e3,
                "train_eval_ms": mean("train_s") * 1e3, "val_eval_ms": mean("val_s") * 1e3}))
        model.close()
        if world > 1:
            dist.destroy_process_group()
        return
    tok_d = torch.from_numpy(tok).cuda()
    tgt_d = torch.from_numpy(tgt).cuda()
    tok_h = torch.from_numpy(tok).pin_memory()
    tgt_h = torch.from_numpy(tgt).pin_memory()
    model.set_tokens(tok_d, tgt_d)
    losses_all = torch.empty(2 * pairs_total, dtype=torch.float32, device="cuda")
    losses_host = torch.empty(2 * pairs_total, dtype=torch.float32).pin_memory()
    coll_spans = []  # (name, start event, end event) around every collective of the timed steps

    def step(epoch: int, from_host: bool, spans=None):
        if from_host:
            model.set_tokens(tok_h, tgt_h)            # H2D of the step's inputs (pinned host memory)
        # evaluate this rank's pairs, all-gather the losses (NCCL), shape (4 KB host round trip, as the reference), update
        losses = population.es_step(model, 1, epoch, pairs_total, rank, world, lr=0.8, thresh=0.008, losses_out=losses_all, spans=spans)
        if from_host:
            losses_host.copy_(losses, non_blocking=True)  # D2H of the step's result

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n_steps: int, first_epoch: int, from_host: bool, spans=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_steps):
            step(first_epoch + i, from_host, spans)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for i in range(max(args.warmup, 3)):
        step(i, False)
    barrier()
    assert bhost.device_error() == 0, "a bounded wait expired in a kernel during warm-up"

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    model.set_timing(True)
    launches0 = L.bnf4_launch_count()
    ms_total = timed(args.steps, 100, False, coll_spans if world > 1 else None)
    launches = L.bnf4_launch_count() - launches0
    timing = model.get_timing()
    model.set_timing(False)
    clocks = sampler.stop() if sampler else None
    assert bhost.device_error() == 0, "a bounded wait expired in a kernel during the timed region"

    ms_e2e = timed(args.steps, 200, True)
    assert torch.isfinite(losses_host).all()
    assert bhost.device_error() == 0

    # exposed time of the collectives on the launching stream (max over ranks), and a digest of every rank's weights
    coll_ms = {}
    for name, a, b in coll_spans:
        coll_ms[name] = coll_ms.get(name, 0.0) + a.elapsed_time(b)
    ranks_bit_identical = None
    if world > 1:
        names = sorted(coll_ms)
        t = torch.tensor([coll_ms[n] for n in names], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        coll_ms = {n: t[i].item() / args.steps for i, n in enumerate(names)}
        w_now = model.get_weights()
        shadow, ema = model.get_optimizer_state()
        hsh = hashlib.sha256()
        for n in sorted(w_now):
            hsh.update(w_now[n].tobytes())
        hsh.update(shadow.tobytes())
        hsh.update(ema.tobytes())
        digests = [None] * world
        dist.all_gather_object(digests, hsh.hexdigest())
        ranks_bit_identical = len(set(digests)) == 1

    ms_step = ms_total / args.steps
    value = tokens_per_step / (ms_step * 1e-3)
    e2e_value = tokens_per_step / (ms_e2e / args.steps * 1e-3)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ------------------------------------------------------------------ per kernel class: achieved rate on algorithmic work
    peaks, peak_src = load_peaks()
    wave_members = model.wave_members
    dedup_input = cfg.vocab <= 256 and cfg.vocab < cfg.batch * cfg.seq
    half_io = (cfg.hidden // cfg.heads) == 64 and not args.exact_scan
    work = algorithmic_work(cfg, wave_members, dedup_input, half_io)
    n_waves = args.steps * ((my_pairs * 2 + wave_members - 1) // wave_members)
    fp4_peak = 4.0 * peaks["bf16_tflops_sustained"]
    kernels = []
    for name, (ms, cnt) in timing.items():
        if cnt == 0 or ms <= 0:
            continue
        ent = {"name": name, "launch_groups_ms": ms, "launches": cnt, "share": ms / ms_total}
        if name in work:
            # HBM: measured copy bandwidth / nominal 8 TB/s; GEMMs: 4 x measured sustained bf16 / nominal dense FP4 9 PF
            bound, amount, per_wave = work[name]
            dur = ms * 1e-3 / (n_waves * per_wave)   # average duration of one launch
            if bound == "hbm":
                ent.update(achieved=amount / dur / 1e9, unit="GB/s", frac_measured=amount / dur / 1e9 / peaks["hbm_gbs"],
                           frac_nominal=amount / dur / 1e9 / NOMINAL_HBM_GBS, avg_launch_ms=dur * 1e3)
            else:
                ent.update(achieved=amount / dur / 1e12, unit="TFLOP/s", frac_measured=amount / dur / 1e12 / fp4_peak,
                           frac_nominal=amount / dur / 1e12 / NOMINAL_FP4_TFLOPS, avg_launch_ms=dur * 1e3)
        kernels.append(ent)
    kernels.sort(key=lambda e: -e["launch_groups_ms"])
    roof = None
    for ent in kernels:   # the class with the largest share of the step
        if ent["name"] in work:
            bound, amount, per_wave = work[ent["name"]]
            bpr = NCU_DRAM_BYTES_PER_ROW.get(ent["name"])
            roof = {"kernel": ent["name"], "bound": bound, "achieved": ent["achieved"], "peak": peaks["hbm_gbs"] if bound == "hbm" else fp4_peak,
                    "unit": ent["unit"], "frac": ent["frac_measured"],
                    "traffic": bpr * wave_members * cfg.batch * cfg.seq if bpr else None, "avg_launch_ms": ent["avg_launch_ms"],
                    "peak_source": peak_src + (" (FP4 dense peak taken as 4x the measured sustained bf16 GEMM rate)" if bound == "tensor" else " (copy bandwidth)")}
            break

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        orc, om = oracle_model(cfg, weights)
        pair_s = oracle_pairs_seconds(orc, om, tok, tgt, 1)
        pairs = max(1, min(args.cpu_pairs, int(args.cpu_seconds / max(pair_s, 1e-3))))
        sec = oracle_pairs_seconds(orc, om, tok, tgt, pairs)
        cpu_baseline = {"value": 2 * pairs * cfg.batch * cfg.seq / sec, "unit": "tokens/s", "cores": orc.lib().orc_num_threads(), "kind": "port",
                        "sample": f"{pairs} antithetic pair(s) = {2 * pairs} members x {cfg.batch * cfg.seq} tokens, forward + loss, {sec:.1f} s of CPU work"}

    # the reference's tok/s_eval excludes the update (src/train_efla_lm.cpp:5786-5792)
    update_ms = sum(ms for name, (ms, cnt) in timing.items() if name in ("update_z_sumsq", "update_apply", "requantize_weights"))
    tokens_per_s_eval = tokens_per_step / ((ms_total - update_ms) / args.steps * 1e-3)
    out = {
        "metric": "population tokens/s per ES step", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": config,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": int(tok_h.numel() + tgt_h.numel()),
                "d2h_bytes_per_step": int(losses_host.numel() * 4)},
        "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu_baseline,
        "kernels": [{k: (round(v, 4) if isinstance(v, float) else v) for k, v in e.items()} for e in kernels],
        "tokens_per_s_eval": tokens_per_s_eval, "device_bytes": model.device_bytes, "wave_members": wave_members,
        "efla_scan_kernel": "per-token (fp16 state rounding every token)" if args.exact_scan else "chunked (16 tokens per step, fp16 state rounding every chunk)",
    }
    if args.graph:
        out["cuda_graph_launches"] = model.graph_launches
    if world > 1:
        out["allgather_exposed_ms"] = coll_ms.get("loss_allgather")
        out["collectives_exposed_ms"] = coll_ms
        out["ranks_bit_identical"] = ranks_bit_identical
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

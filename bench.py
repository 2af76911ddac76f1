#!/usr/bin/env python
"""Benchmark of the population-evaluation ES step (BASELINE.json metric: population tokens/s per ES step).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

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


def oracle_member_seconds(cfg, weights, tok, tgt, pairs: int):
    """Seconds the CPU oracle needs for `pairs` antithetic pairs of the benchmark model, and the threads it used."""
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_lib as orc
    ocfg = dict(vocab=cfg.vocab, hidden=cfg.hidden, layers=cfg.layers, mlp_mult=cfg.mlp_mult, seq=cfg.seq, batch=cfg.batch,
                heads=cfg.heads, rank=cfg.rank, sigma_shift=cfg.sigma_shift, use_clt=cfg.use_clt, clt_k=cfg.clt_k, method=cfg.method,
                act_scale=cfg.act_scale, mlp_act_scale=cfg.mlp_act_scale, ln_scale=cfg.ln_scale, residual_scale=cfg.residual_scale,
                mlp_residual_scale=cfg.mlp_residual_scale, eps=cfg.eps)
    om = orc.OracleModel(ocfg, weights)
    threads = orc.lib().orc_num_threads()
    t0 = time.perf_counter()
    for p in range(pairs):
        ps = orc.mix(1, orc.mix(0, p))
        om.forward(tok, tgt, ps, 1)
        om.forward(tok, tgt, ps, -1)
    return time.perf_counter() - t0, threads


def algorithmic_work(cfg, members: int):
    """Per kernel class: (bound, bytes or flops) for ONE wave launch over `members` members."""
    H, F, V, T, B, L, r = cfg.hidden, cfg.hidden * cfg.mlp_mult, cfg.vocab, cfg.seq, cfg.batch, cfg.layers, cfg.rank
    rows = members * B * T
    fp4 = lambda k: k / 2 + k / 16  # codes + scale bytes per row
    return {
        "embed_quant": ("hbm", rows * (1 + fp4(H) + 4 * r)),
        "gemm_win": ("tensor", 2.0 * rows * H * H + 2.0 * rows * r * H),
        "pos_gelu_norm_quant": ("hbm", rows * (4 * H + H + fp4(H) + 16 * r)),
        "gemm_qkv": ("tensor", 2.0 * rows * (3 * H + 1) * H + 2.0 * rows * r * (3 * H + 1)),
        "efla_scan": ("hbm", rows * ((3 * H + 1) * 4 + 4 * H)),
        "add_norm_quant": ("hbm", rows * (4 * H + H + H + fp4(H) + 4 * r)),
        "norm_quant": ("hbm", rows * (H + fp4(H) + 16 * r)),
        "gemm_ff1_gelu_fp4": ("tensor", 2.0 * rows * F * H + 2.0 * rows * r * F),
        "gemm_ff2": ("tensor", 2.0 * rows * H * F + 2.0 * rows * r * H),
        "gemm_head": ("tensor", 2.0 * rows * V * H + 2.0 * rows * r * V),
        "cross_entropy": ("hbm", rows * (4 * V + 1)),
    }


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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-pairs", type=int, default=6, help="pairs in the CPU-baseline sample (about 2 s of CPU work each on 16 threads)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

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
        pairs = max(1, args.cpu_pairs)
        for _ in range(min(args.warmup, 1)):
            oracle_member_seconds(cfg, weights, tok, tgt, 1)
        times, threads = [], 1
        for _ in range(args.steps):
            t, threads = oracle_member_seconds(cfg, weights, tok, tgt, pairs)
            times.append(t)
        sec = sum(times) / len(times)
        val = 2 * pairs * cfg.batch * cfg.seq / sec
        sample = f"{pairs} antithetic pair(s) = {2 * pairs} members x {cfg.batch * cfg.seq} tokens per step (forward + loss only)"
        print(json.dumps({
            "impl": "reference", "metric": "population tokens/s per ES step", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3) with fp32 accumulation", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ------------------------------------------------------------------ our arm
    import torch
    import torch.distributed as dist
    from bitnet_nvfp4_b200 import lib as blib
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libbnf4 has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = blib.load()

    pairs_total = args.pop // 2
    assert pairs_total % world == 0, "population pairs must divide evenly over ranks"
    my_pairs = pairs_total // world
    my_begin = rank * my_pairs

    model = population.PopulationModel(cfg)
    model.set_weights(weights)
    tok_d = torch.from_numpy(tok).cuda()
    tgt_d = torch.from_numpy(tgt).cuda()
    tok_h = torch.from_numpy(tok).pin_memory()
    tgt_h = torch.from_numpy(tgt).pin_memory()
    model.set_tokens(tok_d, tgt_d)
    losses_all = torch.empty(2 * pairs_total, dtype=torch.float32, device="cuda")
    losses_host = torch.empty(2 * pairs_total, dtype=torch.float32).pin_memory()

    def step(epoch: int, from_host: bool):
        if from_host:
            model.set_tokens(tok_h, tgt_h)            # H2D of the step's inputs (pinned host memory)
        # evaluate this rank's pairs, all-gather the losses (NCCL), shape (4 KB host round trip, as the reference), update
        losses = population.es_step(model, 1, epoch, pairs_total, rank, world, lr=0.8, thresh=0.008, losses_out=losses_all)
        if from_host:
            losses_host.copy_(losses, non_blocking=True)  # D2H of the step's result

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n_steps: int, first_epoch: int, from_host: bool):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_steps):
            step(first_epoch + i, from_host)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for i in range(max(args.warmup, 3)):
        step(i, False)
    barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    model.set_timing(True)
    launches0 = L.bnf4_launch_count()
    ms_total = timed(args.steps, 100, False)
    launches = L.bnf4_launch_count() - launches0
    timing = model.get_timing()
    model.set_timing(False)
    clocks = sampler.stop() if sampler else None

    ms_e2e = timed(args.steps, 200, True)
    assert torch.isfinite(losses_host).all()

    ms_step = ms_total / args.steps
    value = tokens_per_step / (ms_step * 1e-3)
    e2e_value = tokens_per_step / (ms_e2e / args.steps * 1e-3)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ------------------------------------------------------------------ roofline of the dominant kernel class
    peaks, peak_src = load_peaks()
    wave_members = model.wave_members
    work = algorithmic_work(cfg, wave_members)
    kernels = []
    n_waves = args.steps * ((my_pairs * 2 + wave_members - 1) // wave_members)
    for name, (ms, cnt) in timing.items():
        if cnt == 0 or ms <= 0:
            continue
        ent = {"name": name, "launch_groups_ms": ms, "launches": cnt, "share": ms / ms_total}
        if name in work:
            # achieved rate on algorithmic work, as a fraction of the measured peak and of the nominal one
            # (HBM: measured copy bandwidth / nominal 8 TB/s; GEMMs: 4 x measured sustained bf16 / nominal dense FP4 9 PF)
            bound, amount = work[name]
            per_wave = cfg.layers if name in ("gemm_qkv", "efla_scan", "gemm_ff1_gelu_fp4", "gemm_ff2") else \
                (cfg.layers if name in ("add_norm_quant", "norm_quant") else 1)
            rate = amount * n_waves * per_wave / (ms * 1e-3)
            if bound == "hbm":
                ent.update(achieved=rate / 1e9, unit="GB/s", frac_measured=rate / 1e9 / peaks["hbm_gbs"], frac_nominal=rate / 8e12)
                if name == "efla_scan":
                    # not bandwidth-bound in this formulation: also the arithmetic rate (6 * head_dim^2 flops per head and token)
                    # and the share of the mma.sync tensor pipe that its 48 MMAs per head and token (8.6 cycles each per SM
                    # sub-partition, measured) take at the sampled SM clock
                    hd = cfg.hidden // cfg.heads
                    rows_total = amount / ((3 * cfg.hidden + 1) * 4 + 4 * cfg.hidden) * n_waves * per_wave
                    ent["achieved_tflops"] = rows_total * 6.0 * cfg.heads * hd * hd / (ms * 1e-3) / 1e12
                    if hd == 64:
                        sms = torch.cuda.get_device_properties(local_rank).multi_processor_count
                        ent["mma_pipe_frac"] = rows_total * cfg.heads * 48 * 8.6 / (4 * sms * 1.965e9 * ms * 1e-3)
            else:
                ent.update(achieved=rate / 1e12, unit="TFLOP/s", frac_measured=rate / 1e12 / (4.0 * peaks["bf16_tflops_sustained"]),
                           frac_nominal=rate / 9e15)
        kernels.append(ent)
    kernels.sort(key=lambda e: -e["launch_groups_ms"])
    roof = None
    for ent in kernels:
        if ent["name"] in work:
            bound, amount = work[ent["name"]]
            per_layer = cfg.layers if ent["name"] in ("gemm_qkv", "efla_scan", "gemm_ff1_gelu_fp4", "gemm_ff2") else \
                (cfg.layers if ent["name"] in ("add_norm_quant", "norm_quant") else 1)
            n_wave_launches = args.steps * ((my_pairs * 2 + wave_members - 1) // wave_members) * per_layer
            dur = ent["launch_groups_ms"] * 1e-3 / n_wave_launches
            if bound == "hbm":
                achieved, peak, unit = amount / dur / 1e9, peaks["hbm_gbs"], "GB/s"
            else:
                achieved, peak, unit = amount / dur / 1e12, 4.0 * peaks["bf16_tflops_sustained"], "TFLOP/s"
            # DRAM bytes (read + write) per row from the ncu capture of a smaller launch of the same kernel
            # (profiles/efla_scan64_seqs512_T128.md: 527.85 MB for 65536 rows), scaled by the rows of one launch here
            ncu_bytes_per_row = {"efla_scan": 524.71e6 / 65536}
            traffic = ncu_bytes_per_row[ent["name"]] * wave_members * cfg.batch * cfg.seq if ent["name"] in ncu_bytes_per_row else None
            roof = {"kernel": ent["name"], "bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                    "traffic": traffic, "avg_launch_ms": dur * 1e3, "peak_source": peak_src +
                    (" (FP4 dense peak taken as 4x the measured sustained bf16 GEMM rate)" if bound == "tensor" else " (copy bandwidth)")}
            break

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        sec, threads = oracle_member_seconds(cfg, weights, tok, tgt, args.cpu_pairs)
        cpu_baseline = {"value": 2 * args.cpu_pairs * cfg.batch * cfg.seq / sec, "unit": "tokens/s", "cores": threads, "kind": "port",
                        "sample": f"{args.cpu_pairs} antithetic pair(s) = {2 * args.cpu_pairs} members x {cfg.batch * cfg.seq} tokens, "
                                  f"forward + loss, {sec:.1f} s of CPU work"}

    # the reference's tok/s_eval excludes the update (src/train_efla_lm.cpp:5786-5792)
    update_ms = sum(ms for name, (ms, cnt) in timing.items() if name in ("update_z_sumsq", "update_apply", "requantize_weights"))
    tokens_per_s_eval = tokens_per_step / ((ms_total - update_ms) / args.steps * 1e-3)
    out = {
        "metric": "population tokens/s per ES step", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3) with fp32 accumulation", "data": "synthetic", "config": config,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": int(tok_h.numel() + tgt_h.numel()),
                "d2h_bytes_per_step": int(losses_host.numel() * 4)},
        "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu_baseline,
        "kernels": [{k: (round(v, 4) if isinstance(v, float) else v) for k, v in e.items()} for e in kernels],
        "tokens_per_s_eval": tokens_per_s_eval, "device_bytes": model.device_bytes, "wave_members": wave_members,
    }
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

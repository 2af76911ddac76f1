"""The reference driver's epoch loop around the batched ES step.

Per epoch, as src/train_efla_lm.cpp:5255-5800 does: schedules for lr and the update threshold (:405-418, :5263-5266), a
training batch drawn with seed mix(data_seed, epoch) (:5243-5250, :5283), the population evaluation and update, the loss of
the UPDATED unperturbed model on the training batch (:5717-5733), every `val_every` epochs the loss on a fixed validation
batch drawn with `val_seed` (:5741-5764), and the throughput figures tok/s_eval and tok/s_total with the reference's
definitions (:5786-5792). The model's sigma is fixed at creation (the reference's sigma schedule defaults to constant).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from . import population, synth

SCHEDULES = {"constant": 0, "linear": 1, "cosine": 2, "exp": 3}  # TrainConfig::Schedule, src/train_efla_lm.cpp:278


def schedule_value(start: float, end: float, schedule: int | str, t01: float) -> float:
    """schedule_value of the reference (src/train_efla_lm.cpp:405-418), evaluated in fp32 like it."""
    f = np.float32
    sc = SCHEDULES[schedule] if isinstance(schedule, str) else int(schedule)
    start, end = f(start), f(end)
    t = f(min(max(f(t01), f(0.0)), f(1.0)))
    e = end if end >= 0 else start
    if sc == 0:
        return float(start)
    if sc == 1:
        return float(f(start + f(f(e - start) * t)))
    if sc == 2:
        ct = f(f(0.5) * f(f(1.0) - f(math.cos(float(f(f(math.pi) * t))))))
        return float(f(start + f(f(e - start) * ct)))
    if start <= 0 or e <= 0:
        return float(f(start + f(f(e - start) * t)))
    return float(f(start * f(math.pow(float(f(e / start)), float(t)))))


@dataclass
class TrainConfig:
    """The subset of the reference's TrainConfig this loop reads (same names, same defaults; src/train_efla_lm.cpp:205-300)."""
    epochs: int = 1
    pairs: int = 1024
    seed: int = 1
    data_seed: int = 0          # 0: inherit from seed (:4790)
    val_seed: int = 12345
    val_every: int = 1
    do_val: bool = True
    fixed_train: bool = False
    lr: float = 0.8
    lr_end: float = 0.05
    lr_schedule: str = "cosine"
    update_threshold: float = 0.008
    update_threshold_end: float = -1.0
    thresh_schedule: str = "exp"
    fitness_mode: int = 2       # centered rank
    fitness_clip: float = 3.0
    update_kw: dict = field(default_factory=dict)


def _loss_of(model, tokens: np.ndarray, targets: np.ndarray) -> float:
    model.set_tokens(tokens, targets)
    return float(model.eval_base().item())


def train(model, corpus: np.ndarray, cfg: TrainConfig, rank: int = 0, world: int = 1, group=None, log=None) -> list[dict]:
    """Runs cfg.epochs epochs on `model` (a population.PopulationModel) and returns one record per epoch with the reference's
    log fields. Every rank must call it with the same arguments; `log` (rank 0) receives each record's line."""
    B, T = model.cfg.batch, model.cfg.seq
    data_seed = cfg.data_seed or cfg.seed
    on_gpu = torch.cuda.is_available()

    def sync():
        if on_gpu:
            torch.cuda.synchronize()

    records = []
    val_batch = synth.sample_batch(corpus, B, T, cfg.val_seed) if cfg.do_val else None
    for epoch in range(cfg.epochs):
        sync()
        t_epoch = time.perf_counter()
        t01 = 1.0 if cfg.epochs <= 1 else epoch / (cfg.epochs - 1)
        lr_t = schedule_value(cfg.lr, cfg.lr_end, cfg.lr_schedule, t01)
        thresh_t = schedule_value(cfg.update_threshold, cfg.update_threshold_end, cfg.thresh_schedule, t01)
        t0 = time.perf_counter()
        seed0 = data_seed if cfg.fixed_train else synth.mix(data_seed, epoch)
        tokens, targets = synth.sample_batch(corpus, B, T, seed0)
        sample_s = time.perf_counter() - t0
        model.set_tokens(tokens, targets)
        marks = {}
        population.es_step(model, cfg.seed, epoch, cfg.pairs, rank=rank, world=world, group=group, lr=lr_t, thresh=thresh_t,
                           fitness_mode=cfg.fitness_mode, fitness_clip=cfg.fitness_clip, marks=marks, **cfg.update_kw)
        sync()
        eval_s, update_s = marks.get("eval_s", 0.0), marks.get("update_s", 0.0)
        t0 = time.perf_counter()
        train_loss = float(model.eval_base().item())  # the updated model on the batch it was just trained on
        train_s = time.perf_counter() - t0
        rec = {"epoch": epoch, "lr": lr_t, "thresh": thresh_t, "sigma": model.cfg.sigma_shift, "train_loss": train_loss,
               "train_ppl": math.exp(train_loss)}
        do_val = cfg.do_val and cfg.val_every > 0 and epoch % cfg.val_every == 0
        val_s = 0.0
        if do_val:
            t0 = time.perf_counter()
            rec["val_loss"] = _loss_of(model, *val_batch)
            rec["val_ppl"] = math.exp(rec["val_loss"])
            if cfg.fixed_train:
                model.set_tokens(tokens, targets)
            val_s = time.perf_counter() - t0
        sync()
        wall_s = time.perf_counter() - t_epoch
        tokens_eval = cfg.pairs * 2.0 * B * T
        tokens_total = tokens_eval + B * T + (B * T if do_val else 0)
        rec.update(wall_s=wall_s, sample_s=sample_s, eval_s=eval_s, update_s=update_s, train_s=train_s, val_s=val_s,
                   tok_s_eval=tokens_eval / eval_s if eval_s > 0 else 0.0, tok_s_total=tokens_total / wall_s if wall_s > 0 else 0.0)
        records.append(rec)
        if log is not None and rank == 0:
            log(" ".join(f"{k} {v:.6g}" if isinstance(v, float) else f"{k} {v}" for k, v in rec.items()))
    return records

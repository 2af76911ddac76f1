"""CPU test of the data-parallel ES step: world_size 2 over gloo.

The orchestration under test is the product's population.es_step (shard pairs -> evaluate -> all-gather losses ->
shape -> identical update on every rank). The evaluator injected here is a CPU stand-in built on the oracle
(test infrastructure), so the test needs no GPU; on the GPU the same function drives the CUDA model.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as orc

CFG = dict(hidden=128, layers=1, seq=8, batch=2, heads=2, rank=1, max_pairs=6)
SALT = dict(emb=0x111111, win=0x222222, wq=0x333333, wk=0x444444, wv=0x555555, wbeta=0x666666, ff1=0x999999, ff2=0xAAAAAA, head=0x777777)


class OracleEvaluator:
    """prepare_step / eval_pairs / update with the oracle's arithmetic (matrices only; enough to test the plumbing)."""

    def __init__(self, cfg, weights, tok, tgt):
        self.cfg, self.w, self.tok, self.tgt = cfg, {k: v.copy() for k, v in weights.items()}, tok, tgt
        self.shadow = {k: v.astype(np.float32) for k, v in self.w.items() if v.dtype == np.int8}
        self.ema = {}
        self.evaluated = []

    def _ocfg(self):
        return {k: getattr(self.cfg, k) for k in "vocab hidden layers mlp_mult seq batch heads rank sigma_shift use_clt clt_k method act_scale "
                                                 "mlp_act_scale ln_scale residual_scale mlp_residual_scale eps".split()}

    def prepare_step(self, seed, epoch, pairs):
        self.seed, self.epoch, self.pairs = seed, epoch, pairs

    def eval_pairs(self, begin, count):
        om = orc.OracleModel(self._ocfg(), self.w)
        out = []
        for p in range(begin, begin + count):
            self.evaluated.append(p)
            ps = orc.mix(self.seed, orc.mix(self.epoch, p))
            out += [om.forward(self.tok, self.tgt, ps, 1), om.forward(self.tok, self.tgt, ps, -1)]
        return torch.tensor(out, dtype=torch.float32)

    def _matrices(self):
        H, V = self.cfg.hidden, self.cfg.vocab
        return (("emb", V, H), ("win", H, H), ("head", V, H))

    def _apply(self, name, rows, cols, Z, lr, th):
        ss = orc.sumsq(Z)
        inv, self.ema[name] = orc.update_inv_rms(ss, self.ema.get(name, 0.0), True, 0.95, 1e-3, rows * cols)
        orc.update_shadow_ternary(self.w[name].reshape(-1), self.shadow[name].reshape(-1), Z, inv, lr, th)

    def update(self, pair_weights, lr, thresh):
        from bitnet_nvfp4_b200 import host
        self.sharded_updates = getattr(self, "sharded_updates", 0)
        pw = pair_weights.numpy().astype(np.float32)
        seeds = orc.fill_pair_seeds(self.seed, self.epoch, self.pairs)
        th = float(np.float32(thresh) * np.sqrt(np.float32(self.pairs)))
        for name, rows, cols in self._matrices():
            Z, _ = orc.compute_z_sumsq_lowrank(pw, seeds, SALT[name], rows, cols, self.cfg.rank, host.c_rank(self.cfg.rank))
            self._apply(name, rows, cols, Z, lr, th)

    def update_sharded(self, pair_weights, rank, world, group, lr, thresh):
        """Row-sharded Z + the product's in-place all-gather (population.gather_z_shards), then the same apply step."""
        from bitnet_nvfp4_b200 import host, population
        self.sharded_updates = getattr(self, "sharded_updates", 0) + 1
        pw = pair_weights.numpy().astype(np.float32)
        seeds = orc.fill_pair_seeds(self.seed, self.epoch, self.pairs)
        th = float(np.float32(thresh) * np.sqrt(np.float32(self.pairs)))
        entries, off = [], 0
        for name, rows, cols in self._matrices():
            entries.append((off, rows * cols, rows % world == 0))
            off += rows * cols
        z_all = torch.full((off,), float("nan"), dtype=torch.float32)
        for (name, rows, cols), (o, n, sharded) in zip(self._matrices(), entries):
            Z, _ = orc.compute_z_sumsq_lowrank(pw, seeds, SALT[name], rows, cols, self.cfg.rank, host.c_rank(self.cfg.rank))
            if sharded:  # this rank contributes only its rows
                per = n // world
                z_all[o + rank * per:o + (rank + 1) * per] = torch.from_numpy(Z[rank * per:(rank + 1) * per])
            else:
                z_all[o:o + n] = torch.from_numpy(Z)
        population.gather_z_shards(z_all, entries, rank, world, group)
        assert not torch.isnan(z_all).any()
        for (name, rows, cols), (o, n, _) in zip(self._matrices(), entries):
            self._apply(name, rows, cols, z_all[o:o + n].numpy().copy(), lr, th)


def _setup():
    from bitnet_nvfp4_b200 import population, synth
    cfg = population.Config(**CFG)
    w = synth.init_weights(cfg)
    tok, tgt = synth.sample_batch(synth.zipf_corpus(1 << 14), cfg.batch, cfg.seq, 5)
    return cfg, w, tok, tgt


def _worker(rank, world, port, pairs, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bitnet_nvfp4_b200 import population
    cfg, w, tok, tgt = _setup()
    ev = OracleEvaluator(cfg, w, tok, tgt)
    losses = None
    for epoch in range(2):
        losses = population.es_step(ev, 1, epoch, pairs, rank, world, lr=0.8, thresh=0.008)
    assert ev.sharded_updates == 2  # with more than one rank the step takes the row-sharded update
    q.put((rank, sorted(set(ev.evaluated)), losses.numpy(), {k: ev.w[k].copy() for k in ("emb", "win", "head")}))
    dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@pytest.mark.parametrize("pairs", [6, 5])
def test_two_ranks_agree_with_one(pairs):
    from bitnet_nvfp4_b200 import population
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, pairs, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=240) for _ in range(2)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # single-rank run of the same two steps
    cfg, w, tok, tgt = _setup()
    ev = OracleEvaluator(cfg, w, tok, tgt)
    for epoch in range(2):
        ref_losses = population.es_step(ev, 1, epoch, pairs, 0, 1, lr=0.8, thresh=0.008)
    (r0, ev0, l0, w0), (r1, ev1, l1, w1) = res
    # the shards partition the pairs, contiguous and disjoint
    assert ev0 == list(range(*(lambda b, c: (b, b + c))(*population.shard_pairs(pairs, 0, 2))))
    assert ev1 == list(range(*(lambda b, c: (b, b + c))(*population.shard_pairs(pairs, 1, 2))))
    assert sorted(ev0 + ev1) == list(range(pairs))
    # every rank sees the same gathered losses and ends with the same weights as the single-rank run
    assert np.array_equal(l0, l1) and np.array_equal(l0, ref_losses.numpy())
    for k in ("emb", "win", "head"):
        assert np.array_equal(w0[k], w1[k]) and np.array_equal(w0[k], ev.w[k])
    assert any((w0[k] != w[k]).any() for k in ("emb", "win", "head"))


class TrainableEvaluator(OracleEvaluator):
    """The evaluator with the two calls the epoch loop adds: a new batch, and the loss of the unperturbed model."""

    def set_tokens(self, tokens, targets):
        self.tok, self.tgt = np.ascontiguousarray(tokens), np.ascontiguousarray(targets)

    def eval_base(self):
        return torch.tensor([orc.OracleModel(self._ocfg(), self.w).forward(self.tok, self.tgt, 0, 0)], dtype=torch.float32)


def _train_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from bitnet_nvfp4_b200 import synth, trainer
    cfg, w, tok, tgt = _setup()
    ev = TrainableEvaluator(cfg, w, tok, tgt)
    recs = trainer.train(ev, synth.zipf_corpus(1 << 14), trainer.TrainConfig(epochs=2, pairs=4, seed=9, val_every=2), rank=rank, world=world)
    q.put((rank, [(r["train_loss"], r.get("val_loss")) for r in recs], {k: ev.w[k].copy() for k in ("emb", "win", "head")}))
    if world > 1:
        dist.destroy_process_group()


def test_epoch_loop_on_two_ranks_equals_one():
    """trainer.train over gloo: both ranks log the same train / validation losses as a single-rank run and end with its weights."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_train_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=240) for _ in range(2)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    import queue as _queue
    single = _queue.Queue()
    _train_worker(0, 1, port, single)
    _, ref_losses, ref_w = single.get()
    for _, losses, wts in res:
        assert losses == ref_losses
        assert all(np.array_equal(wts[k], ref_w[k]) for k in ref_w)
    assert ref_losses[0][1] is not None and ref_losses[1][1] is None  # validation on epoch 0 only (val_every = 2)


def test_shard_pairs_partitions():
    from bitnet_nvfp4_b200 import population
    for total in (1, 5, 1024, 1023):
        for world in (1, 2, 3, 8):
            spans = [population.shard_pairs(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (b0, c0), (b1, _) in zip(spans, spans[1:]):
                assert b0 + c0 == b1
    assert [population.shard_pairs(1024, r, 8) for r in (0, 7)] == [(0, 128), (896, 128)]

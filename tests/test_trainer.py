"""The epoch loop (bitnet_nvfp4_b200/trainer.py) against the reference driver's: schedules bit-exact against values recorded
from the reference's own schedule_value, batch seeds, validation cadence and the throughput definitions; on a GPU the loop
must equal the same sequence of ES steps issued by hand."""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from bitnet_nvfp4_b200 import synth, trainer

GOLD = np.load(Path(__file__).parent / "golden" / "ref_host.npz")


def test_schedule_value_matches_reference():
    for (start, end, sched, t01), ref in zip(GOLD["sched_in"], GOLD["sched_out"]):
        assert np.float32(trainer.schedule_value(start, end, int(sched), t01)) == ref


def test_seed_mixer_matches_reference():
    for a, b, m in zip(GOLD["mix_a"], GOLD["mix_b"], GOLD["mix"]):
        assert synth.mix(int(a), int(b)) == int(m)


class FakeModel:
    """Records what the loop asks of the model; the loss is a hash of the tokens it holds."""

    class Cfg:
        batch, seq, sigma_shift = 4, 16, 3

    def __init__(self):
        self.cfg = self.Cfg()
        self.calls = []
        self.tokens = None

    def set_tokens(self, tokens, targets):
        self.tokens = np.asarray(tokens).copy()
        self.calls.append(("tokens", int(self.tokens.astype(np.int64).sum())))

    def prepare_step(self, seed, epoch, pairs):
        self.calls.append(("prepare", seed, epoch, pairs))

    def eval_pairs(self, begin, count):
        self.calls.append(("eval", begin, count))
        return torch.arange(2 * count, dtype=torch.float32)

    def update(self, weights, lr, thresh, **kw):
        self.calls.append(("update", round(lr, 6), round(thresh, 6)))

    def eval_base(self):
        self.calls.append(("base", int(self.tokens.astype(np.int64).sum())))
        return torch.tensor([1.0 + (int(self.tokens.sum()) % 7) * 0.1])


def test_epoch_loop_follows_the_reference_driver():
    corpus = synth.zipf_corpus(1 << 12, 1.1, 5)
    cfg = trainer.TrainConfig(epochs=4, pairs=8, seed=77, val_every=2, lr=0.8, lr_end=0.05, update_threshold=0.008)
    m = FakeModel()
    lines = []
    recs = trainer.train(m, corpus, cfg, log=lines.append)
    assert len(recs) == 4 and len(lines) == 4
    # batches: mix(data_seed = seed, epoch); validation batch from val_seed on epochs 0 and 2 only
    tok_sums = [int(synth.sample_batch(corpus, 4, 16, synth.mix(77, e))[0].astype(np.int64).sum()) for e in range(4)]
    val_sum = int(synth.sample_batch(corpus, 4, 16, 12345)[0].astype(np.int64).sum())
    expect = []
    for e in range(4):
        t01 = e / 3
        expect += [("tokens", tok_sums[e]), ("prepare", 77, e, 8), ("eval", 0, 8),
                   ("update", round(trainer.schedule_value(0.8, 0.05, "cosine", t01), 6), round(trainer.schedule_value(0.008, -1.0, "exp", t01), 6)),
                   ("base", tok_sums[e])]
        if e % 2 == 0:
            expect += [("tokens", val_sum), ("base", val_sum)]
    assert m.calls == expect
    assert [("val_loss" in r) for r in recs] == [True, False, True, False]
    for r in recs:
        assert r["train_ppl"] == math.exp(r["train_loss"])
        tokens_eval = 8 * 2 * 4 * 16
        assert r["tok_s_eval"] == pytest.approx(tokens_eval / r["eval_s"])
        assert r["tok_s_total"] == pytest.approx((tokens_eval + 64 + (64 if "val_loss" in r else 0)) / r["wall_s"])
    assert recs[0]["lr"] == pytest.approx(0.8) and recs[-1]["lr"] == pytest.approx(0.05)


def test_fixed_train_restores_the_training_batch():
    corpus = synth.zipf_corpus(1 << 12, 1.1, 5)
    m = FakeModel()
    trainer.train(m, corpus, trainer.TrainConfig(epochs=2, pairs=2, seed=3, data_seed=9, fixed_train=True))
    train_sum = int(synth.sample_batch(corpus, 4, 16, 9)[0].astype(np.int64).sum())   # the seed itself, not mix(seed, epoch)
    toks = [c for c in m.calls if c[0] == "tokens"]
    assert toks[0] == ("tokens", train_sum) and toks[2] == ("tokens", train_sum)  # set, validation, restored
    assert toks[3] == ("tokens", train_sum)


@pytest.mark.gpu
def test_train_loop_equals_manual_steps():
    from bitnet_nvfp4_b200 import population
    cfgm = population.Config(hidden=128, layers=2, seq=32, batch=4, heads=2, max_pairs=8)
    corpus = synth.zipf_corpus(1 << 14, 1.1, 123)
    tc = trainer.TrainConfig(epochs=3, pairs=8, seed=11, val_every=2)

    def fresh():
        m = population.PopulationModel(cfgm)
        m.set_weights(synth.init_weights(cfgm))
        return m

    a = fresh()
    recs = trainer.train(a, corpus, tc)
    b = fresh()
    manual = []
    for e in range(3):
        tok, tgt = synth.sample_batch(corpus, 4, 32, synth.mix(11, e))
        b.set_tokens(tok, tgt)
        t01 = e / 2
        population.es_step(b, 11, e, 8, lr=trainer.schedule_value(0.8, 0.05, "cosine", t01),
                           thresh=trainer.schedule_value(0.008, -1.0, "exp", t01))
        manual.append(float(b.eval_base().item()))
    assert [r["train_loss"] for r in recs] == manual
    wa, wb = a.get_weights(), b.get_weights()
    assert all(np.array_equal(wa[k], wb[k]) for k in wa)
    assert "val_loss" in recs[0] and "val_loss" not in recs[1] and "val_loss" in recs[2]
    assert all(math.isfinite(r["train_loss"]) and r["tok_s_eval"] > 0 for r in recs)
    a.close(); b.close()

"""Multi-GPU check of the row-sharded ES update, launched by torchrun (one rank per GPU, NCCL):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        tests/multigpu_sharded_update.py

Every rank runs the same two ES steps twice on two models: once with the noise sums of the update computed by rows across
the ranks and all-gathered (the default with more than one rank), once replicated, once through the single C entry point
bnf4_model_es_step with the collectives as callbacks. Weights and optimiser state must be bit-identical between the three and
across ranks. test_gpu_population.py runs this file when two GPUs are visible.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from bitnet_nvfp4_b200 import population, synth
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    cfg = population.Config(hidden=128, layers=2, seq=16, batch=4, heads=2, rank=2, max_pairs=8, wave_members=8)
    w = synth.init_weights(cfg)
    tok, tgt = synth.sample_batch(synth.zipf_corpus(1 << 16, 1.1, 123), cfg.batch, cfg.seq, 123)
    models = []
    for mode in ("sharded", "replicated", "single call"):
        m = population.PopulationModel(cfg)
        m.set_weights(w)
        m.set_tokens(tok, tgt)
        for epoch in range(2):
            if mode == "single call":  # bnf4_model_es_step with the collectives supplied as callbacks
                population.es_step_native(m, 1, epoch, 8, rank, world)
            else:
                population.es_step(m, 1, epoch, 8, rank, world, shard_update=(mode == "sharded"))
        models.append(m)
    wa, wb, wc = (m.get_weights() for m in models)
    for k in wa:
        assert np.array_equal(wa[k], wb[k]), k
        assert np.array_equal(wa[k], wc[k]), k
    (sa, ea), (sb, eb), (sc, ec) = (m.get_optimizer_state() for m in models)
    assert np.array_equal(sa, sb) and np.array_equal(ea, eb)
    assert np.array_equal(sa, sc) and np.array_equal(ea, ec)
    assert any((wa[k] != w[k]).any() for k in ("emb", "win", "ff1"))
    # the same bits on every rank
    digest = torch.tensor([float(np.abs(sa).sum()), float(sum(int(np.abs(wa[k].astype(np.int64)).sum()) for k in wa if wa[k].dtype == np.int8))],
                          dtype=torch.float64, device="cuda")
    parts = [torch.empty_like(digest) for _ in range(world)]
    dist.all_gather(parts, digest)
    assert all(torch.equal(p, parts[0]) for p in parts)
    dist.barrier()
    if rank == 0:
        print(f"sharded update OK on {world} ranks")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

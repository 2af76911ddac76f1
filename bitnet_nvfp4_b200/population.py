"""Population-evaluation ES step on one GPU: binding of the bnf4_model_* entry points (include/bnf4.h).

Mirrors, at the granularity of one ES step, what the reference's train_efla_lm does per epoch
(src/train_efla_lm.cpp:5255-5657): derive pair seeds, evaluate every antithetic pair, shape the fitness,
update the weights. The work is done by libbnf4.so; this module only moves pointers.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, asdict

import numpy as np
import torch

from . import lib as _l

c_int, c_float, c_void_p = C.c_int, C.c_float, C.c_void_p


class ModelCfg(C.Structure):
    """bnf4_model_cfg"""

    _fields_ = [(n, c_int) for n in "vocab hidden layers mlp_mult seq batch heads rank sigma_shift use_clt clt_k method".split()] + \
               [(n, c_float) for n in "act_scale mlp_act_scale ln_scale residual_scale mlp_residual_scale eps".split()] + \
               [("max_pairs", c_int), ("wave_members", c_int)]


class ModelWeights(C.Structure):
    """bnf4_model_weights (host pointers)"""

    _fields_ = [(n, c_void_p) for n in "emb win wq wk wv wbeta ff1 ff2 head head_bias beta_bias pos".split()]


class UpdateCfg(C.Structure):
    """bnf4_update_cfg"""

    _fields_ = [("lr", c_float), ("thresh", c_float), ("use_adaptive", c_int), ("adaptive_beta", c_float),
                ("adaptive_eps", c_float), ("train_pos", c_int)]


_ALLGATHER_FN = C.CFUNCTYPE(c_int, c_void_p, c_void_p, C.c_size_t, c_void_p)
_GROUP_FN = C.CFUNCTYPE(c_int, c_void_p)


class Collectives(C.Structure):
    """bnf4_collectives"""

    _fields_ = [("ctx", c_void_p), ("allgather_inplace", _ALLGATHER_FN), ("group_begin", _GROUP_FN), ("group_end", _GROUP_FN)]


class EsStepCfg(C.Structure):
    """bnf4_es_step_cfg"""

    _fields_ = [("seed", C.c_uint64), ("epoch", C.c_uint64), ("pairs", c_int), ("rank", c_int), ("world", c_int), ("fitness_mode", c_int),
                ("fitness_clip", c_float), ("update", UpdateCfg)]


_l.register({
    "bnf4_model_es_step": (c_int, [c_void_p, C.POINTER(EsStepCfg), C.POINTER(Collectives), c_void_p, c_void_p]),
    "bnf4_model_create": (c_int, [C.POINTER(ModelCfg), C.POINTER(c_void_p)]),
    "bnf4_model_destroy": (c_int, [c_void_p]),
    "bnf4_model_device_bytes": (C.c_size_t, [c_void_p]),
    "bnf4_model_set_weights": (c_int, [c_void_p, C.POINTER(ModelWeights)]),
    "bnf4_model_get_weights": (c_int, [c_void_p, C.POINTER(ModelWeights)]),
    "bnf4_model_set_tokens": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "bnf4_model_prepare_step": (c_int, [c_void_p, C.c_uint64, C.c_uint64, c_int, c_void_p]),
    "bnf4_model_prepare_step_range": (c_int, [c_void_p, C.c_uint64, C.c_uint64, c_int, c_int, c_int, c_void_p]),
    "bnf4_model_eval_pairs": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "bnf4_model_eval_base": (c_int, [c_void_p, c_void_p, c_void_p]),
    "bnf4_model_update": (c_int, [c_void_p, c_void_p, C.POINTER(UpdateCfg), c_void_p]),
    "bnf4_model_update_z_layout": (c_int, [c_void_p, c_int, c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong), C.POINTER(c_int),
                                           C.POINTER(C.c_longlong)]),
    "bnf4_model_update_z": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "bnf4_model_update_apply": (c_int, [c_void_p, c_void_p, c_void_p, C.POINTER(UpdateCfg), c_void_p]),
    "bnf4_model_read_buffer": (c_int, [c_void_p, C.c_char_p, c_void_p, C.c_size_t]),
    "bnf4_model_launches_per_wave": (c_int, [c_void_p]),
    "bnf4_model_wave_members": (c_int, [c_void_p]),
    "bnf4_model_optimizer_state_sizes": (c_int, [c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "bnf4_model_get_optimizer_state": (c_int, [c_void_p, c_void_p, c_void_p]),
    "bnf4_model_set_optimizer_state": (c_int, [c_void_p, c_void_p, c_void_p]),
    "bnf4_model_set_timing": (c_int, [c_void_p, c_int]),
    "bnf4_model_set_graph": (c_int, [c_void_p, c_int]),
    "bnf4_model_graph_launches": (C.c_longlong, [c_void_p]),
    "bnf4_model_num_kernel_classes": (c_int, []),
    "bnf4_model_kernel_class_name": (C.c_char_p, [c_int]),
    "bnf4_model_get_timing": (c_int, [c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_longlong), c_int]),
})

WEIGHT_NAMES = "emb win wq wk wv wbeta ff1 ff2 head head_bias beta_bias pos".split()


@dataclass
class Config:
    """Defaults are the reference's (TrainConfig, src/train_efla_lm.cpp:186-300) except heads and rank, which follow
    the benchmark configuration (8 heads of 64, rank-1 perturbations)."""
    vocab: int = 256
    hidden: int = 512
    layers: int = 4
    mlp_mult: int = 2
    seq: int = 128
    batch: int = 32
    heads: int = 8
    rank: int = 1
    sigma_shift: int = 3
    use_clt: int = 1
    clt_k: int = 4
    method: int = 1
    act_scale: float = 0.8
    mlp_act_scale: float = 1.0
    ln_scale: float = 1.0
    residual_scale: float = 1.0
    mlp_residual_scale: float = 1.0
    eps: float = 1e-6
    max_pairs: int = 1024
    wave_members: int = 0

    def weight_shapes(self) -> dict:
        V, H, L, F, T = self.vocab, self.hidden, self.layers, self.hidden * self.mlp_mult, self.seq
        return {"emb": (V, H), "win": (H, H), "wq": (L, H, H), "wk": (L, H, H), "wv": (L, H, H), "wbeta": (L, H),
                "ff1": (L, F, H), "ff2": (L, H, F), "head": (V, H), "head_bias": (V,), "beta_bias": (L,), "pos": (T, H)}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class PopulationModel:
    def __init__(self, cfg: Config):
        self.cfg = cfg
        self.lib = _l.load()
        self._c = ModelCfg(**asdict(cfg))
        self.h = c_void_p()
        _l.check(self.lib.bnf4_model_create(C.byref(self._c), C.byref(self.h)))
        self.pairs = 0

    def close(self):
        if self.h:
            self.lib.bnf4_model_destroy(self.h)
            self.h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def device_bytes(self) -> int:
        return self.lib.bnf4_model_device_bytes(self.h)

    @property
    def launches_per_wave(self) -> int:
        return self.lib.bnf4_model_launches_per_wave(self.h)

    @property
    def wave_members(self) -> int:
        return self.lib.bnf4_model_wave_members(self.h)

    def _weights_struct(self, arrays: dict) -> ModelWeights:
        return ModelWeights(*[arrays[n].ctypes.data for n in WEIGHT_NAMES])

    def set_weights(self, weights: dict):
        shapes = self.cfg.weight_shapes()
        arrays = {}
        for n in WEIGHT_NAMES:
            dt = np.float32 if n in ("head_bias", "beta_bias", "pos") else np.int8
            a = np.ascontiguousarray(weights[n], dtype=dt)
            assert a.shape == shapes[n], (n, a.shape, shapes[n])
            arrays[n] = a
        _l.check(self.lib.bnf4_model_set_weights(self.h, C.byref(self._weights_struct(arrays))))

    def get_weights(self) -> dict:
        shapes = self.cfg.weight_shapes()
        arrays = {n: np.zeros(shapes[n], np.float32 if n in ("head_bias", "beta_bias", "pos") else np.int8) for n in WEIGHT_NAMES}
        _l.check(self.lib.bnf4_model_get_weights(self.h, C.byref(self._weights_struct(arrays))))
        return arrays

    def get_optimizer_state(self):
        """(shadow, ema): fp32 shadows of the nine weight tensors, concatenated, and the RMS-EMA scalars."""
        ns, ne = C.c_size_t(0), C.c_size_t(0)
        _l.check(self.lib.bnf4_model_optimizer_state_sizes(self.h, C.byref(ns), C.byref(ne)))
        shadow, ema = np.zeros(ns.value, np.float32), np.zeros(ne.value, np.float32)
        _l.check(self.lib.bnf4_model_get_optimizer_state(self.h, shadow.ctypes.data, ema.ctypes.data))
        return shadow, ema

    def set_optimizer_state(self, shadow, ema):
        shadow, ema = np.ascontiguousarray(shadow, np.float32), np.ascontiguousarray(ema, np.float32)
        ns, ne = C.c_size_t(0), C.c_size_t(0)
        _l.check(self.lib.bnf4_model_optimizer_state_sizes(self.h, C.byref(ns), C.byref(ne)))
        assert shadow.size == ns.value and ema.size == ne.value
        _l.check(self.lib.bnf4_model_set_optimizer_state(self.h, shadow.ctypes.data, ema.ctypes.data))

    def save_checkpoint(self, path, epoch: int):
        """Everything a resumed run needs: weights, optimiser state and the epoch counter (noise is a function of seed and epoch)."""
        shadow, ema = self.get_optimizer_state()
        np.savez(path, epoch=np.int64(epoch), shadow=shadow, ema=ema, **self.get_weights())

    def load_checkpoint(self, path) -> int:
        z = np.load(path)
        self.set_weights({n: z[n] for n in WEIGHT_NAMES})
        self.set_optimizer_state(z["shadow"], z["ema"])
        return int(z["epoch"])

    def set_tokens(self, tokens, targets):
        """tokens/targets: uint8 [B][T], torch CUDA tensors or (pinned) host tensors / numpy arrays."""
        def ptr(x):
            if isinstance(x, torch.Tensor):
                assert x.dtype == torch.uint8 and x.is_contiguous()
                return x.data_ptr(), x.is_cuda
            x = np.ascontiguousarray(x, np.uint8)
            self._keep = getattr(self, "_keep", []) + [x]
            return x.ctypes.data, False
        (pt, dt), (pg, dg) = ptr(tokens), ptr(targets)
        assert dt == dg
        _l.check(self.lib.bnf4_model_set_tokens(self.h, pt, pg, int(dt), _stream()))
        if getattr(self, "_keep", None):
            # numpy inputs were copied to temporaries: wait for the H2D copies before releasing them
            torch.cuda.current_stream().synchronize()
            self._keep = []

    def prepare_step(self, seed: int, epoch: int, pairs: int):
        _l.check(self.lib.bnf4_model_prepare_step(self.h, seed, epoch, pairs, _stream()))
        self.pairs = pairs

    def prepare_step_range(self, seed: int, epoch: int, pairs: int, eval_begin: int, eval_count: int):
        """prepare_step for a rank that evaluates only pairs [eval_begin, eval_begin + eval_count): the per-pair noise that
        only an evaluation reads is generated for that range alone."""
        self.pairs = pairs
        _l.check(self.lib.bnf4_model_prepare_step_range(self.h, seed, epoch, pairs, eval_begin, eval_count, _stream()))

    def eval_pairs(self, pair_begin: int, pair_count: int, out: torch.Tensor | None = None) -> torch.Tensor:
        """Returns a float32 CUDA tensor [2*pair_count]: (loss+, loss-) per pair."""
        if out is None:
            out = torch.empty(2 * pair_count, dtype=torch.float32, device="cuda")
        _l.check(self.lib.bnf4_model_eval_pairs(self.h, pair_begin, pair_count, out.data_ptr(), _stream()))
        return out

    def eval_base(self) -> torch.Tensor:
        out = torch.empty(1, dtype=torch.float32, device="cuda")
        _l.check(self.lib.bnf4_model_eval_base(self.h, out.data_ptr(), _stream()))
        return out

    def update(self, pair_weights: torch.Tensor, lr=0.8, thresh=0.008, use_adaptive=True, adaptive_beta=0.95, adaptive_eps=1e-3,
               train_pos=True):
        assert pair_weights.is_cuda and pair_weights.dtype == torch.float32 and pair_weights.numel() == self.pairs
        u = UpdateCfg(lr, thresh, int(use_adaptive), adaptive_beta, adaptive_eps, int(train_pos))
        _l.check(self.lib.bnf4_model_update(self.h, pair_weights.data_ptr(), C.byref(u), _stream()))

    def z_layout(self, nshards: int):
        """[(offset, elems, sharded)] of every ternary matrix inside the Z buffer of a sharded update, and its size in floats."""
        n = self.lib.bnf4_model_update_z_layout(self.h, nshards, 0, None, None, None, None)
        if n < 0:
            _l.check(1)
        off, el, sh, tot = (C.c_longlong * n)(), (C.c_longlong * n)(), (c_int * n)(), C.c_longlong(0)
        if self.lib.bnf4_model_update_z_layout(self.h, nshards, n, off, el, sh, C.byref(tot)) < 0:
            _l.check(1)
        return [(off[i], el[i], bool(sh[i])) for i in range(n)], tot.value

    def update_sharded(self, pair_weights: torch.Tensor, rank: int, world: int, group=None, lr=0.8, thresh=0.008, use_adaptive=True,
                       adaptive_beta=0.95, adaptive_eps=1e-3, train_pos=True, spans=None):
        """The update of `update`, with Z of every ternary matrix computed by rows on `world` ranks and all-gathered in place
        (same kernels, same summation order: the weights end bit-identical to `update`)."""
        assert pair_weights.is_cuda and pair_weights.dtype == torch.float32 and pair_weights.numel() == self.pairs
        key = world
        if getattr(self, "_z_key", None) != key:
            self._z_entries, total = self.z_layout(world)
            self._z_all = torch.empty(total, dtype=torch.float32, device="cuda")
            self._z_key = key
        u = UpdateCfg(lr, thresh, int(use_adaptive), adaptive_beta, adaptive_eps, int(train_pos))
        _l.check(self.lib.bnf4_model_update_z(self.h, pair_weights.data_ptr(), rank, world, self._z_all.data_ptr(), _stream()))
        with _span(spans, "z_allgather"):
            gather_z_shards(self._z_all, self._z_entries, rank, world, group)
        _l.check(self.lib.bnf4_model_update_apply(self.h, pair_weights.data_ptr(), self._z_all.data_ptr(), C.byref(u), _stream()))

    def set_graph(self, enable: bool):
        """Replay every wave of the evaluation as one CUDA graph (the reference's --cuda_graph, src/train_efla_lm.cpp:3779-3819):
        first run of a wave eager, second captured, then one graph launch per wave. Same results as the eager launches."""
        _l.check(self.lib.bnf4_model_set_graph(self.h, int(enable)))

    @property
    def graph_launches(self) -> int:
        return int(self.lib.bnf4_model_graph_launches(self.h))

    def set_timing(self, enable: bool):
        _l.check(self.lib.bnf4_model_set_timing(self.h, int(enable)))

    def get_timing(self) -> dict:
        """{kernel class: (milliseconds, launches)} accumulated since set_timing(True). Synchronises."""
        n = self.lib.bnf4_model_num_kernel_classes()
        ms = (C.c_double * n)()
        cnt = (C.c_longlong * n)()
        _l.check(self.lib.bnf4_model_get_timing(self.h, ms, cnt, n))
        return {self.lib.bnf4_model_kernel_class_name(i).decode(): (ms[i], cnt[i]) for i in range(n)}

    def read_buffer(self, name: str, dtype, count: int) -> np.ndarray:
        out = np.zeros(count, dtype)
        _l.check(self.lib.bnf4_model_read_buffer(self.h, name.encode(), out.ctypes.data, out.nbytes))
        return out


class _span:
    """Records a CUDA-event pair on the current stream around a block and appends (name, start, end) to `spans`: the time the
    stream spends between the two events is the exposed time of the collectives issued inside. No-op when spans is None."""

    def __init__(self, spans, name):
        self.spans, self.name = spans, name

    def __enter__(self):
        if self.spans is not None:
            self.a = torch.cuda.Event(enable_timing=True)
            self.a.record()

    def __exit__(self, *exc):
        if self.spans is not None:
            b = torch.cuda.Event(enable_timing=True)
            b.record()
            self.spans.append((self.name, self.a, b))
        return False


def shard_pairs(pairs_total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous pair range [begin, begin + count) evaluated by `rank` (reference: eval_ranges,
    src/train_efla_lm.cpp:5067-5077). Both members of a pair stay on one rank."""
    base, rem = divmod(pairs_total, world)
    begin = rank * base + min(rank, rem)
    return begin, base + (1 if rank < rem else 0)


def gather_z_shards(z_all: torch.Tensor, entries, rank: int, world: int, group=None):
    """In-place all-gather of the row shards of every sharded matrix inside z_all: rank r owns the r-th of `world` equal
    contiguous blocks of each (offset, elems, sharded=True) entry."""
    import contextlib
    import torch.distributed as dist
    if world <= 1:
        return
    # NCCL: one grouped launch for all tensors; other backends: one collective per tensor
    batch = contextlib.nullcontext()
    if dist.get_backend(group) == "nccl" and hasattr(dist, "_coalescing_manager"):
        batch = dist._coalescing_manager(group=group, device=z_all.device, async_ops=False)
    with batch:
        for off, n, sharded in entries:
            if not sharded:
                continue
            full = z_all[off:off + n]
            per = n // world
            dist.all_gather_into_tensor(full, full[rank * per:(rank + 1) * per], group=group)


def es_step(model, seed: int, epoch: int, pairs_total: int, rank: int = 0, world: int = 1, group=None, lr: float = 0.8,
            thresh: float = 0.008, fitness_mode: int = 2, fitness_clip: float = 3.0, losses_out: torch.Tensor | None = None,
            shard_update: bool = True, spans: list | None = None, marks: dict | None = None, **update_kw) -> torch.Tensor:
    """One ES step on this rank: evaluate this rank's pairs, all-gather the per-member losses over `group`
    (torch.distributed), shape the fitness and apply the identical deterministic update on every rank. With more than one
    rank the noise sums of the update are computed by rows across the ranks and all-gathered (shard_update=False replicates
    them like the reference does); either way every rank ends with the same bits.
    `model` is a PopulationModel (or any object with prepare_step / eval_pairs / update). Returns all 2*pairs_total losses.
    `spans`: optional list that receives (name, start event, end event) around every collective (CUDA devices only).
    `marks`: optional dict that receives the host-clock durations "eval_s" (noise + evaluation + loss gather, the reference's
    eval_s) and "update_s" (shaping + update); asking for them adds two device synchronisations."""
    import time
    import torch.distributed as dist

    def _now():
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return time.perf_counter()

    t_start = _now() if marks is not None else 0.0
    begin, count = shard_pairs(pairs_total, rank, world)
    if world > 1 and hasattr(model, "prepare_step_range"):
        model.prepare_step_range(seed, epoch, pairs_total, begin, count)
    else:
        model.prepare_step(seed, epoch, pairs_total)
    mine = model.eval_pairs(begin, count)
    if world > 1:
        if pairs_total % world == 0:
            losses = losses_out if losses_out is not None else torch.empty(2 * pairs_total, dtype=mine.dtype, device=mine.device)
            with _span(spans if mine.is_cuda else None, "loss_allgather"):
                dist.all_gather_into_tensor(losses, mine, group=group)
        else:  # ragged shards: gather with padding
            cap = 2 * (pairs_total // world + 1)
            padded = torch.zeros(cap, dtype=mine.dtype, device=mine.device)
            padded[: mine.numel()] = mine
            parts = [torch.empty_like(padded) for _ in range(world)]
            dist.all_gather(parts, padded, group=group)
            losses = torch.cat([parts[r][: 2 * shard_pairs(pairs_total, r, world)[1]] for r in range(world)])
    else:
        losses = mine
    t_eval = _now() if marks is not None else 0.0
    weights = shape_fitness(fitness_from_losses(losses), fitness_mode, fitness_clip)
    if world > 1 and shard_update and hasattr(model, "update_sharded"):
        model.update_sharded(weights, rank, world, group, lr=lr, thresh=thresh, **({"spans": spans} if spans is not None else {}), **update_kw)
    else:
        model.update(weights, lr=lr, thresh=thresh, **update_kw)
    if marks is not None:
        marks["eval_s"] = t_eval - t_start
        marks["update_s"] = _now() - t_eval
    return losses


class _DevBytes:
    """A raw device range as an object torch.as_tensor accepts."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def torch_collectives(rank: int, world: int, group=None):
    """bnf4_collectives over torch.distributed (NCCL): what a C++ host writes with ncclAllGather / ncclGroupStart / ncclGroupEnd.
    Returns the struct and the objects that must stay alive while it is in use."""
    import torch.distributed as dist
    state = {"batch": None}

    def allgather(_ctx, recv, bytes_per_rank, _stream_ptr):
        try:
            full = torch.as_tensor(_DevBytes(recv, bytes_per_rank * world), device="cuda")
            dist.all_gather_into_tensor(full, full[rank * bytes_per_rank:(rank + 1) * bytes_per_rank], group=group)
            return 0
        except Exception:  # an exception must not cross the C boundary
            import traceback
            traceback.print_exc()
            return 1

    def begin(_ctx):
        if dist.get_backend(group) == "nccl" and hasattr(dist, "_coalescing_manager"):
            state["batch"] = dist._coalescing_manager(group=group, device=torch.device("cuda", torch.cuda.current_device()), async_ops=False)
            state["batch"].__enter__()
        return 0

    def end(_ctx):
        if state["batch"] is not None:
            state["batch"].__exit__(None, None, None)
            state["batch"] = None
        return 0

    fns = (_ALLGATHER_FN(allgather), _GROUP_FN(begin), _GROUP_FN(end))
    return Collectives(None, *fns), fns


def es_step_native(model: "PopulationModel", seed: int, epoch: int, pairs_total: int, rank: int = 0, world: int = 1, group=None,
                   lr: float = 0.8, thresh: float = 0.008, fitness_mode: int = 2, fitness_clip: float = 3.0,
                   losses_out: torch.Tensor | None = None, use_adaptive=True, adaptive_beta=0.95, adaptive_eps=1e-3, train_pos=True) -> torch.Tensor:
    """es_step through the single C entry point bnf4_model_es_step: the rank orchestration runs inside the library and only the
    collectives come back to the host as callbacks. Same results as es_step, bit for bit."""
    losses = losses_out if losses_out is not None else torch.empty(2 * pairs_total, dtype=torch.float32, device="cuda")
    cfg = EsStepCfg(seed, epoch, pairs_total, rank, world, fitness_mode, fitness_clip,
                    UpdateCfg(lr, thresh, int(use_adaptive), adaptive_beta, adaptive_eps, int(train_pos)))
    coll, keep = (torch_collectives(rank, world, group) if world > 1 else (None, None))
    _l.check(model.lib.bnf4_model_es_step(model.h, C.byref(cfg), C.byref(coll) if coll is not None else None, losses.data_ptr(), _stream()))
    del keep
    return losses


def fitness_from_losses(losses: torch.Tensor) -> torch.Tensor:
    """f_p = -(loss+ - loss-)  (reference: src/train_efla_lm.cpp:5466)."""
    l2 = losses.view(-1, 2)
    return -(l2[:, 0] - l2[:, 1])


def shape_fitness(fitness: torch.Tensor, mode: int = 2, clip: float = 3.0) -> torch.Tensor:
    """Centered-rank shaping on the host (2 KB round trip), returned as a CUDA tensor."""
    from . import host
    w = fitness.detach().to("cpu", torch.float32).contiguous().numpy().copy()
    host.shape_pair_weights(w, mode, clip)
    return torch.from_numpy(w).to(fitness.device)

#!/usr/bin/env python
"""Regenerates the golden fixtures of tests/golden/ (run where a checkout of the reference project and the CUTLASS headers are present;
the fixtures themselves are committed and need neither).

  cutlass_codec.npz   e2m1 / ue4m3 conversions and the scale-factor layout, produced by gen_codec_golden.cpp from the
                      CUTLASS headers found in the image (the reference's own CUTLASS pin is unknown: the submodule is
                      empty and carries no commit id).
  ref_host.npz        outputs of the reference's own host functions (rng, noise hash, ternary init, fitness shaping,
                      token cross-entropy), called through oracle/_ref/libref_host.so, which #includes the reference's
                      src/train_efla_lm.cpp unmodified.
"""
import ctypes as C
import struct
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT / "oracle"))
import paths as oracle_paths  # noqa: E402

CUTLASS = oracle_paths.cutlass_include()


def gen_codec():
    with tempfile.TemporaryDirectory() as td:
        exe, out = Path(td) / "gen", Path(td) / "codec.bin"
        subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-w", f"-I{CUTLASS}", "-I/usr/local/cuda/include", "-o", str(exe),
                        str(HERE / "gen_codec_golden.cpp")], check=True)
        subprocess.run([str(exe), str(out)], check=True)
        raw = out.read_bytes()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, raw, pos)
        pos += struct.calcsize(fmt)
        return v

    (n,) = take("<I")
    e2m1_x = np.frombuffer(raw, np.float32, n, pos).copy(); pos += 4 * n
    e2m1_c = np.frombuffer(raw, np.uint8, n, pos).copy(); pos += n
    (n,) = take("<I")
    ue_x = np.frombuffer(raw, np.float32, n, pos).copy(); pos += 4 * n
    rec = np.frombuffer(raw, np.dtype([("b", "u1"), ("f", "<f4")]), n, pos).copy(); pos += 5 * n
    (ns,) = take("<I")
    d = {"e2m1_x": e2m1_x, "e2m1_code": e2m1_c, "ue4m3_x": ue_x, "ue4m3_byte": rec["b"].copy(), "ue4m3_value": rec["f"].copy()}
    shapes = []
    for i in range(ns):
        rows, K, nbytes = take("<iiQ")
        cnt = rows * (K // 16)
        off = np.frombuffer(raw, np.uint32, cnt, pos).copy(); pos += 4 * cnt
        (probe,) = take("<I")
        shapes.append((rows, K, nbytes, probe))
        d[f"sf_off_{rows}x{K}"] = off.reshape(rows, K // 16)
    d["sf_shapes"] = np.array(shapes, np.int64)
    np.savez_compressed(HERE / "cutlass_codec.npz", **d)
    print("cutlass_codec.npz", (HERE / "cutlass_codec.npz").stat().st_size, "bytes")


def gen_ref_host():
    so = ROOT / "oracle" / "_ref" / "libref_host.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "_ref/libref_host.so"], check=True)
    L = C.CDLL(str(so))
    u64 = C.c_uint64
    L.ref_mix.restype = u64; L.ref_mix.argtypes = [u64, u64]
    L.ref_splitmix64.restype = u64; L.ref_splitmix64.argtypes = [C.POINTER(u64)]
    L.ref_ternary_from_u64.argtypes = [u64]
    L.ref_noise_hash.argtypes = [u64, u64, C.c_int, C.c_int, C.c_int]
    L.ref_init_rand.restype = C.c_float; L.ref_init_rand.argtypes = [C.c_void_p, C.c_int, C.c_int, u64]
    L.ref_shape_pair_weights.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float]
    L.ref_cross_entropy_token.restype = C.c_float
    L.ref_cross_entropy_token.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int]
    L.ref_count_parameters.restype = u64
    rng = np.random.default_rng(2024)
    a = rng.integers(0, 2**63, 64, dtype=np.uint64) * 2 + rng.integers(0, 2, 64, dtype=np.uint64)
    b = rng.integers(0, 2**63, 64, dtype=np.uint64)
    a[:4] = [0, 1, 2**64 - 1, 0x1000]; b[:4] = [0, 2, 2**64 - 1, 0x111111]
    mix = np.array([L.ref_mix(int(x), int(y)) for x, y in zip(a, b)], np.uint64)
    sm_seed = np.array([0, 1, 0x1000, 0xABCDEF, 2**64 - 1], np.uint64)
    sm_out = np.zeros((len(sm_seed), 16), np.uint64)
    for i, s in enumerate(sm_seed):
        st = u64(int(s))
        for j in range(16):
            sm_out[i, j] = L.ref_splitmix64(C.byref(st))
    tern_in = rng.integers(0, 2**63, 512, dtype=np.uint64)
    tern = np.array([L.ref_ternary_from_u64(int(x)) for x in tern_in], np.int8)
    nh_seed = np.array([1, 0xDEADBEEF, 2**64 - 5], np.uint64)
    nh = np.zeros((len(nh_seed), 2, 4, 256), np.int8)  # [seed][use_clt][clt_k-1][idx]
    for i, s in enumerate(nh_seed):
        for uc in (0, 1):
            for k in range(1, 5):
                for idx in range(256):
                    nh[i, uc, k - 1, idx] = L.ref_noise_hash(int(s), idx, 1, uc, k)
    init = np.zeros((3, 4096), np.int8)
    init_scale = np.zeros(3, np.float32)
    for i, (seed, rows, cols) in enumerate([(0x1000, 8, 512), (0x3005, 4, 1024), (0x7000, 16, 256)]):
        init_scale[i] = L.ref_init_rand(init[i].ctypes.data, rows, cols, seed)
    fit = rng.standard_normal(1024).astype(np.float32)  # continuous draws: no ties, so std::sort's tie order is irrelevant
    shaped = np.zeros((3, 1024), np.float32)
    for mode in range(3):
        w = fit.copy()
        L.ref_shape_pair_weights(w.ctypes.data, len(w), mode, 3.0)
        shaped[mode] = w
    logits = (rng.standard_normal((8, 256)) * 3).astype(np.float32)
    bias = (rng.standard_normal(256) * 0.1).astype(np.float32)
    bnoise = rng.integers(-4, 5, 256).astype(np.float32)
    ys = rng.integers(0, 256, 8).astype(np.int32)
    ce = np.array([L.ref_cross_entropy_token(logits[i].ctypes.data, bias.ctypes.data, bnoise.ctypes.data, -0.125, 256, int(ys[i]))
                   for i in range(8)], np.float32)
    nparams = np.array([L.ref_count_parameters(256, 512, 4, 2, 128, 1)], np.uint64)
    fused_cols = np.array([L.ref_qkv_fused_cols_aligned(h) for h in (128, 512, 2048)], np.int32)
    # batch sampling of the reference's ByteDataset on a seeded synthetic corpus file (a hash of the windows is stored)
    sys.path.insert(0, str(ROOT))
    from bitnet_nvfp4_b200 import synth
    corpus = synth.zipf_corpus(1 << 16, 1.1, 123)
    L.ref_sample_batch_packed.argtypes = [C.c_char_p, C.c_int, C.c_int, u64, C.c_void_p, C.c_void_p]
    sb_tok = np.zeros((3, 32, 128), np.uint8)
    sb_tgt = np.zeros((3, 32, 128), np.uint8)
    sb_seed = np.array([123, 0x1234567, 2**64 - 3], np.uint64)
    with tempfile.TemporaryDirectory() as td:
        f = Path(td) / "corpus.bin"
        corpus.tofile(f)
        for i, sd in enumerate(sb_seed):
            assert L.ref_sample_batch_packed(str(f).encode(), 32, 128, int(sd), sb_tok[i].ctypes.data, sb_tgt[i].ctypes.data) == 0
    # per-epoch schedules: (start, end, schedule enum, t01) -> value
    L.ref_schedule_value.restype = C.c_float
    L.ref_schedule_value.argtypes = [C.c_float, C.c_float, C.c_int, C.c_float]
    sched_in = np.array([(st, en, sc, t) for (st, en) in [(0.8, 0.05), (0.008, -1.0), (3.0, 5.0), (0.0, 0.5), (0.5, 0.0)]
                         for sc in range(4) for t in (0.0, 1.0 / 3.0, 0.5, 0.9, 1.0, 1.5)], np.float32)
    sched_out = np.array([L.ref_schedule_value(float(a_), float(b_), int(c_), float(d_)) for a_, b_, c_, d_ in sched_in], np.float32)
    np.savez_compressed(HERE / "ref_host.npz", mix_a=a, mix_b=b, mix=mix, sm_seed=sm_seed, sm_out=sm_out, tern_in=tern_in, tern=tern,
                        nh_seed=nh_seed, nh=nh, init=init, init_scale=init_scale, fit=fit, shaped=shaped, ce_logits=logits, ce_bias=bias,
                        ce_noise=bnoise, ce_y=ys, ce=ce, nparams=nparams, fused_cols=fused_cols, sb_seed=sb_seed, sb_tok=sb_tok, sb_tgt=sb_tgt,
                        sched_in=sched_in, sched_out=sched_out)
    print("ref_host.npz", (HERE / "ref_host.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    gen_codec()
    gen_ref_host()

"""The reference's own host driver running on this library's kernels (GPU).

oracle/_ref/libref_host.so is the reference's src/train_efla_lm.cpp, #included unmodified, linked against libbnf4.so: every
bitnet_cuda:: / efla_lm_cuda:: entry point its DeviceWeights / CudaEflaLm classes call is one of this library's exports.
  * ref_eval_pair builds those classes with the reference's default flags (NVFP4 back-end, fused QKV, dense CLT noise as a
    second GEMM with beta = 1, int8 residual stream, token-serial loop) and calls evaluate_loss for anti = 0, +1, -1. The three
    losses are compared with the CPU oracle's token-major forward of the same model (one head of width hidden, dense
    perturbation: the reference's live configuration).
  * ref_train runs the reference's main() for two epochs of a tiny configuration on a synthetic corpus file.
The one thing the shim changes is the compute-capability query that gates the reference's NVFP4 path to sm_120.
"""
import ctypes as C
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as orc

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
SO = ROOT / "oracle" / "_ref" / "libref_host.so"


@pytest.fixture(scope="module")
def R():
    if not SO.exists():
        pytest.skip("oracle/_ref/libref_host.so not built (needs the reference tree at build time)")
    import torch
    assert torch.cuda.is_available()
    lib = C.CDLL(str(SO))
    if not hasattr(lib, "ref_eval_pair"):
        pytest.skip("oracle/_ref/libref_host.so predates ref_eval_pair")
    lib.ref_eval_pair.argtypes = [C.c_int] * 5 + [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_int, C.c_void_p, C.c_char_p, C.c_int]
    return lib


@pytest.mark.parametrize("hidden,layers,batch,seq", [(128, 2, 4, 16), (256, 1, 8, 8)])
def test_reference_model_classes_on_this_library(R, hidden, layers, batch, seq):
    from bitnet_nvfp4_b200 import population, synth
    cfg = population.Config(hidden=hidden, layers=layers, seq=seq, batch=batch, heads=1)
    w = synth.init_weights(cfg)
    tok, tgt = synth.sample_batch(synth.zipf_corpus(1 << 16), batch, seq, 123)
    out3 = np.zeros(3, np.float32)
    err = C.create_string_buffer(512)
    seed, epoch, pair = 1, 0, 2
    rc = R.ref_eval_pair(hidden, layers, cfg.mlp_mult, batch, seq, tok.ctypes.data, tgt.ctypes.data, seed, epoch, pair, cfg.sigma_shift,
                         out3.ctypes.data, err, 512)
    assert rc == 0, err.value.decode()
    # (an entry point outside the path, or a rejected argument, would have thrown inside the reference classes: rc != 0)
    ocfg = {k: getattr(cfg, k) for k in "vocab hidden layers mlp_mult seq batch heads rank sigma_shift use_clt clt_k method act_scale "
                                        "mlp_act_scale ln_scale residual_scale mlp_residual_scale eps".split()}
    ocfg["rank"] = 0  # dense noise: the reference driver's perturbation
    om = orc.OracleModel(ocfg, w)
    ps = orc.mix(seed, orc.mix(epoch, pair))
    for got, anti in zip(out3, (0, 1, -1)):
        ref = om.forward(tok, tgt, ps, anti, token_major=True)
        assert np.isfinite(got) and abs(got - ref) <= 1e-4 * abs(ref), (anti, got, ref)
    assert out3[1] != out3[2]  # the perturbation reached the model


def test_reference_driver_main_runs_on_this_library():
    """The reference's main(), argv as for its executable, two epochs; run in a child process because it owns stdout."""
    if not SO.exists():
        pytest.skip("oracle/_ref/libref_host.so not built")
    from bitnet_nvfp4_b200 import synth
    with tempfile.TemporaryDirectory() as td:
        corpus = Path(td) / "corpus.bin"
        synth.zipf_corpus(1 << 16).tofile(corpus)
        code = (
            "import ctypes as C, sys\n"
            f"L = C.CDLL({str(SO)!r})\n"
            f"argv = [b'train_efla_lm', b'--data', {str(corpus).encode()!r}, b'--epochs', b'2', b'--pop', b'8', b'--batch', b'4', b'--seq', b'16',\n"
            "        b'--hidden', b'128', b'--layers', b'2', b'--gpu_workers', b'1', b'--no_adaptive_pop', b'--device', b'0']\n"
            "arr = (C.c_char_p * len(argv))(*argv)\n"
            "sys.exit(L.ref_train(len(argv), arr))\n")
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=dict(os.environ))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "cutlass nvfp4 GEMM selected" in r.stderr, r.stderr[-2000:]       # the NVFP4 back-end, not the dp4a fallback
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("epoch ")]
    assert len(lines) == 2, r.stdout[-2000:]
    for ln in lines:
        f = ln.split()
        loss = float(f[f.index("train_loss") + 1])
        assert np.isfinite(loss) and 3.0 < loss < 8.0, ln

"""GPU parity against the reference's OWN device kernels.

oracle/_ref/libref_efla.so is the reference's src/efla_lm_kernels.cu compiled for sm_100a from where it lies (it needs no
CUTLASS). These tests run its EFLA step, cross-entropy, noise and ES-update kernels and this library's kernels on the
same inputs on the GPU. The reference's NVFP4 GEMM/quantiser file needs CUTLASS + sm_120 and cannot be built.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as orc

pytestmark = pytest.mark.gpu
SO = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_efla.so"


@pytest.fixture(scope="module")
def R():
    if not SO.exists():
        pytest.skip("oracle/_ref/libref_efla.so not built (needs the reference tree at build time)")
    import torch
    assert torch.cuda.is_available()
    lib = C.CDLL(str(SO))
    vp, ci, cf, u64 = C.c_void_p, C.c_int, C.c_float, C.c_uint64
    lib.ref_efla_step_half_qkv_fused.argtypes = [vp, vp, ci, cf, ci, ci, ci, cf, vp, vp, vp, vp, vp, vp, vp]
    lib.ref_cross_entropy_loss.argtypes = [vp, vp, vp, cf, vp, ci, ci, ci, vp, vp]
    lib.ref_fill_ternary_noise.argtypes = [vp, C.c_size_t, u64, ci, ci, vp]
    lib.ref_fill_pair_seeds.argtypes = [u64, u64, ci, vp, vp]
    lib.ref_compute_z_sumsq.argtypes = [vp, vp, u64, ci, ci, ci, ci, vp, vp, vp]
    lib.ref_update_inv_rms.argtypes = [vp, vp, ci, cf, cf, ci, vp, vp]
    lib.ref_update_shadow_ternary_device.argtypes = [vp, vp, vp, ci, vp, cf, cf, vp]
    return lib


@pytest.fixture(scope="module")
def H():
    from bitnet_nvfp4_b200 import host
    return host


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("hidden", [128, 512])
def test_efla_step_matches_reference_kernels(R, H, hidden):
    """Six reference kernels per step (prepare, zero, kS, diff, update, out) vs one kernel here; three steps with fp16 state."""
    import torch
    rng = np.random.default_rng(hidden)
    B = 6
    fc = (3 * hidden + 1 + 31) & ~31
    S_ref = torch.zeros((B, hidden, hidden), dtype=torch.float16, device="cuda")
    S_my = torch.zeros_like(S_ref)
    scratch = [torch.zeros(B * hidden, dtype=torch.float32, device="cuda") for _ in range(4)] + [torch.zeros(B, dtype=torch.float32, device="cuda")]
    for step in range(3):
        qkv = np.zeros((B, fc), np.float32)
        qkv[:, :3 * hidden] = (rng.standard_normal((B, 3 * hidden)) * 0.5).astype(np.float32)
        qkv[:, 3 * hidden] = rng.standard_normal(B).astype(np.float32)
        qd = dev(qkv)
        out_ref = torch.zeros((B, hidden), dtype=torch.float32, device="cuda")
        R.ref_efla_step_half_qkv_fused(S_ref.data_ptr(), qd.data_ptr(), fc, -2.0, hidden, B, 1, 1e-6, out_ref.data_ptr(),
                                       *[s.data_ptr() for s in scratch], stream())
        out_my = H.efla_step_half_qkv_fused(S_my, qd, fc, -2.0, hidden, B, 1, 1e-6)
        torch.cuda.synchronize()
        a, b = out_my.cpu().numpy(), out_ref.cpu().numpy()
        # the reference accumulates k.S and S.q with unordered float atomics over tiles; same values up to summation order
        assert np.abs(a - b).max() <= 2e-4 * max(1e-6, np.abs(b).max())
    sa = S_my.cpu().numpy().view(np.uint16).astype(np.int32)
    sb = S_ref.cpu().numpy().view(np.uint16).astype(np.int32)
    assert (np.abs(sa - sb) > 1).mean() <= 1e-4 and (sa != sb).mean() <= 2e-2


def test_cross_entropy_matches_reference_kernel(R, H):
    import torch
    rng = np.random.default_rng(2)
    B, V, T = 32, 256, 8
    logits = dev((rng.standard_normal((B, V)) * 3).astype(np.float32))
    bias = dev((rng.standard_normal(V) * 0.1).astype(np.float32))
    noise = dev(orc.fill_noise(V, 7).astype(np.float32))
    targets = dev(rng.integers(0, 256, (B, T)).astype(np.uint8)).view(-1)
    acc_ref = torch.zeros(1, dtype=torch.float32, device="cuda")
    acc_my = torch.zeros(1, dtype=torch.float32, device="cuda")
    R.ref_cross_entropy_loss(logits.data_ptr(), bias.data_ptr(), noise.data_ptr(), 0.125, targets[3:].data_ptr(), T, V, B, acc_ref.data_ptr(),
                             stream())
    H.cross_entropy_loss(logits, bias, noise, 0.125, targets[3:], T, acc_my)
    assert abs(acc_my.item() - acc_ref.item()) <= 2e-6 * abs(acc_ref.item())


def test_noise_and_seeds_match_reference_kernels(R, H):
    import torch
    n = 70001
    for use_clt in (0, 1):
        ref = torch.zeros(n, dtype=torch.int8, device="cuda")
        R.ref_fill_ternary_noise(ref.data_ptr(), n, 0xFEEDFACE, use_clt, 4, stream())
        assert torch.equal(ref, H.fill_ternary_noise(n, 0xFEEDFACE, bool(use_clt), 4))
    seeds = torch.zeros(1024, dtype=torch.int64, device="cuda")
    R.ref_fill_pair_seeds(1, 9, 1024, seeds.data_ptr(), stream())
    assert torch.equal(seeds, H.fill_pair_seeds(1, 9, 1024))


def test_es_update_matches_reference_kernels(R, H):
    """Z is bit-identical; the sum of squares differs only by the reference's unordered atomics; the resulting ternary weights
    agree except where a shadow weight sits within an ulp of the gate or of a rounding boundary (none expected at this size)."""
    import torch
    rng = np.random.default_rng(4)
    n, pairs = 50000, 64
    pw = dev(orc.shape_pair_weights(rng.standard_normal(pairs).astype(np.float32)))
    seeds = H.fill_pair_seeds(1, 0, pairs)
    w0 = orc.init_rand_ternary(n, 0x2000)
    Z_ref = torch.zeros(n, dtype=torch.float32, device="cuda")
    ss_ref = torch.zeros(1, dtype=torch.float32, device="cuda")
    R.ref_compute_z_sumsq(pw.data_ptr(), seeds.data_ptr(), 0x222222, pairs, n, 1, 4, Z_ref.data_ptr(), ss_ref.data_ptr(), stream())
    Z_my, ss_my = H.compute_z_sumsq(pw, seeds, 0x222222, n)
    assert torch.equal(Z_ref, Z_my)
    assert abs(ss_ref.item() - ss_my.item()) <= 1e-5 * ss_my.item()
    ema_ref = torch.zeros(1, dtype=torch.float32, device="cuda")
    ema_my = torch.zeros(1, dtype=torch.float32, device="cuda")
    inv_ref = torch.zeros(1, dtype=torch.float32, device="cuda")
    R.ref_update_inv_rms(ss_ref.data_ptr(), ema_ref.data_ptr(), 1, 0.95, 1e-3, n, inv_ref.data_ptr(), stream())
    inv_my = H.update_inv_rms(ss_my, ema_my, True, 0.95, 1e-3, n)
    assert abs(inv_ref.item() - inv_my.item()) <= 1e-5 * inv_my.item()  # rsqrtf (reference) vs 1/sqrt (here), different sum order
    w_ref, w_my = dev(w0), dev(w0)
    s_ref, s_my = dev(w0.astype(np.float32)), dev(w0.astype(np.float32))
    thresh = float(np.float32(0.008) * np.sqrt(np.float32(pairs)))
    R.ref_update_shadow_ternary_device(w_ref.data_ptr(), s_ref.data_ptr(), Z_ref.data_ptr(), n, inv_ref.data_ptr(), 0.8, thresh, stream())
    H.update_shadow_ternary_device(w_my, s_my, Z_my, inv_my, 0.8, thresh)
    torch.cuda.synchronize()
    assert (w_ref != w_my).sum().item() <= 2
    assert (w_my.cpu().numpy() != w0).any()

"""BASELINE configuration 0, as written: a single perturbed NVFP4 GEMM, pop = 4 members, M = 4096 (batch 32 x seq 128),
K = N = 512, rank-1 perturbation, sigma = 2^-3, fp32 output.

  * activations X_i ~ 0.8 N(0,1) in fp32 from the oracle's counter-RNG Gaussian map keyed (seed 1, member i);
  * weights: fp32 latents ~ 0.02 N(0,1) keyed (seed 1, tag W), ternarised by |w| > 0.008;
  * a_i, b_i in R^512 keyed (seed 1, i, tag A / B): sqrt(3/8) x the reference's CLT-4 integer noise (variance 8/3), which is
    the reference's own stand-in for a standard normal ("CLT/approx-Gaussian perturbations", src/train_efla_lm.cpp:204);
  * both quantiser forms: fp32 -> int8 -> NVFP4 (the reference's live path, activation_quantize_nvfp4 mode 0) and
    fp32 -> NVFP4 directly (bnf4_nvfp4_quantize_f32).
Checks: int8 values, e2m1 codes and ue4m3 scale bytes of X and W bit-exact against the oracle; Y_i within 1e-3 of
max |Y_i| (fp32 accumulation order); the rank-1 term is an exact integer product.
"""
import numpy as np
import pytest

import oracle_lib as orc

pytestmark = pytest.mark.gpu
TAG_W, TAG_X, TAG_A, TAG_B = 0x57, 0x58, 0xA11CE, 0xB0B
POP, M, K, N, SIGMA = 4, 4096, 512, 512, 0.125


@pytest.fixture(scope="module")
def H():
    import torch
    from bitnet_nvfp4_b200 import host
    assert torch.cuda.is_available()
    return host


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def inputs():
    lat = orc.gaussian_f32(1, TAG_W, N * K, 0.02).reshape(N, K)
    w = (np.sign(lat) * (np.abs(lat) > 0.008)).astype(np.int8)
    xs = [orc.gaussian_f32(1, orc.mix(TAG_X, i), M * K, 0.8).reshape(M, K) for i in range(POP)]
    a = [orc.fill_noise(N, orc.mix(orc.mix(1, i), TAG_A)) for i in range(POP)]
    b = [orc.fill_noise(K, orc.mix(orc.mix(1, i), TAG_B)) for i in range(POP)]
    return w, xs, a, b


def test_config0_reference_quantiser_path(H):
    import torch
    w, xs, a, b = inputs()
    out_scale = float(np.float32(1.0) / np.sqrt(np.float32(K)))
    cr = H.c_rank(1)
    wc, wsf = H.nvfp4_quantize_b(dev(w))
    rwc, rwsf = orc.quantize_rowmajor(w)
    assert np.array_equal(wc.cpu().numpy(), rwc) and np.array_equal(wsf.cpu().numpy(), rwsf)
    for i in range(POP):
        q, codes, sf = H.activation_quantize_nvfp4(dev(xs[i]), K, 0)
        rq, rc, rs = orc.activation_quant(xs[i], K, 0, 1.0)
        assert np.array_equal(q.cpu().numpy(), rq) and np.array_equal(codes.cpu().numpy(), rc) and np.array_equal(sf.cpu().numpy(), rs)
        t = H.lora_compute_t(q, dev(b[i].reshape(K, 1)), 1)
        rt = orc.lora_compute_t(rq, b[i].reshape(K, 1), 1)
        assert np.array_equal(t.cpu().numpy(), rt)
        d = torch.empty((M, N), dtype=torch.float32, device="cuda")
        lscale = float(np.float32(SIGMA) * np.float32(out_scale)) * cr
        H.gemm_nvfp4_ex(a=codes, b=wc, sfa=sf, sfb=wsf, m=M, n=N, k=K, alpha=out_scale, d=d, ldd=N, epilogue=H.EPI_F32, rank=1,
                        rows_per_member=M, lora_t=t, t_stride=1, lora_A=dev(a[i].reshape(1, N, 1)), lora_A_pair_stride=N, lora_scale=lscale)
        assert H.device_error() == 0
        ref = orc.gemm_nvfp4(rc, rwc, rs, rwsf, M, N, K, out_scale)
        base = ref.copy()
        orc.lora_add(rt, a[i].reshape(N, 1), N, lscale, ref)
        got = d.cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
        assert np.abs(ref - base).max() > 1e-2 * np.abs(ref).max()   # the perturbation is a visible part of Y_i


def test_config0_direct_fp32_quantiser(H):
    w, xs, _, _ = inputs()
    out_scale = float(np.float32(1.0) / np.sqrt(np.float32(K)))
    wc, wsf = H.nvfp4_quantize_b(dev(w))
    rwc, rwsf = orc.quantize_rowmajor(w)
    for i in range(2):
        codes, sf = H.nvfp4_quantize_f32(dev(xs[i]))
        rc, rs = orc.quantize_direct_f32(xs[i])
        assert np.array_equal(codes.cpu().numpy(), rc) and np.array_equal(sf.cpu().numpy(), rs)
        d = H.gemm_ternary_f_nvfp4(codes, wc, sf, wsf, M, N, K, out_scale)
        ref = orc.gemm_nvfp4(rc, rwc, rs, rwsf, M, N, K, out_scale)
        assert np.abs(d.cpu().numpy() - ref).max() <= 1e-3 * np.abs(ref).max()
    # edge cases of the direct form: zero blocks, a block whose scale underflows ue4m3, saturation, short input rows
    x = np.zeros((5, 64), np.float32)
    x[1, :16] = 1e-5
    x[2, :] = np.linspace(-3000, 3000, 64)
    x[3, 16:32] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
    x[4, :] = np.random.default_rng(0).standard_normal(64)
    codes, sf = H.nvfp4_quantize_f32(dev(x))
    rc, rs = orc.quantize_direct_f32(x)
    assert np.array_equal(codes.cpu().numpy(), rc) and np.array_equal(sf.cpu().numpy(), rs)
    codes, sf = H.nvfp4_quantize_f32(dev(x[:, :40]), k_out=64)
    rc, rs = orc.quantize_direct_f32(np.ascontiguousarray(x[:, :40]), 64)
    assert np.array_equal(codes.cpu().numpy(), rc) and np.array_equal(sf.cpu().numpy(), rs)

"""GPU parity of the tcgen05 block-scaled FP4 GEMM (C ABI of libbnf4) against the CPU oracle.

Tolerance: |D - D_ref| <= 1e-3 * max|D_ref| per matrix (fp32 accumulation order differs between the tensor
core and the oracle). The rank-r term is an exact integer product, so it does not loosen the bound.
"""
import numpy as np
import pytest

import oracle_lib as orc

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.fixture(scope="module")
def H():
    import torch
    from bitnet_nvfp4_b200 import host
    assert torch.cuda.is_available()
    return host


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_operands(rng, m, n, k, act_std=40.0):
    x = np.clip(np.rint(rng.standard_normal((m, k)) * act_std), -127, 127).astype(np.int8)
    w = rng.integers(-1, 2, (n, k)).astype(np.int8)
    a, sfa = orc.quantize_rowmajor(x)
    b, sfb = orc.quantize_rowmajor(w)
    return x, w, a, sfa, b, sfb


def rel_err(d, ref):
    return float(np.abs(d - ref).max() / max(1e-30, np.abs(ref).max()))


@pytest.mark.parametrize("tma_store", [1, 0])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 128, 256), (128, 128, 512), (32, 512, 512), (1, 256, 512),
                                   (31, 1024, 512), (129, 512, 1024), (4096, 512, 512), (256, 1568, 512), (200, 72, 128),
                                   (384, 256, 1536)])
def test_gemm_f32(H, m, n, k, tma_store):
    from bitnet_nvfp4_b200 import lib
    rng = np.random.default_rng(m * 31 + n * 7 + k)
    _, _, a, sfa, b, sfb = make_operands(rng, m, n, k)
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(k)))
    lib.check(lib.load().bnf4_set_option(b"gemm_tma_store", tma_store))
    try:
        d = H.gemm_ternary_f_nvfp4(dev(a), dev(b), dev(sfa), dev(sfb), m, n, k, alpha)
        assert H.device_error() == 0
    finally:
        lib.load().bnf4_set_option(b"gemm_tma_store", 1)
    ref = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, alpha)
    assert rel_err(d.cpu().numpy(), ref) <= TOL


def test_gemm_beta_accumulate(H):
    """The reference's dense-noise form: D = alpha2 * A*E^T + 1.0 * D."""
    rng = np.random.default_rng(77)
    m, n, k = 160, 384, 512
    _, _, a, sfa, b, sfb = make_operands(rng, m, n, k)
    e = rng.integers(-4, 5, (n, k)).astype(np.int8)
    eb, esf = orc.quantize_rowmajor(e)
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(k)))
    d = H.gemm_ternary_f_nvfp4(dev(a), dev(b), dev(sfa), dev(sfb), m, n, k, alpha)
    d = H.gemm_ternary_f_nvfp4(dev(a), dev(eb), dev(sfa), dev(esf), m, n, k, alpha * 0.125, 1.0, d, d)
    assert H.device_error() == 0
    ref = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, alpha)
    ref = orc.gemm_nvfp4(a, eb, sfa, esf, m, n, k, alpha * 0.125, 1.0, ref)
    assert rel_err(d.cpu().numpy(), ref) <= TOL


def test_gemm_gelu_i8(H):
    rng = np.random.default_rng(78)
    m, n, k = 96, 1024, 512
    _, _, a, sfa, b, sfb = make_operands(rng, m, n, k)
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(k)))
    c = (rng.standard_normal((m, n)) * 3).astype(np.float32)
    d8 = H.gemm_ternary_f_nvfp4_gelu_i8(dev(a), dev(b), dev(sfa), dev(sfb), m, n, k, alpha, 1.0, dev(c), 1.0)
    assert H.device_error() == 0
    ref = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, alpha, 1.0, c, gelu_i8=True, act_scale=1.0)
    diff = np.abs(d8.cpu().numpy().astype(int) - ref.astype(int))
    # int8 after a float GEMM: one step on elements that sit on a rounding boundary
    assert diff.max() <= 1 and (diff != 0).mean() <= 5e-3


@pytest.mark.parametrize("rank,R", [(1, 128), (4, 64), (2, 4096)])
def test_gemm_lowrank_population(H, rank, R):
    """Per-member rank-r perturbation fused in the epilogue; members = row / R, pair = member / 2, sign by parity."""
    import torch
    rng = np.random.default_rng(79 + rank)
    pairs = 2 if R < 4096 else 1
    m, n, k = 2 * pairs * R, 512, 512
    x, w, a, sfa, b, sfb = make_operands(rng, m, n, k)
    A = rng.integers(-4, 5, (pairs, n, rank)).astype(np.int8)
    Bm = rng.integers(-4, 5, (pairs, k, rank)).astype(np.int8)
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(k)))
    sigma = 0.125
    cr = H.c_rank(rank)
    lscale = float(np.float32(np.float32(sigma) * np.float32(alpha)) * np.float32(cr))
    t = np.concatenate([orc.lora_compute_t(x[mm * R:(mm + 1) * R], Bm[mm // 2], rank) for mm in range(2 * pairs)])
    d = torch.empty((m, n), dtype=torch.float32, device="cuda")
    H.gemm_nvfp4_ex(a=dev(a), b=dev(b), sfa=dev(sfa), sfb=dev(sfb), m=m, n=n, k=k, alpha=alpha, d=d, ldd=n, epilogue=H.EPI_F32,
                    rank=rank, rows_per_member=R, lora_t=dev(t), t_stride=rank, lora_A=dev(A), lora_A_pair_stride=n * rank,
                    lora_scale=lscale)
    assert H.device_error() == 0
    ref = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, alpha)
    for mm in range(2 * pairs):
        sl = slice(mm * R, (mm + 1) * R)
        sgn = 1.0 if mm % 2 == 0 else -1.0
        blk = np.ascontiguousarray(ref[sl])
        orc.lora_add(np.ascontiguousarray(t[sl]), A[mm // 2], n, sgn * lscale, blk)
        ref[sl] = blk
    assert rel_err(d.cpu().numpy(), ref) <= TOL


def test_gemm_qkv_groups_lowrank(H):
    """Stacked QKV(+beta) projection: N = 3H+1 with ldd = padded columns; group g reads t[g*rank ..]."""
    import torch
    rng = np.random.default_rng(90)
    hid, R, rank = 128, 64, 2
    m, n, k = 2 * R, 3 * hid + 1, hid
    ldd = (n + 31) & ~31
    x = np.clip(np.rint(rng.standard_normal((m, k)) * 40), -127, 127).astype(np.int8)
    a, sfa = orc.quantize_rowmajor(x)
    wq, wk, wv = (rng.integers(-1, 2, (hid, hid)).astype(np.int8) for _ in range(3))
    wb = rng.integers(-1, 2, (hid,)).astype(np.int8)
    s = float(np.float32(1.0) / np.sqrt(np.float32(hid)))
    b, sfb = orc.quantize_wqkv_fused(wq, wk, wv, wb, hid, s)
    bpad = np.zeros(ldd * hid // 2, np.uint8)
    bpad[: n * hid // 2] = b[: n * hid // 2]
    sfpad = np.zeros(orc.sf_bytes(ldd, hid), np.uint8)
    sfpad[: len(sfb)] = sfb
    A = rng.integers(-4, 5, (1, n, rank)).astype(np.int8)
    Bg = rng.integers(-4, 5, (4, hid, rank)).astype(np.int8)
    t = np.concatenate([orc.lora_compute_t(x, Bg[g], rank) for g in range(4)], axis=1)  # [m][4*rank]
    sigma = 0.125
    lscale = float(np.float32(np.float32(sigma) * np.float32(s)) * np.float32(H.c_rank(rank)))
    d = torch.zeros((m, ldd), dtype=torch.float32, device="cuda")
    H.gemm_nvfp4_ex(a=dev(a), b=dev(bpad), sfa=dev(sfa), sfb=dev(sfpad), m=m, n=n, k=k, alpha=1.0, d=d, ldd=ldd,
                    epilogue=H.EPI_F32, rank=rank, rows_per_member=R, lora_t=dev(t), t_stride=4 * rank, lora_A=dev(A),
                    lora_A_pair_stride=n * rank, lora_scale=lscale, group_cols=hid)
    assert H.device_error() == 0
    ref = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, 1.0, ldd=ldd)
    grows = [hid, hid, hid, 1]
    for mm in range(2):
        sgn = 1.0 if mm == 0 else -1.0
        for g in range(4):
            blk = np.ascontiguousarray(ref[mm * R:(mm + 1) * R, g * hid:g * hid + grows[g]])
            orc.lora_add(np.ascontiguousarray(t[mm * R:(mm + 1) * R, g * rank:(g + 1) * rank]),
                         np.ascontiguousarray(A[0, g * hid:g * hid + grows[g]]), grows[g], sgn * lscale, blk)
            ref[mm * R:(mm + 1) * R, g * hid:g * hid + grows[g]] = blk
    got = d.cpu().numpy()
    assert rel_err(got[:, :n], ref[:, :n]) <= TOL
    assert np.all(got[:, n:] == 0)  # padded columns are never written


def test_gemm_gelu_fp4_epilogue(H):
    """ff1 form: GELU -> int8 -> e2m1 codes + scales written by the epilogue, plus the next GEMM's projections."""
    import torch
    rng = np.random.default_rng(91)
    R, rank = 128, 2
    m, n, k = 2 * R, 1024, 512
    x, w, a, sfa, b, sfb = make_operands(rng, m, n, k)
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(k)))
    tvec = rng.integers(-4, 5, (1, rank, n)).astype(np.int8)
    d8 = torch.zeros((m, n), dtype=torch.int8, device="cuda")
    codes = torch.zeros(m * n // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(m, n), dtype=torch.uint8, device="cuda")
    nt = torch.zeros((m, rank), dtype=torch.int32, device="cuda")
    H.gemm_nvfp4_ex(a=dev(a), b=dev(b), sfa=dev(sfa), sfb=dev(sfb), m=m, n=n, k=k, alpha=alpha, epilogue=H.EPI_GELU_FP4,
                    act_scale=1.0, d_i8=d8, ld_i8=n, d_codes=codes, d_sf=sf, rows_per_member=R, next_tvec=dev(tvec),
                    next_tvec_pair_stride=rank * n, next_nvec=rank, next_t=nt)
    assert H.device_error() == 0
    ref = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, alpha, gelu_i8=True, act_scale=1.0)
    got = d8.cpu().numpy()
    diff = np.abs(got.astype(int) - ref.astype(int))
    assert diff.max() <= 1 and (diff != 0).mean() <= 5e-3
    rc, rs = orc.quantize_rowmajor(got)  # exact given the device's own int8 values
    assert np.array_equal(codes.cpu().numpy(), rc) and np.array_equal(sf.cpu().numpy(), rs)
    assert np.array_equal(nt.cpu().numpy(), got.astype(np.int32) @ tvec[0].astype(np.int32).T)


@pytest.mark.parametrize("m,n,k,rank", [(512, 512, 1024, 1), (300, 512, 512, 0), (200, 72, 128, 2), (129, 200, 256, 0)])
def test_gemm_residual_add_epilogue(H, m, n, k, rank):
    """BNF4_EPI_ADD_I8: the GEMM adds its product into the int8 residual stream, resid = clip8(resid + rint(v * add_scale)).

    Bit-exact against the oracle's add step applied to the same kernel's fp32 output (same accumulators, same epilogue
    arithmetic up to the store); against the oracle's own GEMM an int8 may differ by one step where v * add_scale falls on a
    rounding boundary. Ragged sizes take the per-byte path."""
    import torch
    rng = np.random.default_rng(5 * m + n + k + rank)
    x, w, a, sfa, b, sfb = make_operands(rng, m, n, k)
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(k)))
    add_scale = 0.37
    R = 64 if m % 128 == 0 else m
    kw = dict(a=dev(a), b=dev(b), sfa=dev(sfa), sfb=dev(sfb), m=m, n=n, k=k, alpha=alpha)
    if rank:
        pairs = (m // R + 1) // 2
        A = rng.integers(-4, 5, (pairs, n, rank)).astype(np.int8)
        t = rng.integers(-3000, 3000, (m, rank)).astype(np.int32)
        lscale = float(np.float32(0.125) * np.float32(alpha) * np.float32(H.c_rank(rank)))
        kw.update(rank=rank, rows_per_member=R, lora_t=dev(t), t_stride=rank, lora_A=dev(A), lora_A_pair_stride=n * rank, lora_scale=lscale)
    resid0 = rng.integers(-127, 128, (m, n)).astype(np.int8)
    d = torch.empty((m, n), dtype=torch.float32, device="cuda")
    H.gemm_nvfp4_ex(d=d, ldd=n, epilogue=H.EPI_F32, **kw)
    resid = dev(resid0)
    H.gemm_nvfp4_ex(epilogue=H.EPI_ADD_I8, resid=resid, ld_resid=n, add_scale=add_scale, **kw)
    assert H.device_error() == 0
    got = resid.cpu().numpy()
    want = np.clip(resid0.astype(np.int32) + np.rint(d.cpu().numpy() * np.float32(add_scale)).astype(np.int32), -127, 127).astype(np.int8)
    assert np.array_equal(got, want)
    ref = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, alpha)
    if rank:
        for mm in range(m // R):
            blk = np.ascontiguousarray(ref[mm * R:(mm + 1) * R])
            orc.lora_add(np.ascontiguousarray(t[mm * R:(mm + 1) * R]), A[mm // 2], n, (1.0 if mm % 2 == 0 else -1.0) * lscale, blk)
            ref[mm * R:(mm + 1) * R] = blk
    want2 = np.clip(resid0.astype(np.int32) + np.rint(ref * np.float32(add_scale)).astype(np.int32), -127, 127)
    diff = np.abs(got.astype(np.int32) - want2)
    assert diff.max() <= 1 and (diff != 0).mean() <= 5e-3


def test_gemm_fp16_epilogue_rounds_the_fp32_result(H):
    """BNF4_EPI_F16 (the fused q | k | v | beta projection feeding the chunked scan): the leading columns are the fp32 epilogue's
    values rounded once to IEEE half (bit for bit: same accumulators), the remaining columns stay fp32."""
    import torch
    rng = np.random.default_rng(77)
    hid, R, pairs, rank = 128, 64, 2, 2
    m, n, k = 2 * pairs * R, 3 * hid + 1, hid
    x, w, a, sfa, b, sfb = make_operands(rng, m, n, k)
    A = rng.integers(-4, 5, (pairs, n, rank)).astype(np.int8)
    t = rng.integers(-500, 500, (m, 4 * rank)).astype(np.int32)
    kw = dict(a=dev(a), b=dev(b), sfa=dev(sfa), sfb=dev(sfb), m=m, n=n, k=k, alpha=0.05, rank=rank, rows_per_member=R, lora_t=dev(t),
              t_stride=4 * rank, lora_A=dev(A), lora_A_pair_stride=n * rank, lora_scale=0.003, group_cols=hid)
    ld = (n + 31) & ~31
    d32 = torch.zeros((m, ld), dtype=torch.float32, device="cuda")
    H.gemm_nvfp4_ex(**kw, d=d32, ldd=ld, epilogue=H.EPI_F32)
    d16 = torch.zeros((m, 3 * hid), dtype=torch.float16, device="cuda")
    tail = torch.zeros((m, 1), dtype=torch.float32, device="cuda")
    H.gemm_nvfp4_ex(**kw, d_f16=d16, ld_f16=3 * hid, n_f16=3 * hid, d=tail, ldd=1, epilogue=H.EPI_F16)
    assert H.device_error() == 0
    assert torch.equal(d16, d32[:, :3 * hid].to(torch.float16))
    assert torch.equal(tail[:, 0], d32[:, 3 * hid])


def test_gemm_rejects_bad_arguments(H):
    import torch
    from bitnet_nvfp4_b200 import lib
    z = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(lib.Bnf4Error):
        H.gemm_ternary_f_nvfp4(z, z, z, z, 16, 16, 48, 1.0)  # k not a multiple of 64
    with pytest.raises(lib.Bnf4Error):
        H.gemm_ternary_f_nvfp4(z, z, z, z, 16, 16, 64, 1.0, 1.0, None)  # beta without C


def test_gemm_kernel_instances_agree(H):
    """The kernel instance for the batched driver's calls (rank 1, m a multiple of 128, tiles inside one member) against the general
    instance: the same call with its last row dropped (m = 511) runs the general instance, and the 511 common rows of every epilogue's
    output must be bit-identical."""
    import torch
    rng = np.random.default_rng(1234)
    R, members, n, k = 128, 4, 512, 512
    m = members * R
    x, w, a, sfa, b, sfb = make_operands(rng, m, n, k)
    A = torch.from_numpy(rng.integers(-4, 5, (members // 2, n, 1)).astype(np.int8)).cuda()
    t = torch.from_numpy(rng.integers(-1000, 1000, (m, 1)).astype(np.int32)).cuda()
    tv = torch.from_numpy(rng.integers(-4, 5, (members // 2, 1, n)).astype(np.int8)).cuda()
    resid0 = torch.from_numpy(rng.integers(-100, 101, (m, n)).astype(np.int8)).cuda()
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(k)))
    base = dict(a=dev(a), b=dev(b), sfa=dev(sfa), sfb=dev(sfb), n=n, k=k, alpha=alpha, rank=1, rows_per_member=R, lora_t=t, t_stride=1,
                lora_A=A, lora_A_pair_stride=n, lora_scale=0.01)
    out = {}
    for rows in (m, m - 1):
        d = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        H.gemm_nvfp4_ex(**base, m=rows, d=d, ldd=n, epilogue=H.EPI_F32)
        d16 = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        H.gemm_nvfp4_ex(**base, m=rows, d_f16=d16, ld_f16=n, n_f16=n, epilogue=H.EPI_F16)
        res = resid0.clone()
        H.gemm_nvfp4_ex(**base, m=rows, resid=res, ld_resid=n, add_scale=0.0625, epilogue=H.EPI_ADD_I8)
        codes = torch.zeros(m * n // 2, dtype=torch.uint8, device="cuda")
        sf = torch.zeros(H.sf_bytes(m, n), dtype=torch.uint8, device="cuda")
        nt = torch.zeros((m, 1), dtype=torch.int32, device="cuda")
        H.gemm_nvfp4_ex(**base, m=rows, epilogue=H.EPI_GELU_FP4, act_scale=4.0, d_codes=codes, d_sf=sf, next_tvec=tv,
                        next_tvec_pair_stride=n, next_nvec=1, next_t=nt)
        assert H.device_error() == 0
        out[rows] = (d, d16, res, codes.view(m, n // 2), nt)
    keep = m - 1
    for full, part in zip(out[m], out[m - 1]):
        assert torch.equal(full[:keep], part[:keep])
    assert out[m][0][keep].abs().sum() > 0 and out[m - 1][0][keep].abs().sum() == 0   # the dropped row really was not computed

"""GPU parity of the NVFP4 quantisers (C ABI of libbnf4) against the CPU oracle.

Integer stages (int8 copy, e2m1 codes, ue4m3 scale bytes, rank-r projections) must match bit-exactly.
Front-ends that pass through tanhf before rounding may differ by one int8 step on a vanishing fraction of
elements (device vs host libm); the bound is stated in each test.
"""
import numpy as np
import pytest

import oracle_lib as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import torch
    from bitnet_nvfp4_b200 import host
    assert torch.cuda.is_available()
    return host


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def same(t, ref):
    return np.array_equal(t.cpu().numpy().reshape(-1), np.asarray(ref).reshape(-1))


@pytest.mark.parametrize("rows,k", [(1, 16), (31, 512), (32, 512), (129, 1024), (512, 2048), (300, 4096), (4096, 512)])
def test_quantize_a_bit_exact(H, rows, k):
    rng = np.random.default_rng(rows * 7 + k)
    x = rng.integers(-127, 128, (rows, k)).astype(np.int8)
    x[rng.random((rows, k)) < 0.3] = 0
    if rows > 2:
        x[1, :] = 0           # all-zero row -> scale 1.0, codes 0
        x[2, : k // 2] = 1    # ternary-like blocks
    codes, sf = H.nvfp4_quantize_a(dev(x))
    rc, rs = orc.quantize_rowmajor(x)
    assert same(codes, rc)
    assert same(sf, rs)


def every_block_maximum_and_value():
    """16-element blocks covering every (block maximum, value) combination: the first element is +-amax, the other fifteen
    walk through all values of magnitude <= amax (exact ties of value / scale and negative values that quantise to zero
    included)."""
    blocks = []
    for amax in range(0, 128):
        vals = np.arange(-amax, amax + 1, dtype=np.int64)
        for lead in (amax, -amax):
            for o in range(0, len(vals), 15):
                chunk = vals[o:o + 15]
                blk = np.zeros(16, dtype=np.int64)
                blk[0] = lead
                blk[1:1 + len(chunk)] = chunk
                blocks.append(blk)
    return blocks


def test_quantize_a_every_block_maximum_and_value(H):
    blocks = every_block_maximum_and_value()
    k = 512
    while len(blocks) % (k // 16):
        blocks.append(np.zeros(16, dtype=np.int64))
    x = np.stack(blocks).reshape(-1, k).astype(np.int8)
    codes, sf = H.nvfp4_quantize_a(dev(x))
    rc, rs = orc.quantize_rowmajor(x)
    assert same(codes, rc)
    assert same(sf, rs)


def test_absmean_rows_every_block_maximum_and_value(H):
    """The same blocks through the float-domain quantiser of int8 rows (codes from the conversion instruction applied to
    value x 1 / scale): one block per otherwise empty row of 2048 columns, so that the abs-mean clamps to 1 and the values pass
    the normalisation unchanged; the block sits at a different position in every row."""
    import torch
    blocks = every_block_maximum_and_value()
    hid = 2048
    rows = len(blocks)
    x = np.zeros((rows, hid), dtype=np.int8)
    for i, blk in enumerate(blocks):
        pos = (i * 7) % (hid // 16)
        x[i, 16 * pos:16 * pos + 16] = blk
    assert np.abs(x.astype(np.int32)).sum(axis=1).max() < hid
    yq = torch.zeros((rows, hid), dtype=torch.int8, device="cuda")
    codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
    H.rowquant(H.FE_ABSMEAN, rows=rows, cols_in=hid, cols_out=hid, in_i8=dev(x), ld_in=hid, norm_scale=1.0,
               out_q=yq, ld_q=hid, out_codes=codes, out_sf=sf)
    rq, rc, rs = orc.absmean_norm_q(x.copy(), None, 0.0, 1.0)
    assert same(yq, x)
    assert same(yq, rq) and same(codes, rc) and same(sf, rs)


def test_quantize_b_ternary_and_kin_smaller(H):
    rng = np.random.default_rng(5)
    w = rng.integers(-1, 2, (1568, 512)).astype(np.int8)
    codes, sf = H.nvfp4_quantize_b(dev(w))
    rc, rs = orc.quantize_rowmajor(w)
    assert same(codes, rc) and same(sf, rs)
    # k_in < k_out: the tail is zero-filled
    x = rng.integers(-127, 128, (40, 96)).astype(np.int8)
    codes, sf = H.nvfp4_quantize_a(dev(x), k_out=128)
    rc, rs = orc.quantize_rowmajor(x, 128)
    assert same(codes, rc) and same(sf, rs)


@pytest.mark.parametrize("hidden", [128, 512])
def test_quantize_wqkv_fused(H, hidden):
    rng = np.random.default_rng(hidden)
    wq, wk, wv = (rng.integers(-1, 2, (hidden, hidden)).astype(np.int8) for _ in range(3))
    wb = rng.integers(-1, 2, (hidden,)).astype(np.int8)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hidden)))
    rows_total = (3 * hidden + 1 + 31) & ~31
    codes, sf = H.nvfp4_quantize_wqkv_fused(dev(wq), dev(wk), dev(wv), dev(wb), hidden, rows_total, scale)
    rc, rs = orc.quantize_wqkv_fused(wq, wk, wv, wb, hidden, scale)
    n = (3 * hidden + 1) * hidden // 2
    assert same(codes[:n], rc[:n])
    assert same(sf, rs)
    # the folded scale of a ternary block is 2^-7 for hidden=512 and the codes saturate at +-6
    if hidden == 512:
        assert set(np.unique(rs[rs != 0])) <= {0x04, 0x38}


@pytest.mark.parametrize("anti,noise_scale", [(0, 0.0), (1, 0.125), (-1, 0.125), (1, 0.0625)])
def test_embedding_dense(H, anti, noise_scale):
    rng = np.random.default_rng(11)
    V, hid, B, T = 256, 512, 32, 16
    emb = orc.init_rand_ternary(V * hid, 0x1000).reshape(V, hid)
    noise = orc.fill_noise(V * hid, 0xABCDEF).reshape(V, hid)
    toks = rng.integers(0, 256, (B, T)).astype(np.uint8)
    t = 3
    q, codes, sf = H.embedding_lookup_noise_quantize_nvfp4(dev(toks).view(-1)[t:], T, dev(emb), dev(noise) if anti else None,
                                                           hid, B, noise_scale, anti)
    rq, rc, rs = orc.embedding_quant(toks.reshape(-1)[t:], T, emb, noise if anti else None, hid, B, noise_scale, anti)
    assert same(q, rq) and same(codes, rc) and same(sf, rs)


def test_embedding_lowrank_population(H):
    """Population addressing: rows of 2 pairs x 2 signs share tokens; perturbation = ns*c_r * A[tok]B[j]."""
    import torch
    rng = np.random.default_rng(12)
    V, hid, B, T, rank, pairs = 256, 128, 4, 16, 2, 2
    R = B * T
    emb = orc.init_rand_ternary(V * hid, 0x1000).reshape(V, hid)
    toks = rng.integers(0, 256, (B, T)).astype(np.uint8)
    A = rng.integers(-4, 5, (pairs, V, rank)).astype(np.int8)
    Bm = rng.integers(-4, 5, (pairs, hid, rank)).astype(np.int8)
    tvec = rng.integers(-4, 5, (pairs, 3, hid)).astype(np.int8)
    sigma = 0.125
    cr = H.c_rank(rank)
    rows = 2 * pairs * R
    q = torch.zeros((rows, hid), dtype=torch.int8, device="cuda")
    codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
    tout = torch.zeros((rows, 3), dtype=torch.int32, device="cuda")
    H.rowquant(H.FE_EMBED_LOWRANK, rows=rows, cols_in=hid, cols_out=hid, rows_per_member=R, sigma=sigma, c_rank=cr,
               tokens=dev(toks), token_stride=1, row_mod=R, emb_w=dev(emb), embA=dev(A), embB=dev(Bm.transpose(0, 2, 1)),
               embA_pair_stride=V * rank, embB_pair_stride=hid * rank, rank=rank, out_q=q, ld_q=hid, out_codes=codes,
               out_sf=sf, tvec=dev(tvec), tvec_pair_stride=3 * hid, nvec=3, t_out=tout)
    qs, ts = [], []
    for member in range(2 * pairs):
        p, anti = member // 2, (1 if member % 2 == 0 else -1)
        scale = float(np.float32(anti * sigma) * np.float32(cr))
        rq, _, _ = orc.embedding_lowrank_quant(toks.reshape(-1), 1, emb, A[p], Bm[p], rank, hid, R, scale)
        qs.append(rq)
        ts.append(rq.astype(np.int32) @ tvec[p].astype(np.int32).T)
    rq = np.concatenate(qs)
    assert same(q, rq)
    rc, rs = orc.quantize_rowmajor(rq)
    assert same(codes, rc) and same(sf, rs)
    assert same(tout, np.concatenate(ts))


def test_add_pos_gelu(H):
    rng = np.random.default_rng(13)
    B, hid = 32, 512
    x = (rng.standard_normal((B, hid)) * 30).astype(np.float32)
    pos = (rng.random(hid).astype(np.float32) * 0.04 - 0.02)
    q, codes, sf = H.add_pos_gelu_quantize_nvfp4(dev(x), dev(pos), 0.8)
    rq, rc, rs = orc.add_pos_gelu_quant(x, pos, None, 0.8)
    qd = q.cpu().numpy()
    diff = np.abs(qd.astype(int) - rq.astype(int))
    assert diff.max() <= 1 and (diff != 0).mean() <= 1e-3  # tanhf: device vs host libm
    # the codes and scales must be the exact quantisation of the device's own int8 values
    rc2, rs2 = orc.quantize_rowmajor(qd)
    assert same(codes, rc2) and same(sf, rs2)


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_activation_and_gelu_quantize(H, mode):
    rng = np.random.default_rng(14 + mode)
    rows, cols = 33, 1024
    x = (rng.standard_normal((rows, cols)) * 60).astype(np.float32)
    if mode == 3:
        q, codes, sf = H.gelu_quantize_nvfp4(dev(x), cols, 1.0)
    else:
        q, codes, sf = H.activation_quantize_nvfp4(dev(x), cols, mode)
    rq, rc, rs = orc.activation_quant(x, cols, mode, 1.0)
    qd = q.cpu().numpy()
    if mode in (0, 1):
        assert same(q, rq) and same(codes, rc) and same(sf, rs)
    else:
        diff = np.abs(qd.astype(int) - rq.astype(int))
        assert diff.max() <= 1 and (diff != 0).mean() <= 1e-3
        rc2, rs2 = orc.quantize_rowmajor(qd)
        assert same(codes, rc2) and same(sf, rs2)


@pytest.mark.parametrize("rows,hid", [(1, 128), (32, 512), (257, 1024), (64, 2048)])
def test_absmean_norm_bit_exact(H, rows, hid):
    rng = np.random.default_rng(rows + hid)
    x = rng.integers(-127, 128, (rows, hid)).astype(np.int8)
    x[0, :] = 0  # abs-mean below 1 clamps to 1
    q, codes, sf = H.absmean_norm_q_nvfp4(dev(x), 1.0)
    rq, rc, rs = orc.absmean_norm_q(x.copy(), None, 0.0, 1.0)
    assert same(q, rq) and same(codes, rc) and same(sf, rs)


@pytest.mark.parametrize("rows,hid,add_scale", [(32, 512, 1.0), (129, 512, 0.37), (8, 1024, 1.0)])
def test_add_scaled_absmean_norm_bit_exact(H, rows, hid, add_scale):
    rng = np.random.default_rng(rows * 3 + hid)
    x = rng.integers(-127, 128, (rows, hid)).astype(np.int8)
    y = (rng.standard_normal((rows, hid)) * 40).astype(np.float32)
    xd = dev(x)
    q, codes, sf = H.add_scaled_to_int8_absmean_norm_q_nvfp4(xd, dev(y), add_scale, 1.0)
    xr = x.copy()
    rq, rc, rs = orc.absmean_norm_q(xr, y, add_scale, 1.0)
    assert same(xd, xr)  # residual stream updated in place
    assert same(q, rq) and same(codes, rc) and same(sf, rs)


def test_add_absmean_with_half_branch_input(H):
    """FE_ADD_ABSMEAN reading the branch output as IEEE halves (the scan's fp16 output): bit-exact against the oracle's
    residual add + abs-mean norm on the same values widened to fp32."""
    import torch
    rng = np.random.default_rng(21)
    rows, hid = 96, 512
    x = rng.integers(-127, 128, (rows, hid)).astype(np.int8)
    y16 = (rng.standard_normal((rows, hid)) * 3).astype(np.float16)
    tvec = rng.integers(-4, 5, (1, 1, hid)).astype(np.int8)
    xd = dev(x)
    yq = torch.zeros((rows, hid), dtype=torch.int8, device="cuda")
    codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
    tout = torch.zeros((rows, 1), dtype=torch.int32, device="cuda")
    H.rowquant(H.FE_ADD_ABSMEAN, rows=rows, cols_in=hid, cols_out=hid, rows_per_member=rows, sigma=0.125, inout_i8=xd, in_f32=dev(y16),
               ld_in=hid, in_f16=1, add_scale=1.0, norm_scale=1.0, out_q=yq, ld_q=hid, out_codes=codes, out_sf=sf, tvec=dev(tvec),
               tvec_pair_stride=hid, nvec=1, t_out=tout)
    xr = x.copy()
    rq, rc, rs = orc.absmean_norm_q(xr, y16.astype(np.float32), 1.0, 1.0)
    assert same(xd, xr) and same(yq, rq) and same(codes, rc) and same(sf, rs)
    assert same(tout, rq.astype(np.int32) @ tvec[0].astype(np.int32).T)


def test_pos_gelu_absmean_fused_population(H):
    """FE_POS_GELU_ABSMEAN = add_pos_gelu (kept as residual stream) followed by abs-mean norm, with per-pair pos noise."""
    import torch
    rng = np.random.default_rng(15)
    hid, B, T, pairs = 512, 2, 8, 2
    R = B * T
    rows = 2 * pairs * R
    x = (rng.standard_normal((rows, hid)) * 30).astype(np.float32)
    pos = (rng.random((T, hid)).astype(np.float32) * 0.04 - 0.02)
    pn = rng.integers(-4, 5, (pairs, T, hid)).astype(np.int8)
    tvec = rng.integers(-4, 5, (pairs, 4, hid)).astype(np.int8)
    sigma = 0.125
    xq = torch.zeros((rows, hid), dtype=torch.int8, device="cuda")
    yq = torch.zeros((rows, hid), dtype=torch.int8, device="cuda")
    codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
    tout = torch.zeros((rows, 4), dtype=torch.int32, device="cuda")
    H.rowquant(H.FE_POS_GELU_ABSMEAN, rows=rows, cols_in=hid, cols_out=hid, rows_per_member=R, sigma=sigma, in_f32=dev(x),
               ld_in=hid, inout_i8=xq, pos=dev(pos), pos_noise=dev(pn), pos_mod=T, noise_pair_stride=T * hid, act_scale=0.8,
               norm_scale=1.0, out_q=yq, ld_q=hid, out_codes=codes, out_sf=sf, tvec=dev(tvec), tvec_pair_stride=4 * hid,
               nvec=4, t_out=tout)
    xq_d = xq.cpu().numpy()
    ref_x = []
    for member in range(2 * pairs):
        p, anti = member // 2, (1 if member % 2 == 0 else -1)
        posn = (pos + np.float32(anti * sigma) * pn[p].astype(np.float32)).astype(np.float32)
        rq, _, _ = orc.add_pos_gelu_quant(x[member * R:(member + 1) * R], posn, np.arange(R) % T, 0.8)
        ref_x.append(rq)
    ref_x = np.concatenate(ref_x)
    diff = np.abs(xq_d.astype(int) - ref_x.astype(int))
    assert diff.max() <= 1 and (diff != 0).mean() <= 1e-3
    # everything downstream of the int8 residual is integer-exact given the device's own residual values
    rq, rc, rs = orc.absmean_norm_q(xq_d.copy(), None, 0.0, 1.0)
    assert same(yq, rq) and same(codes, rc) and same(sf, rs)
    tref = np.concatenate([rq[m * R:(m + 1) * R].astype(np.int32) @ tvec[m // 2].astype(np.int32).T for m in range(2 * pairs)])
    assert same(tout, tref)


@pytest.mark.parametrize("hid,nvec", [(512, 4), (2048, 1), (128, 3)])
def test_absmean_int8_rows_with_projections(H, hid, nvec):
    """FE_ABSMEAN on int8 rows (the quantiser that follows the residual-add GEMM epilogue) with the rank-r projections of
    the next GEMM: normalised int8, codes, scales and t all bit-exact."""
    import torch
    rng = np.random.default_rng(hid + nvec)
    pairs, R = 2, 24
    rows = 2 * pairs * R
    x = rng.integers(-127, 128, (rows, hid)).astype(np.int8)
    x[5, :] = 0
    x[6, :] = 0
    x[6, :5] = [127, -127, 100, -80, 3]  # abs-mean below 1 -> scale 1.7 > 1: the normalised values clip at +-127
    x[7, :] = rng.integers(-1, 2, hid)    # abs-mean just below 1
    tvec = rng.integers(-4, 5, (pairs, nvec, hid)).astype(np.int8)
    yq = torch.zeros((rows, hid), dtype=torch.int8, device="cuda")
    codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
    tout = torch.zeros((rows, nvec), dtype=torch.int32, device="cuda")
    H.rowquant(H.FE_ABSMEAN, rows=rows, cols_in=hid, cols_out=hid, rows_per_member=R, in_i8=dev(x), ld_in=hid, norm_scale=1.7,
               out_q=yq, ld_q=hid, out_codes=codes, out_sf=sf, tvec=dev(tvec), tvec_pair_stride=nvec * hid, nvec=nvec, t_out=tout)
    rq, rc, rs = orc.absmean_norm_q(x.copy(), None, 0.0, 1.7)
    assert same(yq, rq) and same(codes, rc) and same(sf, rs)
    tref = np.concatenate([rq[m * R:(m + 1) * R].astype(np.int32) @ tvec[m // 2].astype(np.int32).T for m in range(2 * pairs)])
    assert same(tout, tref)


@pytest.mark.parametrize("fe", ["absmean", "add_half"])
def test_rowquant_model_instance_agrees_with_the_general_one(fe):
    """The row-quantiser instance for the batched driver's calls (power-of-two shapes, exactly 1 or 4 projections, no int8 copy) against
    the general instance, which the same call takes as soon as it also asks for the int8 copy: codes, scales, projections and the
    residual stream must be bit-identical."""
    import torch
    from bitnet_nvfp4_b200 import host as H
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, hid, rpm = 8192, 512, 4096
    nvec = 4 if fe == "absmean" else 1
    x0 = torch.randint(-127, 128, (rows, hid), dtype=torch.int8, device="cuda", generator=g)
    yh = (torch.randn(rows, hid, device="cuda", generator=g) * 0.2).half()
    tv = torch.randint(-4, 5, (rows // (2 * rpm), nvec, hid), dtype=torch.int8, device="cuda", generator=g)
    outs = []
    for general in (False, True):
        x = x0.clone()
        codes = torch.zeros(rows * hid // 2, dtype=torch.uint8, device="cuda")
        sf = torch.zeros(H.sf_bytes(rows, hid), dtype=torch.uint8, device="cuda")
        t = torch.zeros(rows, nvec, dtype=torch.int32, device="cuda")
        q = torch.zeros(rows, hid, dtype=torch.int8, device="cuda")
        kw = dict(rows=rows, cols_in=hid, cols_out=hid, rows_per_member=rpm, ld_in=hid, norm_scale=24.0, out_codes=codes, out_sf=sf,
                  tvec=tv, tvec_pair_stride=nvec * hid, nvec=nvec, t_out=t)
        if general:
            kw.update(out_q=q, ld_q=hid)
        if fe == "absmean":
            H.rowquant(H.FE_ABSMEAN, in_i8=x, **kw)
        else:
            H.rowquant(H.FE_ADD_ABSMEAN, sigma=0.125, inout_i8=x, in_f32=yh, in_f16=1, add_scale=100.0, **kw)
        assert H.device_error() == 0
        outs.append((codes, sf, t, x))
    for u, v in zip(*outs):
        assert torch.equal(u, v)
    assert outs[0][2].abs().sum() > 0

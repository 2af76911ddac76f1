"""GPU parity against the reference's OWN NVFP4 quantiser kernels, dp4a ternary GEMM and rank-r helpers.

oracle/_ref/libref_quant.so is the reference's src/cuda_kernels.cu compiled for sm_100a from where it lies (its SM120
block-scaled GEMM compiles out behind its own architecture guard; the quantisers, the dp4a GEMMs and the lora helpers do
not). Each test runs a reference entry point and this library's entry point of the same name on the same device inputs
and compares the outputs: int8 values, e2m1 codes, ue4m3 scale bytes, int32 projections and integer dot products
bit-exactly; values downstream of tanhf within one int8 step on a stated fraction (two compilations of tanhf).
The same comparisons pin the CPU oracle (tests/oracle_lib.py) to the reference kernels.

Two quantiser modes of the reference are run (nvfp4_set_quant_mode):
  * Warp4: well-formed kernels; every int8 value, scale byte and code is compared.
  * Warp16 (the reference's default) and the Warp4 embedding kernel: lane 0 alone executes sixteen __shfl_sync calls whose
    mask names sixteen lanes (src/cuda_kernels.cu:1612-1622 and six more kernels), so the codes it gathers from the other
    lanes are undefined; compiled for sm_100a they come back as zero. What does not depend on that gather is compared:
    every int8 value, every scale byte, and the first code of every 16-element block. Shifting the input by 0..15 columns
    makes every element the first of a block once, which pins the code arithmetic of the default mode as well.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as orc

pytestmark = pytest.mark.gpu
SO = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_quant.so"


@pytest.fixture(scope="module")
def R():
    if not SO.exists():
        pytest.skip("oracle/_ref/libref_quant.so not built (needs the reference tree and CUTLASS headers at build time)")
    import torch
    assert torch.cuda.is_available()
    lib = C.CDLL(str(SO))
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    lib.refq_nvfp4_set_quant_mode.argtypes = [ci]
    lib.refq_nvfp4_sfa_bytes.restype = C.c_size_t
    lib.refq_nvfp4_sfb_bytes.restype = C.c_size_t
    lib.refq_nvfp4_sfa_bytes.argtypes = [ci, ci, ci]
    lib.refq_nvfp4_sfb_bytes.argtypes = [ci, ci, ci]
    lib.refq_nvfp4_quantize_a.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp]
    lib.refq_nvfp4_quantize_b.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp]
    lib.refq_nvfp4_quantize_wqkv_fused.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, cf, cf, cf, cf, vp, vp, vp]
    lib.refq_embedding_lookup_noise_quantize_nvfp4.argtypes = [vp, ci, vp, vp, ci, ci, cf, ci, vp, vp, vp, vp]
    lib.refq_add_pos_gelu_quantize_nvfp4.argtypes = [vp, vp, ci, ci, cf, vp, vp, vp, vp]
    lib.refq_gelu_quantize_nvfp4.argtypes = [vp, ci, ci, ci, cf, vp, vp, vp, vp]
    lib.refq_activation_quantize_nvfp4.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp, vp]
    lib.refq_absmean_norm_q_nvfp4.argtypes = [vp, ci, ci, ci, cf, vp, vp, vp, vp]
    lib.refq_add_scaled_to_int8_absmean_norm_q_nvfp4.argtypes = [vp, vp, ci, ci, ci, cf, cf, vp, vp, vp, vp]
    lib.refq_gemm_ternary_f.argtypes = [vp, vp, vp, ci, ci, ci, cf, vp, vp]
    lib.refq_gemm_ternary_f_noise.argtypes = [vp, vp, vp, vp, ci, ci, ci, cf, cf, vp, vp]
    lib.refq_lora_compute_t.argtypes = [vp, vp, ci, ci, ci, vp, vp]
    lib.refq_lora_add.argtypes = [vp, vp, ci, ci, ci, cf, vp, vp]
    lib.refq_gemm_ternary_lora_f.argtypes = [vp, vp, vp, ci, ci, ci, cf, vp, vp, ci, cf, vp, vp]
    lib.refq_split_qkvb_fused.argtypes = [vp, ci, ci, ci, vp, vp, vp, vp, cf, ci, vp]
    for f in ("quantize_a", "quantize_b", "quantize_wqkv_fused"):
        getattr(lib, "refq_nvfp4_" + f).restype = None
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


def sync():
    import torch
    torch.cuda.synchronize()


def bufs(H, rows, cols, want_q=True):
    import torch
    q = torch.zeros((rows, cols), dtype=torch.int8, device="cuda") if want_q else None
    codes = torch.zeros(H.matrix_bytes(rows, cols), dtype=torch.uint8, device="cuda")
    sf = torch.zeros(H.sf_bytes(rows, cols), dtype=torch.uint8, device="cuda")
    return q, codes, sf


WARP16, WARP4 = 0, 1


@pytest.fixture(params=[WARP16, WARP4], ids=["warp16", "warp4"])
def mode(R, request):
    R.refq_nvfp4_set_quant_mode(request.param)
    yield request.param
    R.refq_nvfp4_set_quant_mode(WARP16)


def codes_match(mine, ref, qmode, valid_bytes=None):
    """All codes (well-formed reference kernel) or the first code of every 16-element block (8 bytes per block)."""
    a = mine.cpu().numpy().reshape(-1)
    b = ref.cpu().numpy().reshape(-1)
    if valid_bytes is not None:
        a, b = a[:valid_bytes], b[:valid_bytes]
    if qmode == WARP4:
        return np.array_equal(a, b)
    return np.array_equal(a[0::8] & 0x0F, b[0::8] & 0x0F)


def eq(a, b):
    return np.array_equal(a.cpu().numpy().reshape(-1), (b.cpu().numpy() if hasattr(b, "cpu") else np.asarray(b)).reshape(-1))


def test_scale_buffer_sizes_match_reference(R, H):
    from bitnet_nvfp4_b200 import lib
    L = lib.load()
    for m, n, k in [(32, 512, 512), (32, 512, 1024), (4096, 512, 512), (1, 1568, 512), (129, 72, 128), (262144, 1024, 512)]:
        assert L.bnf4_nvfp4_sfa_bytes(m, n, k) == R.refq_nvfp4_sfa_bytes(m, n, k)
        assert L.bnf4_nvfp4_sfb_bytes(m, n, k) == R.refq_nvfp4_sfb_bytes(m, n, k)
        assert orc.sf_bytes(m, k) == R.refq_nvfp4_sfa_bytes(m, n, k)


@pytest.mark.parametrize("rows,k", [(1, 16), (31, 512), (32, 512), (129, 1024), (512, 2048), (300, 4096), (4096, 512)])
def test_quantize_a_matches_reference_kernel(R, H, mode, rows, k):
    rng = np.random.default_rng(rows * 7 + k)
    x = rng.integers(-127, 128, (rows, k)).astype(np.int8)
    x[rng.random((rows, k)) < 0.3] = 0
    if rows > 2:
        x[1, :] = 0
        x[2, : k // 2] = 1
    xd = dev(x)
    _, rc, rs = bufs(H, rows, k, False)
    R.refq_nvfp4_quantize_a(xd.data_ptr(), rows, 1, k, k, rc.data_ptr(), rs.data_ptr(), stream())
    codes, sf = H.nvfp4_quantize_a(xd)
    sync()
    assert codes_match(codes, rc, mode) and eq(sf, rs)
    oc, os_ = orc.quantize_rowmajor(x)
    assert codes_match(dev(oc), rc, mode) and eq(rs, os_)  # the CPU oracle is pinned by the same reference kernel


def test_default_mode_code_arithmetic_by_column_shifts(R, H):
    """Warp16 reference kernel: the first code of each block is well defined. With the input shifted by j = 0..15 columns
    every element is once the first of a block, with the scale of the 16 elements that start at it."""
    rng = np.random.default_rng(99)
    rows, k = 64, 512
    wide = rng.integers(-127, 128, (rows, k + 16)).astype(np.int8)
    wide[rng.random(wide.shape) < 0.4] = 0
    wide[3, :] = rng.integers(-1, 2, k + 16)
    wide[4, :] = orc.fill_noise(k + 16, 7)
    R.refq_nvfp4_set_quant_mode(WARP16)
    for j in range(16):
        xd = dev(wide[:, j:j + k])
        _, rc, rs = bufs(H, rows, k, False)
        R.refq_nvfp4_quantize_a(xd.data_ptr(), rows, 1, k, k, rc.data_ptr(), rs.data_ptr(), stream())
        codes, sf = H.nvfp4_quantize_a(xd)
        sync()
        assert eq(sf, rs) and codes_match(codes, rc, WARP16)


def test_quantize_b_and_short_input_match_reference_kernel(R, H, mode):
    rng = np.random.default_rng(5)
    w = rng.integers(-1, 2, (1568, 512)).astype(np.int8)
    wd = dev(w)
    _, rc, rs = bufs(H, 1568, 512, False)
    R.refq_nvfp4_quantize_b(wd.data_ptr(), 1, 1568, 512, 512, rc.data_ptr(), rs.data_ptr(), stream())
    codes, sf = H.nvfp4_quantize_b(wd)
    sync()
    assert codes_match(codes, rc, mode) and eq(sf, rs)
    # CLT noise operand (values in [-4, 4]) -- the reference's dense perturbation matrices
    e = orc.fill_noise(512 * 512, 0xE1).reshape(512, 512)
    ed = dev(e)
    _, rc, rs = bufs(H, 512, 512, False)
    R.refq_nvfp4_quantize_b(ed.data_ptr(), 1, 512, 512, 512, rc.data_ptr(), rs.data_ptr(), stream())
    codes, sf = H.nvfp4_quantize_b(ed)
    sync()
    assert codes_match(codes, rc, mode) and eq(sf, rs)
    oc, os_ = orc.quantize_rowmajor(e)
    assert codes_match(dev(oc), rc, mode) and eq(rs, os_)
    # k_in < k_out: the tail is zero
    x = rng.integers(-127, 128, (40, 96)).astype(np.int8)
    xd = dev(x)
    _, rc, rs = bufs(H, 40, 128, False)
    R.refq_nvfp4_quantize_a(xd.data_ptr(), 40, 1, 96, 128, rc.data_ptr(), rs.data_ptr(), stream())
    codes, sf = H.nvfp4_quantize_a(xd, k_out=128)
    sync()
    assert codes_match(codes, rc, mode) and eq(sf, rs)


@pytest.mark.parametrize("hidden", [128, 512])
def test_quantize_wqkv_fused_matches_reference_kernel(R, H, mode, hidden):
    import torch
    rng = np.random.default_rng(hidden)
    wq, wk, wv = (rng.integers(-1, 2, (hidden, hidden)).astype(np.int8) for _ in range(3))
    wb = rng.integers(-1, 2, (hidden,)).astype(np.int8)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hidden)))
    rows_total = (3 * hidden + 1 + 31) & ~31
    d = [dev(t) for t in (wq, wk, wv, wb)]
    rc = torch.zeros(H.matrix_bytes(rows_total, hidden), dtype=torch.uint8, device="cuda")
    rs = torch.zeros(H.sf_bytes(rows_total, hidden), dtype=torch.uint8, device="cuda")
    R.refq_nvfp4_quantize_wqkv_fused(*[t.data_ptr() for t in d], 1, hidden, hidden, rows_total, scale, scale, scale, scale,
                                     rc.data_ptr(), rs.data_ptr(), stream())
    codes, sf = H.nvfp4_quantize_wqkv_fused(*d, hidden, rows_total, scale)
    sync()
    n = (3 * hidden + 1) * hidden // 2
    assert codes_match(codes, rc, mode, n) and eq(sf, rs)
    oc, os_ = orc.quantize_wqkv_fused(wq, wk, wv, wb, hidden, scale)
    assert codes_match(dev(oc), rc, mode, n) and eq(rs, os_)


@pytest.mark.parametrize("anti,noise_scale", [(0, 0.0), (1, 0.125), (-1, 0.125), (1, 0.0625)])
def test_embedding_matches_reference_kernel(R, H, mode, anti, noise_scale):
    rng = np.random.default_rng(11)
    V, hid, B, T = 256, 512, 32, 16
    emb = orc.init_rand_ternary(V * hid, 0x1000).reshape(V, hid)
    noise = orc.fill_noise(V * hid, 0xABCDEF).reshape(V, hid)
    toks = dev(rng.integers(0, 256, (B, T)).astype(np.uint8))
    ed, nd = dev(emb), dev(noise)
    t = 3
    rq, rc, rs = bufs(H, B, hid)
    R.refq_embedding_lookup_noise_quantize_nvfp4(toks.view(-1)[t:].data_ptr(), T, ed.data_ptr(), nd.data_ptr() if anti else None, hid, B,
                                                 noise_scale, anti, rq.data_ptr(), rc.data_ptr(), rs.data_ptr(), stream())
    q, codes, sf = H.embedding_lookup_noise_quantize_nvfp4(toks.view(-1)[t:], T, ed, nd if anti else None, hid, B, noise_scale, anti)
    sync()
    if mode == WARP4:
        # the reference's Warp4 embedding kernel converts one value per lane only (src/cuda_kernels.cu:1994-2010): its int8
        # copy and scale bytes are complete, of its codes only the block's first one is the block's first element
        assert eq(q, rq) and eq(sf, rs) and codes_match(codes, rc, WARP16)
    else:
        assert eq(q, rq) and eq(sf, rs) and codes_match(codes, rc, mode)
    oq, oc, os_ = orc.embedding_quant(toks.cpu().numpy().reshape(-1)[t:], T, emb, noise if anti else None, hid, B, noise_scale, anti)
    assert eq(rq, oq) and eq(rs, os_)


def test_add_pos_gelu_matches_reference_kernel(R, H, mode):
    rng = np.random.default_rng(13)
    B, hid = 32, 512
    x = dev((rng.standard_normal((B, hid)) * 30).astype(np.float32))
    pos = dev(rng.random(hid).astype(np.float32) * 0.04 - 0.02)
    rq, rc, rs = bufs(H, B, hid)
    R.refq_add_pos_gelu_quantize_nvfp4(x.data_ptr(), pos.data_ptr(), hid, B, 0.8, rq.data_ptr(), rc.data_ptr(), rs.data_ptr(), stream())
    q, codes, sf = H.add_pos_gelu_quantize_nvfp4(x, pos, 0.8)
    sync()
    a, b = q.cpu().numpy().astype(int), rq.cpu().numpy().astype(int)
    assert np.abs(a - b).max() <= 1 and (a != b).mean() <= 1e-3   # tanhf of two compilations
    if np.array_equal(a, b):
        assert codes_match(codes, rc, mode) and eq(sf, rs)
    else:  # codes and scales are the reference quantiser's on this library's own int8 values
        _, c2, s2 = bufs(H, B, hid, False)
        R.refq_nvfp4_quantize_a(q.data_ptr(), B, 1, hid, hid, c2.data_ptr(), s2.data_ptr(), stream())
        sync()
        assert codes_match(codes, c2, mode) and eq(sf, s2)


@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_activation_and_gelu_quantize_match_reference_kernels(R, H, mode, act):
    """act 0..2 = activation_quantize_nvfp4 (none / ReLU / tanh), act 3 = gelu_quantize_nvfp4."""
    rng = np.random.default_rng(14 + act)
    rows, cols = 33, 1024
    x = dev((rng.standard_normal((rows, cols)) * (60 if act != 2 else 1.5)).astype(np.float32))
    rq, rc, rs = bufs(H, rows, cols)
    if act == 3:
        R.refq_gelu_quantize_nvfp4(x.data_ptr(), rows, cols, cols, 1.0, rq.data_ptr(), rc.data_ptr(), rs.data_ptr(), stream())
        q, codes, sf = H.gelu_quantize_nvfp4(x, cols, 1.0)
    else:
        R.refq_activation_quantize_nvfp4(x.data_ptr(), rows, cols, cols, act, rq.data_ptr(), rc.data_ptr(), rs.data_ptr(), stream())
        q, codes, sf = H.activation_quantize_nvfp4(x, cols, act)
    sync()
    a, b = q.cpu().numpy().astype(int), rq.cpu().numpy().astype(int)
    if act in (0, 1):
        assert np.array_equal(a, b) and codes_match(codes, rc, mode) and eq(sf, rs)
    else:
        assert np.abs(a - b).max() <= 1 and (a != b).mean() <= 1e-3
        _, c2, s2 = bufs(H, rows, cols, False)
        R.refq_nvfp4_quantize_a(q.data_ptr(), rows, 1, cols, cols, c2.data_ptr(), s2.data_ptr(), stream())
        sync()
        assert codes_match(codes, c2, mode) and eq(sf, s2)


@pytest.mark.parametrize("rows,hid,scale", [(1, 128, 1.0), (32, 512, 1.0), (257, 1024, 1.0), (64, 2048, 1.7)])
def test_absmean_norm_matches_reference_kernel(R, H, rows, hid, scale):
    rng = np.random.default_rng(rows + hid)
    x = rng.integers(-127, 128, (rows, hid)).astype(np.int8)
    x[0, :] = 0
    if rows > 8:
        x[6, :] = 0
        x[6, :5] = [127, -127, 100, -80, 3]
        x[7, :] = rng.integers(-1, 2, hid)
    xd = dev(x)
    rq, rc, rs = bufs(H, rows, hid)
    R.refq_absmean_norm_q_nvfp4(xd.data_ptr(), hid, rows, hid, scale, rq.data_ptr(), rc.data_ptr(), rs.data_ptr(), stream())
    q, codes, sf = H.absmean_norm_q_nvfp4(xd, scale)
    sync()
    assert eq(q, rq) and eq(codes, rc) and eq(sf, rs)
    oq, oc, os_ = orc.absmean_norm_q(x.copy(), None, 0.0, scale)
    assert eq(rq, oq) and eq(rc, oc) and eq(rs, os_)


@pytest.mark.parametrize("rows,hid,add_scale", [(32, 512, 1.0), (129, 512, 0.37), (8, 1024, 1.0), (16, 512, 900.0)])
def test_add_scaled_absmean_norm_matches_reference_kernel(R, H, rows, hid, add_scale):
    """add_scale 900 drives |y*add_scale| far beyond the int8 range: the residual add must saturate at +-127."""
    rng = np.random.default_rng(rows * 3 + hid)
    x = rng.integers(-127, 128, (rows, hid)).astype(np.int8)
    y = (rng.standard_normal((rows, hid)) * 40).astype(np.float32)
    x_ref, x_my, yd = dev(x), dev(x), dev(y)
    rq, rc, rs = bufs(H, rows, hid)
    R.refq_add_scaled_to_int8_absmean_norm_q_nvfp4(x_ref.data_ptr(), yd.data_ptr(), hid, rows, hid, add_scale, 1.0, rq.data_ptr(),
                                                   rc.data_ptr(), rs.data_ptr(), stream())
    q, codes, sf = H.add_scaled_to_int8_absmean_norm_q_nvfp4(x_my, yd, add_scale, 1.0)
    sync()
    assert eq(x_my, x_ref)
    assert eq(q, rq) and eq(codes, rc) and eq(sf, rs)
    xo = x.copy()
    oq, oc, os_ = orc.absmean_norm_q(xo, y, add_scale, 1.0)
    assert eq(x_ref, xo) and eq(rq, oq) and eq(rc, oc) and eq(rs, os_)


@pytest.mark.parametrize("batch,rows,cols", [(32, 512, 512), (5, 1, 512), (32, 256, 1024), (7, 33, 256)])
def test_gemm_ternary_f_matches_reference_kernel(R, H, batch, rows, cols):
    import torch
    rng = np.random.default_rng(batch + rows + cols)
    x = dev(rng.integers(-127, 128, (batch, cols)).astype(np.int8))
    w = dev(rng.integers(-1, 2, (rows, cols)).astype(np.int8))
    sx = dev(np.ones(cols // 256 if cols >= 256 else 1, np.float32))
    out_scale = float(np.float32(1.0) / np.sqrt(np.float32(cols)))
    ref = torch.zeros((batch, rows), dtype=torch.float32, device="cuda")
    R.refq_gemm_ternary_f(x.data_ptr(), w.data_ptr(), sx.data_ptr(), rows, cols, batch, out_scale, ref.data_ptr(), stream())
    got = H.gemm_ternary_f(x, w, sx, out_scale)
    sync()
    assert torch.equal(got, ref)
    assert np.array_equal(ref.cpu().numpy(), orc.gemm_ternary_f(x.cpu().numpy(), w.cpu().numpy(), sx.cpu().numpy(), out_scale))


@pytest.mark.parametrize("rank", [1, 2, 4])
def test_rank_r_helpers_match_reference_kernels(R, H, rank):
    """t = x.B (int32) and out += scale * t.A^T: the reference's lora_compute_t / lora_add / gemm_ternary_lora_f are the
    statement of the rank-r perturbation that the GEMM epilogue fuses."""
    import torch
    rng = np.random.default_rng(rank)
    batch, rows, cols = 24, 384, 512
    x = dev(rng.integers(-127, 128, (batch, cols)).astype(np.int8))
    w = dev(rng.integers(-1, 2, (rows, cols)).astype(np.int8))
    Bm = dev(rng.integers(-4, 5, (cols, rank)).astype(np.int8))
    A = dev(rng.integers(-4, 5, (rows, rank)).astype(np.int8))
    sx = dev(np.ones(cols // 256, np.float32))
    t_ref = torch.zeros((batch, rank), dtype=torch.int32, device="cuda")
    R.refq_lora_compute_t(x.data_ptr(), Bm.data_ptr(), cols, batch, rank, t_ref.data_ptr(), stream())
    t = H.lora_compute_t(x, Bm, rank)
    sync()
    assert torch.equal(t, t_ref)
    base = dev((rng.standard_normal((batch, rows)) * 3).astype(np.float32))
    o_ref, o_my = base.clone(), base.clone()
    R.refq_lora_add(t_ref.data_ptr(), A.data_ptr(), rows, batch, rank, 0.00552, o_ref.data_ptr(), stream())
    H.lora_add(t, A, rows, 0.00552, o_my)
    sync()
    assert torch.equal(o_my, o_ref)
    # the reference's fused form: out = out_scale * x.W^T + lora_scale * t.A^T  ==  ternary GEMM followed by lora_add
    out_scale = float(np.float32(1.0) / np.sqrt(np.float32(cols)))
    fused = torch.zeros((batch, rows), dtype=torch.float32, device="cuda")
    R.refq_gemm_ternary_lora_f(x.data_ptr(), w.data_ptr(), sx.data_ptr(), rows, cols, batch, out_scale, A.data_ptr(), t_ref.data_ptr(),
                               rank, 0.00552, fused.data_ptr(), stream())
    two = H.gemm_ternary_f(x, w, sx, out_scale)
    H.lora_add(t, A, rows, 0.00552, two)
    sync()
    a, b = two.cpu().numpy(), fused.cpu().numpy()
    assert np.abs(a - b).max() <= 2e-6 * np.abs(b).max()  # one fused multiply-add against a multiply and an add


def test_split_qkvb_matches_reference_kernel(R, H):
    import torch
    rng = np.random.default_rng(3)
    batch, hidden = 9, 512
    fc = (3 * hidden + 1 + 31) & ~31
    qkv = dev(rng.standard_normal((batch, fc)).astype(np.float32))
    refs = [torch.zeros((batch, hidden), dtype=torch.float32, device="cuda") for _ in range(3)] + [torch.zeros(batch, dtype=torch.float32, device="cuda")]
    R.refq_split_qkvb_fused(qkv.data_ptr(), batch, hidden, fc, *[t.data_ptr() for t in refs], -2.0, 0, stream())
    got = H.split_qkvb_fused(qkv, hidden, -2.0)
    sync()
    for a, b in zip(got, refs):
        assert torch.equal(a, b)

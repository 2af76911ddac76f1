"""GPU parity of the EFLA recurrence, cross-entropy, noise generation, ES update and the ternary GEMM
(C ABI of libbnf4) against the CPU oracle.

Integer work (noise, pair seeds, ternary weights, int32 group sums) is compared bit-exactly. Floating-point
tolerances are stated per test.
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


def make_qkv(rng, rows, hidden, fused_cols, scale=1.0):
    qkv = np.zeros((rows, fused_cols), np.float32)
    qkv[:, :3 * hidden] = (rng.standard_normal((rows, 3 * hidden)) * scale).astype(np.float32)
    qkv[:, 3 * hidden] = rng.standard_normal(rows).astype(np.float32)
    return qkv


# ---------------------------------------------------------------------------------------------- EFLA
SCAN_TOL = 2e-3  # worst element of a whole-sequence scan against the oracle, relative to max |y|


@pytest.mark.parametrize("hidden,heads,method", [(128, 1, 1), (512, 1, 1), (128, 2, 1), (128, 1, 0), (256, 8, 1)])
def test_efla_step_api_with_hbm_state(H, hidden, heads, method):
    """Single-step entry points: state lives in HBM between calls (fp16), three consecutive steps."""
    import torch
    rng = np.random.default_rng(hidden + heads + method)
    B = 5
    fc = (3 * hidden + 1 + 31) & ~31
    hd = hidden // heads
    S_ref = np.zeros((B, heads, hd, hd), np.uint16)
    S_dev = torch.zeros((B, heads, hd, hd), dtype=torch.float16, device="cuda")
    for step in range(3):
        qkv = make_qkv(rng, B, hidden, fc, 0.5)
        ref = orc.efla_step(S_ref, qkv, -2.0, hidden, heads, method)
        if heads == 1:
            out = H.efla_step_half_qkv_fused(S_dev, dev(qkv), fc, -2.0, hidden, B, method, 1e-6)
        else:
            out = torch.empty((B, hidden), dtype=torch.float32, device="cuda")
            qd = dev(qkv)
            H.efla_scan(state=S_dev, state_fp16=1, q=qd, k=qd[:, hidden:], v=qd[:, 2 * hidden:], beta_raw=qd[:, 3 * hidden:],
                        ld_qkv=fc, ld_beta=fc, beta_bias=-2.0, seqs_per_bias=1, hidden=hidden, heads=heads, seqs=B, T=1,
                        method=method, eps=1e-6, out=out, ld_out=hidden)
        got = out.cpu().numpy()
        assert np.abs(got - ref).max() <= 2e-3 * max(1e-6, np.abs(ref).max())
    # fp16 state: identical up to one fp16 ulp on a small fraction (rsqrt / expm1 differ by an ulp between device and host)
    sd = S_dev.cpu().numpy().view(np.uint16).astype(np.int32)
    assert (np.abs(sd - S_ref.astype(np.int32)) > 1).mean() <= 1e-3


def test_efla_step_fp32_state(H):
    import torch
    rng = np.random.default_rng(3)
    hidden, B = 128, 4
    fc = (3 * hidden + 1 + 31) & ~31
    S = torch.zeros((B, hidden, hidden), dtype=torch.float32, device="cuda")
    qkv = make_qkv(rng, B, hidden, fc, 0.5)
    out = H.efla_step_qkv_fused(S, dev(qkv), fc, -2.0, hidden, B, 1, 1e-6).cpu().numpy()
    # first step from zero state: S = alpha k v^T, y = (k.q^) alpha v -- check against numpy in float64
    q, k, v, br = qkv[:, :hidden], qkv[:, hidden:2 * hidden], qkv[:, 2 * hidden:3 * hidden], qkv[:, 3 * hidden]
    qn = q / np.sqrt((q.astype(np.float64) ** 2).sum(1, keepdims=True) + 1e-6)
    lam = np.maximum((k.astype(np.float64) ** 2).sum(1), 1e-6)
    beta = 1 / (1 + np.exp(-(br.astype(np.float64) - 2.0)))
    alpha = -np.expm1(-beta * lam) / (lam + 1e-6)
    ref = ((k * qn).sum(1) * alpha)[:, None] * v
    assert np.abs(out - ref).max() <= 1e-4 * np.abs(ref).max()


GENERIC, PER_TOKEN, CHUNKED = 1, 2, 3  # bnf4_efla_desc.variant


@pytest.mark.parametrize("variant", [GENERIC, PER_TOKEN, CHUNKED])
@pytest.mark.parametrize("hidden,heads,seqs,T", [(512, 8, 6, 32), (128, 2, 40, 16), (64, 1, 3, 128), (128, 2, 5, 24), (512, 8, 9, 128)])
def test_efla_scan_whole_sequence(H, hidden, heads, seqs, T, variant):
    """Whole-sequence scan with the state on chip: the generic kernel, the per-token register kernel (the reference's fp16
    rounding after every token) and the chunked tensor-core kernel (fp16 operands, state rounded every 16 tokens; T = 24
    ends in a partial chunk). All three are held to the same bound against the oracle's per-token recurrence."""
    import torch
    rng = np.random.default_rng(hidden * 3 + heads + T)
    fc = (3 * hidden + 1 + 31) & ~31
    qkv = make_qkv(rng, seqs * T, hidden, fc, 0.3)
    per_bias = 2
    bb = (rng.standard_normal((seqs + per_bias - 1) // per_bias) * 0.2 - 2.0).astype(np.float32)
    bb_seq = np.repeat(bb, per_bias)[:seqs]
    ref = orc.efla_scan(qkv.reshape(seqs, T, fc), bb_seq, hidden, heads)
    qd = dev(qkv)
    out = torch.empty((seqs * T, hidden), dtype=torch.float32, device="cuda")
    H.efla_scan(state=None, state_fp16=1, q=qd, k=qd[:, hidden:], v=qd[:, 2 * hidden:], beta_raw=qd[:, 3 * hidden:], ld_qkv=fc,
                ld_beta=fc, beta_bias_seq=dev(bb), seqs_per_bias=per_bias, hidden=hidden, heads=heads, seqs=seqs, T=T,
                method=1, eps=1e-6, out=out, ld_out=hidden, variant=variant)
    got = out.cpu().numpy().reshape(seqs, T, hidden)
    # the fp16 state rounding is reproduced; residual differences come from rsqrt/expm1 ulps and summation order, which now
    # and then move a state element to the neighbouring fp16 value
    dev_ = np.abs(got - ref)
    assert dev_.max() <= SCAN_TOL * np.abs(ref).max()
    assert np.median(dev_) <= (3e-4 if variant == CHUNKED else 1e-4) * np.abs(ref).max()


@pytest.mark.parametrize("in16,out16", [(1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("hidden,heads,seqs,T", [(512, 8, 6, 128), (128, 2, 7, 40)])
def test_efla_chunked_scan_with_half_inputs_and_outputs(H, hidden, heads, seqs, T, in16, out16):
    """The chunked kernel reading q | k | v as IEEE halves and / or writing y as halves (what the batched driver uses): against
    the oracle's per-token recurrence on the values the kernel is given, same bound as the fp32 interface plus half an fp16 ulp
    of the output where y is rounded."""
    import torch
    rng = np.random.default_rng(hidden + T + 2 * in16 + out16)
    fc = (3 * hidden + 1 + 31) & ~31
    qkv = make_qkv(rng, seqs * T, hidden, fc, 0.4)
    if in16:
        qkv[:, :3 * hidden] = qkv[:, :3 * hidden].astype(np.float16).astype(np.float32)   # the values the kernel sees
    bb = (rng.standard_normal(seqs) * 0.2 - 2.0).astype(np.float32)
    ref = orc.efla_scan(qkv.reshape(seqs, T, fc), bb, hidden, heads)
    out = torch.zeros((seqs * T, hidden), dtype=torch.float16 if out16 else torch.float32, device="cuda")
    beta = dev(np.ascontiguousarray(qkv[:, 3 * hidden]))
    if in16:
        q16 = dev(np.ascontiguousarray(qkv[:, :3 * hidden]).astype(np.float16))
        H.efla_scan(state=None, state_fp16=1, q=q16, k=q16[:, hidden:], v=q16[:, 2 * hidden:], beta_raw=beta, ld_qkv=3 * hidden, ld_beta=1,
                    beta_bias_seq=dev(bb), seqs_per_bias=1, hidden=hidden, heads=heads, seqs=seqs, T=T, method=1, eps=1e-6, out=out,
                    ld_out=hidden, variant=CHUNKED, qkv_f16=1, out_f16=out16)
    else:
        qd = dev(qkv)
        H.efla_scan(state=None, state_fp16=1, q=qd, k=qd[:, hidden:], v=qd[:, 2 * hidden:], beta_raw=beta, ld_qkv=fc, ld_beta=1,
                    beta_bias_seq=dev(bb), seqs_per_bias=1, hidden=hidden, heads=heads, seqs=seqs, T=T, method=1, eps=1e-6, out=out,
                    ld_out=hidden, variant=CHUNKED, out_f16=out16)
    got = out.float().cpu().numpy().reshape(seqs, T, hidden)
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() <= (SCAN_TOL + (2.0 ** -11 if out16 else 0.0)) * scale


def test_efla_half_interface_is_chunked_only(H):
    import torch
    from bitnet_nvfp4_b200 import lib
    q16 = torch.zeros((16, 192), dtype=torch.float16, device="cuda")
    out = torch.zeros((16, 64), dtype=torch.float32, device="cuda")
    beta = torch.zeros(16, dtype=torch.float32, device="cuda")
    with pytest.raises(lib.Bnf4Error):
        H.efla_scan(state=None, state_fp16=1, q=q16, k=q16[:, 64:], v=q16[:, 128:], beta_raw=beta, ld_qkv=192, ld_beta=1, beta_bias=-2.0,
                    seqs_per_bias=1, hidden=64, heads=1, seqs=1, T=16, method=1, eps=1e-6, out=out, ld_out=64, variant=PER_TOKEN, qkv_f16=1)


def _recover_states(y, q_scale):
    """y [64 probes][T][heads][64] with probe d reading row d of every head's state: S[t][head][d][n] as fp16 bit patterns."""
    s = (y / q_scale).astype(np.float16)          # y = S[d, n] * q^_d exactly (one fp32 rounding); the division undoes it
    return s.transpose(1, 2, 0, 3).view(np.uint16)  # [T][heads][d][n]


def test_efla_scan_state_rounding_matches_multiply_add(H):
    """The register-state scan updates the state with tensor-core MMAs that use fp16 accumulators. The property it relies
    on: the MMA forms the exact products, adds the fp16 state and rounds ONCE to nearest -- i.e. it equals
    fp16_rn(fmaf(alpha k, diff, S)), the reference's update (src/efla_lm_kernels.cu:1349). Checked through the public
    entry point: 64 sequences share k, v, beta and differ in q = e_d, so sequence d reads row d of the state after every
    token (y = S[d, :] * q^_d, one exact product). The recovered states must equal the oracle's multiply-add states except
    for rare one-ulp differences (an exact sum within 2^-21 relative of a rounding midpoint; alpha from expm1f)."""
    import torch
    rng = np.random.default_rng(4242)
    hidden, heads, T, probes = 512, 8, 6, 64
    fc = (3 * hidden + 1 + 31) & ~31
    base = make_qkv(rng, T, hidden, fc, 0.4)                      # one k, v, beta stream for all probes
    qkv = np.repeat(base[None], probes, axis=0)                   # [probe][T][fc]
    qkv[:, :, :hidden] = 0.0
    for d in range(probes):
        qkv[d, :, d:hidden:64] = 1.0                              # q = e_d in every head
    q_scale = np.float32(1.0) / np.sqrt(np.float32(1.0) + np.float32(1e-6))
    ref = orc.efla_scan(qkv, np.full(probes, -2.0, np.float32), hidden, heads)
    qd = dev(qkv.reshape(probes * T, fc))
    out = torch.empty((probes * T, hidden), dtype=torch.float32, device="cuda")
    H.efla_scan(state=None, state_fp16=1, q=qd, k=qd[:, hidden:], v=qd[:, 2 * hidden:], beta_raw=qd[:, 3 * hidden:], ld_qkv=fc,
                ld_beta=fc, beta_bias=-2.0, seqs_per_bias=1, hidden=hidden, heads=heads, seqs=probes, T=T, method=1, eps=1e-6,
                out=out, ld_out=hidden, variant=PER_TOKEN)
    got = out.cpu().numpy().reshape(probes, T, heads, 64)
    s_got = _recover_states(got, q_scale).astype(np.int32)
    s_ref = _recover_states(ref.reshape(probes, T, heads, 64), q_scale).astype(np.int32)
    assert np.abs(s_ref).max() > 0
    # token 0 starts from a zero state: fp16_rn(alpha k * diff) with no accumulation error to inherit
    ulp = np.abs(s_got - s_ref)
    frac = [(ulp[t] != 0).mean() for t in range(T)]
    assert frac[0] <= 1e-2 and ulp[0].max() <= 1, (frac, ulp.max(axis=(1, 2, 3)))
    # later tokens inherit the rare flips through k.S: still few, and small against the state (elements near zero can be many
    # of their own ulps apart, so the bound is one fp16 step of the largest element)
    f_got = s_got.astype(np.uint16).view(np.float16).astype(np.float32)
    f_ref = s_ref.astype(np.uint16).view(np.float16).astype(np.float32)
    for t in range(T):
        assert frac[t] <= 3e-2, frac
        assert np.abs(f_got[t] - f_ref[t]).max() <= 2.0 ** -10 * np.abs(f_ref[t]).max(), t


def test_efla_scan_one_head_of_512(H):
    """heads = 1, head_dim = hidden = 512: the reference's own shape (one H x H state per sequence), through the scan entry point."""
    import torch
    rng = np.random.default_rng(512)
    hidden, heads, seqs, T = 512, 1, 3, 24
    fc = (3 * hidden + 1 + 31) & ~31
    qkv = make_qkv(rng, seqs * T, hidden, fc, 0.3)
    bb = np.array([-2.0, -1.7, -2.3], np.float32)
    ref = orc.efla_scan(qkv.reshape(seqs, T, fc), bb, hidden, heads)
    qd = dev(qkv)
    out = torch.empty((seqs * T, hidden), dtype=torch.float32, device="cuda")
    H.efla_scan(state=None, state_fp16=1, q=qd, k=qd[:, hidden:], v=qd[:, 2 * hidden:], beta_raw=qd[:, 3 * hidden:], ld_qkv=fc,
                ld_beta=fc, beta_bias_seq=dev(bb), seqs_per_bias=1, hidden=hidden, heads=heads, seqs=seqs, T=T, method=1, eps=1e-6,
                out=out, ld_out=hidden)
    got = out.cpu().numpy().reshape(seqs, T, hidden)
    assert np.abs(got - ref).max() <= SCAN_TOL * np.abs(ref).max()


# ---------------------------------------------------------------------------------------------- cross entropy
def test_cross_entropy_step_api(H):
    import torch
    rng = np.random.default_rng(21)
    B, V, T = 32, 256, 16
    logits = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    bias = (rng.standard_normal(V) * 0.1).astype(np.float32)
    noise = orc.fill_noise(V, 99).astype(np.float32)
    targets = rng.integers(0, 256, (B, T)).astype(np.uint8)
    acc = torch.zeros(1, dtype=torch.float32, device="cuda")
    td = dev(targets).view(-1)
    H.cross_entropy_loss(dev(logits), dev(bias), dev(noise), -0.125, td[5:], T, acc)
    H.cross_entropy_loss(dev(logits), dev(bias), dev(noise), -0.125, td[5:], T, acc)  # accumulates
    tot, _ = orc.cross_entropy_sum(logits, bias, noise, -0.125, targets.reshape(-1)[5:], T)
    assert abs(acc.item() - 2 * tot) <= 1e-5 * abs(2 * tot)


def test_cross_entropy_population(H):
    rng = np.random.default_rng(22)
    members, R, V, ld = 6, 200, 256, 256
    logits = (rng.standard_normal((members * R, ld)) * 3).astype(np.float32)
    bias = (rng.standard_normal(V) * 0.1).astype(np.float32)
    noise = np.stack([orc.fill_noise(V, 1000 + p) for p in range(members // 2)])
    targets = rng.integers(0, 256, R).astype(np.uint8)
    loss = H.cross_entropy_population(dev(logits), ld, dev(bias), dev(noise), 0.125, dev(targets), V, members, R).cpu().numpy()
    for m in range(members):
        bns = 0.125 if m % 2 == 0 else -0.125
        tot, _ = orc.cross_entropy_sum(logits[m * R:(m + 1) * R], bias, noise[m // 2].astype(np.float32), bns, targets, 1)
        assert abs(loss[m] - tot / R) <= 1e-5 * abs(tot / R)  # stated bound on the per-member loss: 1e-4


# ---------------------------------------------------------------------------------------------- noise / seeds
@pytest.mark.parametrize("use_clt", [True, False])
def test_noise_and_pair_seeds_bit_exact(H, use_clt):
    n = 100003
    got = H.fill_ternary_noise(n, 0xDEADBEEFCAFE, use_clt, 4).cpu().numpy()
    assert np.array_equal(got, orc.fill_noise(n, 0xDEADBEEFCAFE, use_clt, 4))
    seeds = H.fill_pair_seeds(1, 7, 1024).cpu().numpy().view(np.uint64)
    assert np.array_equal(seeds, orc.fill_pair_seeds(1, 7, 1024))


def test_noise_batched(H):
    import ctypes as C
    import torch
    from bitnet_nvfp4_b200 import lib
    sizes = [1000, 70000, 513]
    outs = [torch.zeros(s, dtype=torch.int8, device="cuda") for s in sizes]
    descs = (lib.NoiseDesc * len(sizes))(*[lib.NoiseDesc(o.data_ptr(), s, 0x55 + i) for i, (o, s) in enumerate(zip(outs, sizes))])
    raw = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
    max_blocks = (max(sizes) + 255) // 256
    lib.check(lib.load().bnf4_fill_ternary_noise_batched(raw.data_ptr(), len(sizes), max_blocks, 1, 4,
                                                         torch.cuda.current_stream().cuda_stream))
    for i, (o, s) in enumerate(zip(outs, sizes)):
        assert np.array_equal(o.cpu().numpy(), orc.fill_noise(s, 0x55 + i, True, 4))


# ---------------------------------------------------------------------------------------------- ES update
def test_es_update_dense_bit_exact(H):
    """Z, sum of squares, inv_rms and the gated round-clip update: int8 weights identical to the oracle."""
    import torch
    rng = np.random.default_rng(31)
    n, pairs = 40000, 96
    pw = orc.shape_pair_weights(rng.standard_normal(pairs).astype(np.float32))
    pw[5] = 0.0
    seeds = orc.fill_pair_seeds(1, 0, pairs)
    salt = 0x222222
    w = orc.init_rand_ternary(n, 0x2000)
    shadow = w.astype(np.float32)
    Zr, ssr = orc.compute_z_sumsq(pw, seeds, salt, n)
    Zd, ssd = H.compute_z_sumsq(dev(pw), dev(seeds.view(np.int64)), salt, n)
    assert np.array_equal(Zd.cpu().numpy(), Zr)
    assert ssd.item() == ssr
    ema_d = torch.zeros(1, dtype=torch.float32, device="cuda")
    ema_r = 0.0
    wd, sd = dev(w), dev(shadow)
    wr, sr = w.copy(), shadow.copy()
    for it in range(2):  # second pass exercises the EMA branch
        inv_d = H.update_inv_rms(ssd, ema_d, True, 0.95, 1e-3, n)
        inv_r, ema_r = orc.update_inv_rms(ssr, ema_r, True, 0.95, 1e-3, n)
        assert inv_d.item() == inv_r and ema_d.item() == ema_r
        thresh = float(np.float32(0.008) * np.sqrt(np.float32(pairs)))
        H.update_shadow_ternary_device(wd, sd, Zd, inv_d, 0.8, thresh)
        orc.update_shadow_ternary(wr, sr, Zr, inv_r, 0.8, thresh)
        assert np.array_equal(wd.cpu().numpy(), wr)
        assert np.array_equal(sd.cpu().numpy(), sr)
    assert (wr != w).any()


@pytest.mark.parametrize("rank,rows,cols", [(1, 100, 130), (4, 64, 512), (2, 1, 512)])
def test_es_update_lowrank_z_bit_exact(H, rank, rows, cols):
    rng = np.random.default_rng(32 + rank)
    pairs = 70
    pw = orc.shape_pair_weights(rng.standard_normal(pairs).astype(np.float32))
    seeds = orc.fill_pair_seeds(1, 3, pairs)
    salt = 0x999999
    cs = H.c_rank(rank)
    Zr, ssr = orc.compute_z_sumsq_lowrank(pw, seeds, salt, rows, cols, rank, cs)
    A = np.zeros((pairs, rows, rank), np.int8)
    Bt = np.zeros((pairs, rank, cols), np.int8)
    for p in range(pairs):
        sm = orc.mix(int(seeds[p]), salt)
        A[p] = orc.fill_noise(rows * rank, orc.mix(sm, 0xA11CE)).reshape(rows, rank)
        Bt[p] = orc.fill_noise(cols * rank, orc.mix(sm, 0xB0B)).reshape(cols, rank).T
    Zd, ssd = H.compute_z_sumsq_lowrank(dev(pw), dev(A), dev(Bt), rows, cols, rank, cs)
    assert np.array_equal(Zd.cpu().numpy(), Zr)
    assert ssd.item() == ssr


def test_shape_pair_weights_host(H):
    rng = np.random.default_rng(33)
    w = rng.standard_normal(1024).astype(np.float32)
    w[10] = w[20]  # a tie: broken by index on both sides
    for mode in (0, 1, 2):
        got = H.shape_pair_weights(w.copy(), mode, 3.0)
        assert np.array_equal(got, orc.shape_pair_weights(w, mode, 3.0))


# ---------------------------------------------------------------------------------------------- ternary GEMM
@pytest.mark.parametrize("batch,rows,cols", [(32, 1, 512), (32, 256, 512), (7, 33, 300), (64, 512, 1024)])
def test_gemm_ternary_f_exact(H, batch, rows, cols):
    rng = np.random.default_rng(batch + rows + cols)
    x = rng.integers(-127, 128, (batch, cols)).astype(np.int8)
    w = rng.integers(-1, 2, (rows, cols)).astype(np.int8)
    sx = np.ones((cols + 255) // 256, np.float32)
    os_ = float(np.float32(1.0) / np.sqrt(np.float32(cols)))
    got = H.gemm_ternary_f(dev(x), dev(w), dev(sx), os_).cpu().numpy()
    assert np.array_equal(got, orc.gemm_ternary_f(x, w, sx, os_))  # integer sums are exact; the few fp32 steps are ordered alike


def test_lora_helpers_and_split(H):
    rng = np.random.default_rng(41)
    batch, cols, rows, rank = 32, 512, 384, 3
    x = rng.integers(-127, 128, (batch, cols)).astype(np.int8)
    Bm = rng.integers(-4, 5, (cols, rank)).astype(np.int8)
    A = rng.integers(-4, 5, (rows, rank)).astype(np.int8)
    t = H.lora_compute_t(dev(x), dev(Bm), rank)
    tr = orc.lora_compute_t(x, Bm, rank)
    assert np.array_equal(t.cpu().numpy(), tr)
    out = rng.standard_normal((batch, rows)).astype(np.float32)
    got = H.lora_add(t, dev(A), rows, 0.00552, dev(out)).cpu().numpy()
    assert np.array_equal(got, orc.lora_add(tr, A, rows, 0.00552, out.copy()))
    hidden = 128
    fc = (3 * hidden + 1 + 31) & ~31
    qkv = make_qkv(rng, 9, hidden, fc)
    q, k, v, b = H.split_qkvb_fused(dev(qkv), hidden, -2.0)
    assert np.array_equal(q.cpu().numpy(), qkv[:, :hidden]) and np.array_equal(v.cpu().numpy(), qkv[:, 2 * hidden:3 * hidden])
    assert np.array_equal(b.cpu().numpy(), qkv[:, 3 * hidden] + np.float32(-2.0))

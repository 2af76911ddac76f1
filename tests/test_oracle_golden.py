"""CPU tests: the oracle (and the host-side pieces of the product) against the committed golden fixtures.

tests/golden/ref_host.npz      outputs of the reference's own host functions (see tests/golden/gen_golden.py)
tests/golden/cutlass_codec.npz e2m1 / ue4m3 conversions and the scale-factor layout from the CUTLASS headers
"""
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as orc

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def ref():
    return np.load(GOLD / "ref_host.npz")


@pytest.fixture(scope="module")
def codec():
    return np.load(GOLD / "cutlass_codec.npz")


# ------------------------------------------------------------------------------------------------ rng / noise / init
def test_mix_and_splitmix64_match_reference(ref):
    L = orc.lib()
    got = np.array([orc.mix(int(a), int(b)) for a, b in zip(ref["mix_a"], ref["mix_b"])], np.uint64)
    assert np.array_equal(got, ref["mix"])
    import ctypes as C
    for i, s in enumerate(ref["sm_seed"]):
        st = C.c_uint64(int(s))
        out = np.array([L.orc_splitmix64(C.byref(st)) for _ in range(16)], np.uint64)
        assert np.array_equal(out, ref["sm_out"][i])
    tern = np.array([L.orc_ternary_from_u64(C.c_uint64(int(x))) for x in ref["tern_in"]], np.int8)
    assert np.array_equal(tern, ref["tern"])


def test_noise_hash_matches_reference(ref):
    L = orc.lib()
    import ctypes as C
    nh = ref["nh"]
    for i, s in enumerate(ref["nh_seed"]):
        for uc in (0, 1):
            for k in range(1, 5):
                got = np.array([L.orc_noise_hash(C.c_uint64(int(s)), C.c_uint64(idx), uc, k) for idx in range(256)], np.int8)
                assert np.array_equal(got, nh[i, uc, k - 1]), (i, uc, k)
    # the bulk generator is the same function
    assert np.array_equal(orc.fill_noise(256, int(ref["nh_seed"][1]), True, 4), nh[1, 1, 3])
    # CLT noise of k = 4 ternary draws lies in [-4, 4] with variance 8/3
    big = orc.fill_noise(200000, 12345, True, 4).astype(np.float64)
    assert big.min() >= -4 and big.max() <= 4 and abs(big.var() - 8 / 3) < 0.05


def test_ternary_init_matches_reference(ref):
    for i, (seed, rows, cols) in enumerate([(0x1000, 8, 512), (0x3005, 4, 1024), (0x7000, 16, 256)]):
        assert np.array_equal(orc.init_rand_ternary(rows * cols, seed), ref["init"][i][: rows * cols])
        assert ref["init_scale"][i] == np.float32(1.0) / np.sqrt(np.float32(cols))


def test_product_host_rng_matches_reference(ref):
    """The numpy generators the product uses for synthetic inputs are the same streams."""
    from bitnet_nvfp4_b200 import synth
    for i, s in enumerate(ref["sm_seed"]):
        assert np.array_equal(synth.splitmix64_stream(int(s), 16), ref["sm_out"][i])
    assert np.array_equal(synth.init_rand_ternary((8, 512), 0x1000).reshape(-1), ref["init"][0])
    assert np.array_equal(synth.ternary_from_u64(ref["tern_in"]), ref["tern"])


def test_fitness_shaping_matches_reference(ref):
    for mode in range(3):
        got = orc.shape_pair_weights(ref["fit"], mode, 3.0)
        assert np.array_equal(got, ref["shaped"][mode]), mode


def test_library_host_shaping_matches_reference(ref):
    """bnf4_shape_pair_weights is a host function of the product library: it runs without a GPU."""
    from bitnet_nvfp4_b200 import host
    for mode in range(3):
        got = host.shape_pair_weights(ref["fit"].copy(), mode, 3.0)
        assert np.array_equal(got, ref["shaped"][mode]), mode


def test_cross_entropy_matches_reference_host(ref):
    logits, bias, noise = ref["ce_logits"], ref["ce_bias"], ref["ce_noise"]
    for i in range(len(ref["ce"])):
        tot, row = orc.cross_entropy_sum(logits[i:i + 1], bias, noise, -0.125, ref["ce_y"][i:i + 1].astype(np.uint8))
        assert abs(row[0] - ref["ce"][i]) <= 1e-6 * abs(ref["ce"][i])


def test_model_size_helpers(ref):
    assert int(ref["nparams"][0]) == 256 * 512 + 512 * 512 + 4 * (3 * 512 * 512 + 512) + 4 * 2 * 512 * 1024 + 256 * 512 + 256 + 4 + 128 * 512
    assert list(ref["fused_cols"]) == [(3 * h + 1 + 31) & ~31 for h in (128, 512, 2048)]


# ------------------------------------------------------------------------------------------------ number formats
def test_e2m1_matches_cutlass(codec):
    L = orc.lib()
    import ctypes as C
    got = np.array([L.orc_e2m1_encode(C.c_float(float(x))) for x in codec["e2m1_x"]], np.uint8)
    assert np.array_equal(got, codec["e2m1_code"])
    # decode table
    assert [L.orc_e2m1_decode(c) for c in range(8)] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert L.orc_e2m1_decode(0xB) == -1.5


def test_ue4m3_matches_cutlass(codec):
    L = orc.lib()
    import ctypes as C
    xs = codec["ue4m3_x"]
    got = np.array([L.orc_ue4m3_encode(C.c_float(float(x))) for x in xs], np.uint8)
    assert np.array_equal(got, codec["ue4m3_byte"])
    back = np.array([L.orc_ue4m3_decode(int(b)) for b in got], np.float32)
    assert np.array_equal(back, codec["ue4m3_value"])
    # facts the reference's quantiser relies on
    assert L.orc_ue4m3_encode(C.c_float(1 / 6)) == 0x23 and L.orc_ue4m3_decode(0x23) == 0.171875
    assert L.orc_ue4m3_encode(C.c_float(0.0009)) == 0 and L.orc_ue4m3_encode(C.c_float(1e9)) == 0x7E


def test_scale_factor_layout_matches_cutlass(codec):
    L = orc.lib()
    for rows, K, nbytes, probe in codec["sf_shapes"]:
        rows, K = int(rows), int(K)
        assert orc.sf_bytes(rows, K) == int(nbytes)
        ref_off = codec[f"sf_off_{rows}x{K}"]
        r = np.arange(rows)[:, None]
        kb = np.arange(K // 16)[None, :]
        kt = ((K + 15) // 16 + 3) // 4
        mine = ((r // 128) * kt + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
        assert np.array_equal(mine.astype(np.uint32), ref_off)
        assert L.orc_sf_offset(rows - 1, K // 16 - 1, K) == int(probe)  # the B-operand layout is the same atom
        for rr, kk in [(0, 0), (rows - 1, K // 16 - 1), (rows // 2, (K // 16) // 2)]:
            assert L.orc_sf_offset(rr, kk, K) == int(ref_off[rr, kk])


def test_product_quantiser_table_matches_oracle():
    """The (amax, |v|) -> code table the CUDA kernels use is built by a host function of the library; rebuild it from the
    oracle's arithmetic (amax/6 -> ue4m3, v/scale -> e2m1) and compare through the quantised output of ternary/int8 rows."""
    rng = np.random.default_rng(3)
    x = rng.integers(-127, 128, (64, 256)).astype(np.int8)
    codes, sf = orc.quantize_rowmajor(x)
    L = orc.lib()
    import ctypes as C
    for r in (0, 17, 63):
        for kb in (0, 7, 15):
            blk = x[r, kb * 16:(kb + 1) * 16].astype(np.float32)
            amax = np.abs(blk).max()
            s = L.orc_ue4m3_decode(L.orc_ue4m3_encode(C.c_float(float(amax / np.float32(6.0))))) if amax > 0 else 1.0
            assert sf[L.orc_sf_offset(r, kb, 256)] == (L.orc_ue4m3_encode(C.c_float(float(amax / np.float32(6.0)))) if amax > 0 else 0x38)
            for i in range(16):
                e = r * 256 + kb * 16 + i
                c = (codes[e // 2] >> (4 * (e & 1))) & 0xF
                assert c == L.orc_e2m1_encode(C.c_float(float(np.float32(blk[i]) / np.float32(s))))


def test_f16_conversion_matches_numpy():
    L = orc.lib()
    import ctypes as C
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in [1e-8, 1e-6, 1e-4, 1, 100, 70000]])
    with np.errstate(over="ignore"):
        ref16 = xs.astype(np.float16)
    for x, h in zip(xs, ref16.view(np.uint16)):
        assert L.orc_f32_to_f16(C.c_float(float(x))) == int(h)
    for h in rng.integers(0, 0x7C00, 2000):
        assert L.orc_f16_to_f32(int(h)) == np.float32(np.uint16(h).view(np.float16))


# ------------------------------------------------------------------------------------------------ oracle self-consistency
def test_quantised_weight_biases_documented_in_the_reference_math():
    """Ternary weights quantise to +-1.03125 (scale 0.171875, code 6), an all-zero block to scale 1.0 / codes 0."""
    w = np.zeros((1, 32), np.int8)
    w[0, :16] = [1, -1, 0, 1] * 4
    codes, sf = orc.quantize_rowmajor(w)
    assert sf[0] == 0x23 and sf[1] == 0x38
    assert all(((b & 0xF) in (0, 7, 0xF)) and ((b >> 4) in (0, 7, 0xF)) for b in codes[:8])
    assert np.all(codes[8:] == 0)


def test_gemm_oracle_is_the_dequantised_product():
    rng = np.random.default_rng(5)
    m, n, k = 24, 40, 128
    x = np.clip(np.rint(rng.standard_normal((m, k)) * 40), -127, 127).astype(np.int8)
    w = rng.integers(-1, 2, (n, k)).astype(np.int8)
    a, sfa = orc.quantize_rowmajor(x)
    b, sfb = orc.quantize_rowmajor(w)
    L = orc.lib()

    def dequant(codes, sf, rows):
        out = np.zeros((rows, k))
        for r in range(rows):
            for j in range(k):
                e = r * k + j
                c = (codes[e // 2] >> (4 * (e & 1))) & 0xF
                out[r, j] = L.orc_e2m1_decode(int(c)) * L.orc_ue4m3_decode(int(sf[L.orc_sf_offset(r, j // 16, k)]))
        return out

    ref = 0.25 * dequant(a, sfa, m) @ dequant(b, sfb, n).T
    got = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, 0.25)
    assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()
    c = rng.standard_normal((m, n)).astype(np.float32)
    got2 = orc.gemm_nvfp4(a, b, sfa, sfb, m, n, k, 0.25, 0.5, c)
    assert np.abs(got2 - (ref + 0.5 * c)).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("rank,heads", [(0, 1), (1, 2), (4, 2)])
def test_layer_major_equals_token_major(rank, heads):
    """Inverting the loop order (all tokens of a layer at once) changes no value: only the recurrent state couples time steps."""
    from bitnet_nvfp4_b200 import population, synth
    cfg = population.Config(hidden=128, layers=2, seq=12, batch=3, heads=heads, rank=max(rank, 1), max_pairs=1)
    w = synth.init_weights(cfg)
    tok, tgt = synth.sample_batch(synth.zipf_corpus(1 << 14), cfg.batch, cfg.seq, 7)
    ocfg = {k: getattr(cfg, k) for k in "vocab hidden layers mlp_mult seq batch heads rank sigma_shift use_clt clt_k method act_scale "
                                        "mlp_act_scale ln_scale residual_scale mlp_residual_scale eps".split()}
    ocfg["rank"] = rank
    om = orc.OracleModel(ocfg, w)
    for anti in (0, 1, -1):
        a = om.forward(tok, tgt, 99, anti)
        b = om.forward(tok, tgt, 99, anti, token_major=True)
        assert a == b
    assert om.forward(tok, tgt, 99, 1) != om.forward(tok, tgt, 99, -1)


def test_synthetic_tokens_are_zipf():
    from bitnet_nvfp4_b200 import synth
    c = synth.zipf_corpus(1 << 18, 1.1, 123)
    counts = np.bincount(c, minlength=256).astype(np.float64)
    p = np.arange(1, 257) ** -1.1
    p /= p.sum()
    assert abs(counts[0] / counts.sum() - p[0]) < 0.01 and counts[0] > counts[1] > counts[5] > counts[50]
    tok, tgt = synth.sample_batch(c, 32, 128, 123)
    assert tok.shape == (32, 128) and np.array_equal(tok[:, 1:], tgt[:, :-1])


def test_batch_sampler_matches_reference_dataset():
    """synth.sample_batch == the reference's ByteDataset::sample_batch_packed (src/dataset.cpp:39-54) on the same corpus bytes."""
    from bitnet_nvfp4_b200 import synth
    g = np.load(GOLD / "ref_host.npz")
    corpus = synth.zipf_corpus(1 << 16, 1.1, 123)
    for i, sd in enumerate(g["sb_seed"]):
        tok, tgt = synth.sample_batch(corpus, 32, 128, int(sd))
        assert np.array_equal(tok, g["sb_tok"][i]) and np.array_equal(tgt, g["sb_tgt"][i])


def test_gaussian_map_is_standard_normal():
    """The oracle's N(0,1) map for the fp32 inputs of the single-GEMM configuration (Box-Muller on the reference's counter
    functions): moments of a standard normal, and the ternarisation threshold 0.008 on 0.02 N(0,1) latents leaves
    P(|z| <= 0.4) = 31 % zeros."""
    z = orc.gaussian_f32(1, 7, 1 << 18)
    assert abs(z.mean()) < 5e-3 and abs(z.std() - 1.0) < 5e-3 and abs((z ** 4).mean() - 3.0) < 0.1
    lat = orc.gaussian_f32(1, 0x57, 512 * 512, 0.02)
    assert abs((np.abs(lat) <= 0.008).mean() - 0.3108) < 5e-3
    assert np.array_equal(orc.gaussian_f32(1, 7, 64), z[:64])   # counter-based: a prefix is a prefix


def test_direct_fp32_quantiser_edge_cases():
    x = np.zeros((3, 32), np.float32)
    x[1, :16] = 1e-5                      # scale underflows ue4m3 -> 1.0, codes 0
    x[2, :16] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
    codes, sf = orc.quantize_direct_f32(x)
    assert sf[orc.lib().orc_sf_offset(0, 0, 32)] == 0x38 and sf[orc.lib().orc_sf_offset(1, 0, 32)] == 0x38
    assert not codes[:32].any()
    # row 2: max 6 -> scale 1.0; ties go to the even code: 0.25->0, 0.75->1.0, 1.25->1.0, 1.75->2.0, 2.5->2.0, 3.5->4.0, 5->4.0
    row = codes[32:40]
    nib = np.stack([row & 15, row >> 4], 1).reshape(-1)
    assert list(nib) == [0, 2, 2, 4, 4, 6, 6, 7, 8, 10, 10, 12, 12, 14, 14, 15]

"""CPU tests of the drop-in boundary: libbnf4.so loads without a GPU, exports every function include/bnf4.h declares and
every C++ name of the reference's two kernel-entry headers, and fails loudly (error code + message, no crash, no CPU
fallback) when a compute entry point is called without a device."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def L():
    from bitnet_nvfp4_b200 import lib
    return lib.load()


def declared_functions():
    text = (ROOT / "include" / "bnf4.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bnf4_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported(L):
    names = declared_functions()
    assert len(names) >= 55
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_reference_cpp_names_are_exported():
    """Every function the reference declares in namespaces bitnet_cuda / efla_lm_cuda has a definition in the library."""
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", str(ROOT / "bitnet_nvfp4_b200" / "libbnf4.so")], capture_output=True, text=True,
                         check=True).stdout
    have = set(re.findall(r"\b((?:bitnet_cuda|efla_lm_cuda)::[a-z0-9_]+)\(", out))
    expected_bitnet = """gemm_ternary gemm_ternary_act_quant gemm_ternary_gelu_quant gemm_ternary_lora_act_quant gemm_ternary_sparse_act_quant
        gemm_ternary_f head_gemm_cross_entropy gemm_ternary_f_noise gemm_ternary_f_noise_tiled gemm_qkvb_fused pack_ternary_i2
        pack_ternary_i2_bitnet init_i2_lut gemm_ternary_f_i2 gemm_ternary_f_i2_noise gemm_ternary_f_i2_bitnet gemm_ternary_f_i2_bitnet_noise
        gemm_ternary_f_cutlass gemm_ternary_lora_f gemm_ternary_sparse_f lora_compute_t lora_add sparse_add activation_quantize
        activation_quantize_nvfp4 embedding_lookup_noise_quantize_nvfp4 add_pos_gelu_quantize_nvfp4 gelu_quantize_nvfp4 absmean_norm_q_nvfp4
        add_scaled_to_int8_absmean_norm_q_nvfp4 embed_update_plain embed_update_lora embed_update_sparse nvfp4_sfa_bytes nvfp4_sfb_bytes
        nvfp4_init nvfp4_set_schedule nvfp4_set_quant_mode nvfp4_set_stage_count nvfp4_set_decomposition nvfp4_set_verbose nvfp4_set_splits
        nvfp4_prepare_gemm nvfp4_quantize_a nvfp4_quantize_b nvfp4_quantize_wqkv_fused split_qkvb_fused gemm_ternary_f_nvfp4
        gemm_ternary_f_nvfp4_gelu_i8""".split()
    expected_efla = """embedding_lookup_noise add_pos_gelu_quantize add_pos_gelu gelu_quantize add_scaled add_scaled_i8 add_scaled_to_int8
        add_scaled_to_int8_absmean_norm_q layernorm_quantize absmean_norm_q init_shadow_from_weights fill_pair_seeds compute_z_sumsq
        update_inv_rms update_shadow_ternary update_shadow_ternary_device update_shadow_ternary_device_packed
        update_shadow_ternary_device_packed_bitnet efla_step efla_step_half efla_step_qkv_fused efla_step_half_qkv_fused efla_step_fused
        efla_step_fused_half efla_step_lowrank cross_entropy_loss fill_ternary_noise fill_ternary_noise_batched fill_float_noise""".split()
    missing = [f"bitnet_cuda::{n}" for n in expected_bitnet if f"bitnet_cuda::{n}" not in have]
    missing += [f"efla_lm_cuda::{n}" for n in expected_efla if f"efla_lm_cuda::{n}" not in have]
    assert not missing, missing


def test_descriptor_layouts_match(L):
    from bitnet_nvfp4_b200 import lib
    a, b = C.c_int(0), C.c_int(0)
    assert L.bnf4_struct_sizes(C.byref(a), C.byref(b)) == 0
    assert a.value == C.sizeof(lib.RowQuantDesc) and b.value == C.sizeof(lib.GemmDesc)


def test_size_helpers(L):
    # scale bytes = ceil(rows/128)*128 * ceil(K/64)*4 (facts recorded from the CUTLASS layout)
    assert [L.bnf4_nvfp4_sfa_bytes(m, 1, k) for m, k in [(32, 512), (32, 1024), (4096, 512), (1, 512)]] == [4096, 8192, 131072, 4096]
    assert L.bnf4_nvfp4_sfb_bytes(1, 1568, 512) == 53248
    assert L.bnf4_nvfp4_matrix_bytes(4096, 512) == 4096 * 512 // 2


def test_invalid_arguments_are_reported(L):
    assert L.bnf4_gemm_ternary_f_nvfp4(1024, 1024, 1024, 1024, 16, 16, 48, 1.0, 0.0, None, 1024, None) == 1  # k % 64 != 0
    assert b"multiple of 64" in L.bnf4_last_error()
    assert L.bnf4_set_option(b"no_such_option", 1) == 1


def test_no_cpu_fallback_without_a_gpu(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    # a well-formed call must fail with an error code and a message, not compute anything on the host
    rc = L.bnf4_gemm_ternary_f_nvfp4(1024, 2048, 4096, 8192, 128, 128, 64, 1.0, 0.0, None, 16384, None)
    assert rc != 0 and len(L.bnf4_last_error()) > 0
    from bitnet_nvfp4_b200 import population
    with pytest.raises(Exception):
        population.PopulationModel(population.Config(hidden=128, layers=1, seq=8, batch=2, heads=2, max_pairs=2))


def test_reference_driver_links_against_the_library():
    """oracle/_ref/libref_host.so is the reference's src/train_efla_lm.cpp linked with --no-undefined against libbnf4.so."""
    so = ROOT / "oracle" / "_ref" / "libref_host.so"
    if not so.exists():
        pytest.skip("oracle/_ref not built (needs the reference tree)")
    lib = C.CDLL(str(so))
    lib.ref_mix.restype = C.c_uint64
    lib.ref_mix.argtypes = [C.c_uint64, C.c_uint64]
    import oracle_lib as orc
    assert lib.ref_mix(1, 2) == orc.mix(1, 2)
    assert hasattr(lib, "ref_train")

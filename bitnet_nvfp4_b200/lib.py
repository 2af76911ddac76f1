"""ctypes binding of libbnf4.so (the C ABI declared in include/bnf4.h).

The library is CUDA-only. Importing this module never falls back to a CPU path: if the shared object
is missing, `load()` raises; if no sm_100 GPU is present, every compute call returns an error code
that `check()` turns into an exception.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libbnf4.so"
_lib = None

c_void_p, c_int, c_float, c_size_t, c_ll = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_longlong


class RowQuantDesc(C.Structure):
    """bnf4_rowquant_desc"""

    _fields_ = [
        ("rows", c_int), ("cols_in", c_int), ("cols_out", c_int),
        ("rows_per_member", c_int), ("anti_fixed", c_int), ("sigma", c_float), ("c_rank", c_float),
        ("in_i8", c_void_p), ("in_f32", c_void_p), ("ld_in", c_int), ("inout_i8", c_void_p),
        ("wq", c_void_p), ("wk", c_void_p), ("wv", c_void_p), ("wb", c_void_p),
        ("q_scale", c_float), ("k_scale", c_float), ("v_scale", c_float), ("b_scale", c_float),
        ("tokens", c_void_p), ("token_stride", c_int), ("row_mod", c_int),
        ("emb_w", c_void_p), ("emb_noise", c_void_p), ("embA", c_void_p), ("embB", c_void_p),
        ("embA_pair_stride", c_ll), ("embB_pair_stride", c_ll), ("rank", c_int),
        ("pos", c_void_p), ("pos_noise", c_void_p), ("pos_mod", c_int), ("noise_pair_stride", c_ll),
        ("act_mode", c_int), ("act_scale", c_float), ("add_scale", c_float), ("norm_scale", c_float),
        ("out_q", c_void_p), ("ld_q", c_int), ("out_codes", c_void_p), ("out_sf", c_void_p),
        ("tvec", c_void_p), ("tvec_pair_stride", c_ll), ("nvec", c_int), ("t_out", c_void_p),
        ("vec_ok", c_int), ("vec_ok_q", c_int), ("gather_rows", c_int), ("in_f16", c_int),
    ]


class GemmDesc(C.Structure):
    """bnf4_gemm_desc"""

    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("sfa", c_void_p), ("sfb", c_void_p),
        ("m", c_int), ("n", c_int), ("k", c_int), ("alpha", c_float), ("beta", c_float),
        ("c", c_void_p), ("ldc", c_int), ("d", c_void_p), ("ldd", c_int),
        ("epilogue", c_int), ("act_scale", c_float), ("d_i8", c_void_p), ("ld_i8", c_int),
        ("d_codes", c_void_p), ("d_sf", c_void_p),
        ("rank", c_int), ("rows_per_member", c_int), ("lora_t", c_void_p), ("t_stride", c_int),
        ("lora_A", c_void_p), ("lora_A_pair_stride", c_ll), ("lora_scale", c_float), ("group_cols", c_int),
        ("next_tvec", c_void_p), ("next_tvec_pair_stride", c_ll), ("next_nvec", c_int), ("next_t", c_void_p),
        ("resid", c_void_p), ("ld_resid", c_int), ("add_scale", c_float),
        ("d_f16", c_void_p), ("ld_f16", c_int), ("n_f16", c_int),
    ]


class EflaDesc(C.Structure):
    """bnf4_efla_desc"""

    _fields_ = [
        ("state", c_void_p), ("state_fp16", c_int),
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("beta_raw", c_void_p),
        ("ld_qkv", c_int), ("ld_beta", c_int),
        ("beta_bias", c_float), ("beta_bias_seq", c_void_p), ("seqs_per_bias", c_int),
        ("hidden", c_int), ("heads", c_int), ("seqs", c_ll), ("T", c_int), ("method", c_int), ("eps", c_float),
        ("out", c_void_p), ("ld_out", c_int), ("variant", c_int), ("qkv_f16", c_int), ("out_f16", c_int),
    ]


class NoiseDesc(C.Structure):
    """bnf4_noise_desc"""

    _fields_ = [("out", c_void_p), ("n", c_size_t), ("seed", C.c_uint64)]


_I8P = c_void_p  # device pointers travel as integers
c_u64 = C.c_uint64

_PROTOS = {
    # name: (restype, argtypes)
    "bnf4_last_error": (C.c_char_p, []),
    "bnf4_version": (C.c_char_p, []),
    "bnf4_launch_count": (C.c_ulonglong, []),
    "bnf4_set_option": (c_int, [C.c_char_p, c_int]),
    "bnf4_device_error": (c_int, [c_void_p, C.POINTER(c_int)]),
    "bnf4_struct_sizes": (c_int, [C.POINTER(c_int), C.POINTER(c_int)]),
    "bnf4_nvfp4_matrix_bytes": (c_size_t, [c_int, c_int]),
    "bnf4_nvfp4_sfa_bytes": (c_size_t, [c_int, c_int, c_int]),
    "bnf4_nvfp4_sfb_bytes": (c_size_t, [c_int, c_int, c_int]),
    "bnf4_rowquant": (c_int, [c_int, C.POINTER(RowQuantDesc), c_void_p]),
    "bnf4_nvfp4_quantize_a": (c_int, [_I8P, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "bnf4_nvfp4_quantize_f32": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "bnf4_nvfp4_quantize_b": (c_int, [_I8P, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "bnf4_nvfp4_quantize_wqkv_fused": (c_int, [_I8P, _I8P, _I8P, _I8P, c_int, c_int, c_int, c_int, c_float, c_float,
                                               c_float, c_float, c_void_p, c_void_p, c_void_p]),
    "bnf4_embedding_lookup_noise_quantize_nvfp4": (c_int, [c_void_p, c_int, _I8P, _I8P, c_int, c_int, c_float, c_int,
                                                           _I8P, c_void_p, c_void_p, c_void_p]),
    "bnf4_add_pos_gelu_quantize_nvfp4": (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, _I8P, c_void_p, c_void_p,
                                                 c_void_p]),
    "bnf4_activation_quantize_nvfp4": (c_int, [c_void_p, c_int, c_int, c_int, c_int, _I8P, c_void_p, c_void_p, c_void_p]),
    "bnf4_gelu_quantize_nvfp4": (c_int, [c_void_p, c_int, c_int, c_int, c_float, _I8P, c_void_p, c_void_p, c_void_p]),
    "bnf4_absmean_norm_q_nvfp4": (c_int, [_I8P, c_int, c_int, c_int, c_float, _I8P, c_void_p, c_void_p, c_void_p]),
    "bnf4_add_scaled_to_int8_absmean_norm_q_nvfp4": (c_int, [_I8P, c_void_p, c_int, c_int, c_int, c_float, c_float, _I8P,
                                                             c_void_p, c_void_p, c_void_p]),
    "bnf4_gemm_nvfp4_ex": (c_int, [C.POINTER(GemmDesc), c_void_p]),
    "bnf4_gemm_ternary_f_nvfp4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                                          c_void_p, c_void_p, c_void_p]),
    "bnf4_gemm_ternary_f_nvfp4_gelu_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                                  c_float, c_void_p, c_float, _I8P, c_void_p]),
    "bnf4_nvfp4_prepare_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                                        c_void_p, c_void_p, c_void_p]),
    "bnf4_gemm_ternary_f": (c_int, [_I8P, _I8P, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "bnf4_lora_compute_t": (c_int, [_I8P, _I8P, c_int, c_int, c_int, c_void_p, c_void_p]),
    "bnf4_lora_add": (c_int, [c_void_p, _I8P, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "bnf4_split_qkvb_fused": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                      c_void_p]),
    "bnf4_efla_scan": (c_int, [C.POINTER(EflaDesc), c_void_p]),
    "bnf4_efla_step_half_qkv_fused": (c_int, [c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_float, c_void_p,
                                              c_void_p]),
    "bnf4_efla_step_qkv_fused": (c_int, [c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_float, c_void_p,
                                         c_void_p]),
    "bnf4_efla_step": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                               c_float, c_void_p, c_void_p]),
    "bnf4_cross_entropy_loss": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p,
                                        c_void_p]),
    "bnf4_cross_entropy_population": (c_int, [c_void_p, c_int, c_void_p, _I8P, c_float, c_void_p, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p]),
    "bnf4_fill_ternary_noise": (c_int, [_I8P, c_size_t, c_u64, c_int, c_int, c_void_p]),
    "bnf4_fill_ternary_noise_batched": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "bnf4_fill_float_noise": (c_int, [c_void_p, c_int, c_u64, c_int, c_int, c_void_p]),
    "bnf4_init_shadow_from_weights": (c_int, [_I8P, c_void_p, c_int, c_void_p]),
    "bnf4_fill_pair_seeds": (c_int, [c_u64, c_u64, c_int, c_void_p, c_void_p]),
    "bnf4_compute_z_sumsq": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "bnf4_compute_z_sumsq_static": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "bnf4_compute_z_sumsq_lowrank": (c_int, [c_void_p, _I8P, c_ll, _I8P, c_ll, c_int, c_int, c_int, c_int, c_float,
                                             c_void_p, c_void_p, c_void_p]),
    "bnf4_update_inv_rms": (c_int, [c_void_p, c_void_p, c_int, c_float, c_float, c_int, c_void_p, c_void_p]),
    "bnf4_update_shadow_ternary_device": (c_int, [_I8P, c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_void_p]),
    "bnf4_update_shadow_ternary": (c_int, [_I8P, c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_void_p]),
    "bnf4_update_vector_device": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_void_p]),
    "bnf4_add_scaled": (c_int, [c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "bnf4_shape_pair_weights": (c_int, [c_void_p, c_int, c_int, c_float]),
}


class Bnf4Error(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def register(protos: dict) -> None:
    """Add prototypes (used by the other binding modules of this package)."""
    _PROTOS.update(protos)
    if _lib is not None:
        _apply(_lib, protos)


def _apply(lib, protos) -> None:
    for name, (res, args) in protos.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing: fail loudly
        fn.restype = res
        fn.argtypes = args


def load():
    """Load libbnf4.so. Raises if the library has not been built (python -m bitnet_nvfp4_b200.build)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise Bnf4Error(f"{_LIB_PATH} is missing: build it with `python -m bitnet_nvfp4_b200.build` "
                            "(there is no CPU fallback)")
        lib = C.CDLL(str(_LIB_PATH))
        _apply(lib, _PROTOS)
        a, b = c_int(0), c_int(0)
        lib.bnf4_struct_sizes(C.byref(a), C.byref(b))
        if a.value != C.sizeof(RowQuantDesc) or b.value != C.sizeof(GemmDesc):
            raise Bnf4Error(f"descriptor layout mismatch: C {a.value}/{b.value} vs ctypes "
                            f"{C.sizeof(RowQuantDesc)}/{C.sizeof(GemmDesc)}")
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise Bnf4Error(f"libbnf4 error {rc}: {load().bnf4_last_error().decode()}")

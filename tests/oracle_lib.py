"""numpy front-end of the CPU oracle (oracle/liboracle.so). Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
_lib = None

vp, ci, cf, cu64, csz = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_size_t


class ModelCfg(C.Structure):
    _fields_ = [(n, ci) for n in "vocab hidden layers mlp_mult seq batch heads rank sigma_shift use_clt clt_k method".split()] + \
               [(n, cf) for n in "act_scale mlp_act_scale ln_scale residual_scale mlp_residual_scale eps".split()]


class ModelWeights(C.Structure):
    _fields_ = [(n, vp) for n in "emb win wq wk wv wbeta ff1 ff2 head head_bias beta_bias pos".split()]


class ModelTaps(C.Structure):
    _fields_ = [(n, vp) for n in "emb_q inproj x_q0 qkv attn_y ff1_q ff2_y x_q y_q logits".split()]


def build_oracle() -> Path:
    so = ORACLE_DIR / "liboracle.so"
    srcs = [ORACLE_DIR / "oracle.cpp", ORACLE_DIR / "model.cpp", ORACLE_DIR / "oracle.h"]
    if not so.exists() or any(s.stat().st_mtime > so.stat().st_mtime for s in srcs):
        subprocess.run(["make", "-C", str(ORACLE_DIR), "liboracle.so"], check=True, capture_output=True)
    return so


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(str(build_oracle()))
        L.orc_mix.restype = cu64
        L.orc_mix.argtypes = [cu64, cu64]
        L.orc_splitmix64.restype = cu64
        L.orc_splitmix64.argtypes = [C.POINTER(cu64)]
        L.orc_noise_hash.argtypes = [cu64, cu64, ci, ci]
        L.orc_ternary_from_u64.argtypes = [cu64]
        L.orc_e2m1_encode.argtypes = [cf]
        L.orc_e2m1_decode.restype = cf
        L.orc_ue4m3_encode.argtypes = [cf]
        L.orc_ue4m3_decode.restype = cf
        L.orc_sf_offset.restype = csz
        L.orc_sf_bytes.restype = csz
        L.orc_f32_to_f16.argtypes = [cf]
        L.orc_f16_to_f32.restype = cf
        L.orc_cross_entropy_sum.restype = C.c_double
        L.orc_compute_z_sumsq.restype = cf
        L.orc_compute_z_sumsq_lowrank.restype = cf
        L.orc_sumsq.restype = cf
        L.orc_update_inv_rms.restype = cf
        L.orc_model_create.restype = vp
        L.orc_model_forward.restype = C.c_double
        L.orc_model_forward_token_major.restype = C.c_double
        _lib = L
    return _lib


def P(a):
    """pointer to a numpy array (or None)"""
    return None if a is None else a.ctypes.data_as(vp)


def mix(a: int, b: int) -> int:
    return lib().orc_mix(cu64(a & (2**64 - 1)), cu64(b & (2**64 - 1)))


def sf_bytes(rows: int, K: int) -> int:
    return lib().orc_sf_bytes(rows, K)


def fill_noise(n: int, seed: int, use_clt=True, clt_k=4) -> np.ndarray:
    out = np.zeros(n, np.int8)
    lib().orc_fill_noise(P(out), csz(n), cu64(seed), int(use_clt), clt_k)
    return out


def init_rand_ternary(n: int, seed: int) -> np.ndarray:
    out = np.zeros(n, np.int8)
    lib().orc_init_rand_ternary(P(out), csz(n), cu64(seed))
    return out


def quantize_rowmajor(x: np.ndarray, k_out: int | None = None):
    rows, k_in = x.shape
    k_out = k_out or k_in
    codes = np.zeros(rows * k_out // 2, np.uint8)
    sf = np.zeros(sf_bytes(rows, k_out), np.uint8)
    lib().orc_quantize_rowmajor(P(np.ascontiguousarray(x)), rows, k_in, k_out, P(codes), P(sf))
    return codes, sf


def gaussian_f32(seed: int, tag: int, n: int, scale: float = 1.0) -> np.ndarray:
    """The oracle's N(0,1) map (Box-Muller on the reference's counter functions), times `scale`, as fp32."""
    out = np.zeros(n, np.float32)
    lib().orc_gaussian_f32(cu64(seed), cu64(tag), csz(n), cf(scale), P(out))
    return out


def quantize_direct_f32(x: np.ndarray, k_out: int | None = None):
    x = np.ascontiguousarray(x, np.float32)
    rows, k_in = x.shape
    k_out = k_out or k_in
    codes = np.zeros(rows * k_out // 2, np.uint8)
    sf = np.zeros(sf_bytes(rows, k_out), np.uint8)
    lib().orc_quantize_direct_f32(P(x), rows, k_in, k_out, P(codes), P(sf))
    return codes, sf


def quantize_wqkv_fused(wq, wk, wv, wb, hidden: int, scale: float):
    rows = 3 * hidden + 1
    codes = np.zeros(rows * hidden // 2 + 8, np.uint8)
    sf = np.zeros(sf_bytes(rows, hidden), np.uint8)
    lib().orc_quantize_wqkv_fused(P(wq), P(wk), P(wv), P(wb), hidden, hidden, cf(scale), cf(scale), cf(scale), cf(scale),
                                  P(codes), P(sf))
    return codes, sf


def _outs(rows, cols):
    return (np.zeros((rows, cols), np.int8), np.zeros(rows * cols // 2, np.uint8), np.zeros(sf_bytes(rows, cols), np.uint8))


def embedding_quant(tokens, token_stride, emb_w, emb_noise, hidden, rows, noise_scale, anti):
    q, codes, sf = _outs(rows, hidden)
    lib().orc_embedding_quant(P(tokens), token_stride, P(emb_w), P(emb_noise), hidden, rows, cf(noise_scale), anti, P(q),
                              P(codes), P(sf))
    return q, codes, sf


def embedding_lowrank_quant(tokens, token_stride, emb_w, A, B, rank, hidden, rows, scale):
    q, codes, sf = _outs(rows, hidden)
    lib().orc_embedding_lowrank_quant(P(tokens), token_stride, P(emb_w), P(A), P(B), rank, hidden, rows, cf(scale), P(q),
                                      P(codes), P(sf))
    return q, codes, sf


def add_pos_gelu_quant(x, pos, pos_row, act_scale):
    rows, hidden = x.shape
    q, codes, sf = _outs(rows, hidden)
    pr = None if pos_row is None else np.ascontiguousarray(pos_row, np.int32)
    lib().orc_add_pos_gelu_quant(P(x), P(pos), P(pr), hidden, rows, cf(act_scale), P(q), P(codes), P(sf))
    return q, codes, sf


def activation_quant(x, cols_out, mode, act_scale=1.0):
    rows, cols_in = x.shape
    q, codes, sf = _outs(rows, cols_out)
    lib().orc_activation_quant(P(x), rows, cols_in, cols_out, mode, cf(act_scale), P(q), P(codes), P(sf))
    return q, codes, sf


def absmean_norm_q(x8, add_in, add_scale, norm_scale):
    """x8 is updated in place when add_in is given."""
    rows, hidden = x8.shape
    q, codes, sf = _outs(rows, hidden)
    lib().orc_absmean_norm_q(P(x8), P(add_in), hidden, rows, cf(add_scale), cf(norm_scale), P(q), P(codes), P(sf))
    return q, codes, sf


def gemm_nvfp4(a, b, sfa, sfb, m, n, k, alpha=1.0, beta=0.0, c=None, gelu_i8=False, act_scale=1.0, ldd=None):
    ldd = ldd or n
    d = np.zeros((m, ldd), np.float32)
    d8 = np.zeros((m, ldd), np.int8)
    lib().orc_gemm_nvfp4(P(a), P(b), P(sfa), P(sfb), m, n, k, cf(alpha), cf(beta), P(c), (c.shape[1] if c is not None else 0),
                         P(d), ldd, int(gelu_i8), cf(act_scale), P(d8))
    return d8 if gelu_i8 else d


def gemm_ternary_f(x, w, scale_x, out_scale):
    batch, cols = x.shape
    rows = w.shape[0]
    out = np.zeros((batch, rows), np.float32)
    lib().orc_gemm_ternary_f(P(x), P(w), P(scale_x), rows, cols, batch, cf(out_scale), P(out))
    return out


def lora_compute_t(x, B, rank):
    batch, cols = x.shape
    t = np.zeros((batch, rank), np.int32)
    lib().orc_lora_compute_t(P(x), P(B), cols, batch, rank, P(t))
    return t


def lora_add(t, A, rows, scale, out):
    batch, rank = t.shape
    lib().orc_lora_add(P(t), P(A), rows, batch, rank, cf(scale), P(out), out.shape[1])
    return out


def efla_step(S, qkv, beta_bias, hidden, heads, method=1, eps=1e-6):
    batch, fused_cols = qkv.shape
    out = np.zeros((batch, hidden), np.float32)
    lib().orc_efla_step_half_qkv_fused(P(S), P(qkv), fused_cols, cf(beta_bias), hidden, heads, batch, method, cf(eps), P(out))
    return out


def efla_scan(qkv, beta_bias_seq, hidden, heads, method=1, eps=1e-6):
    seqs, T, fused_cols = qkv.shape
    out = np.zeros((seqs, T, hidden), np.float32)
    bb = np.ascontiguousarray(beta_bias_seq, np.float32)
    lib().orc_efla_scan(P(qkv), fused_cols, P(bb), hidden, heads, seqs, T, method, cf(eps), P(out))
    return out


def cross_entropy_sum(logits, bias, bias_noise, bns, targets, target_stride=1):
    rows, vocab = logits.shape
    row_loss = np.zeros(rows, np.float32)
    tot = lib().orc_cross_entropy_sum(P(logits), vocab, P(bias), P(bias_noise), cf(bns), P(targets), target_stride, vocab, rows,
                                      P(row_loss))
    return tot, row_loss


def shape_pair_weights(w, mode=2, clip=3.0):
    w = np.ascontiguousarray(w, np.float32).copy()
    lib().orc_shape_pair_weights(P(w), len(w), mode, cf(clip))
    return w


def fill_pair_seeds(base_seed, epoch, pairs):
    out = np.zeros(pairs, np.uint64)
    lib().orc_fill_pair_seeds(cu64(base_seed), cu64(epoch), pairs, P(out))
    return out


def compute_z_sumsq(pair_weights, pair_seeds, salt, n, use_clt=True, clt_k=4):
    Z = np.zeros(n, np.float32)
    ss = lib().orc_compute_z_sumsq(P(pair_weights), P(pair_seeds), cu64(salt), len(pair_weights), n, int(use_clt), clt_k, P(Z))
    return Z, ss


def compute_z_sumsq_lowrank(pair_weights, pair_seeds, salt, rows, cols, rank, cscale, use_clt=True, clt_k=4):
    Z = np.zeros(rows * cols, np.float32)
    ss = lib().orc_compute_z_sumsq_lowrank(P(pair_weights), P(pair_seeds), cu64(salt), len(pair_weights), rows, cols, rank,
                                           int(use_clt), clt_k, cf(cscale), P(Z))
    return Z, ss


def sumsq(Z):
    Z = np.ascontiguousarray(Z, np.float32)
    return lib().orc_sumsq(P(Z), len(Z))


def update_inv_rms(sumsq, rms_ema, use_adaptive, beta, eps, n):
    ema = C.c_float(rms_ema)
    inv = lib().orc_update_inv_rms(cf(sumsq), C.byref(ema), int(use_adaptive), cf(beta), cf(eps), n)
    return inv, ema.value


def update_shadow_ternary(w, shadow, Z, inv_rms, lr, thresh):
    lib().orc_update_shadow_ternary(P(w), P(shadow), P(Z), len(Z), cf(inv_rms), cf(lr), cf(thresh))


def update_vector(v, pair_weights, pair_seeds, salt, rms_ema, use_adaptive, beta, eps, lr, thresh, use_clt=True, clt_k=4):
    """In-place plain update of a float vector; returns the new rms_ema."""
    ema = C.c_float(rms_ema)
    lib().orc_update_vector(P(v), len(v), P(pair_weights), P(pair_seeds), cu64(salt), len(pair_weights), int(use_clt), clt_k,
                            C.byref(ema), int(use_adaptive), cf(beta), cf(eps), cf(lr), cf(thresh))
    return ema.value


class OracleModel:
    """One member's forward on the CPU (oracle/model.cpp)."""

    NAMES = "emb win wq wk wv wbeta ff1 ff2 head head_bias beta_bias pos".split()

    def __init__(self, cfg: dict, weights: dict):
        self.cfg = ModelCfg(**cfg)
        self.arrays = {n: np.ascontiguousarray(weights[n]) for n in self.NAMES}
        self.w = ModelWeights(*[self.arrays[n].ctypes.data for n in self.NAMES])
        self.h = lib().orc_model_create(C.byref(self.cfg), C.byref(self.w))

    def forward(self, tokens, targets, pair_seed, anti, taps: dict | None = None, token_major=False):
        tokens = np.ascontiguousarray(tokens, np.uint8)
        targets = np.ascontiguousarray(targets, np.uint8)
        if token_major:
            return lib().orc_model_forward_token_major(vp(self.h), P(tokens), P(targets), cu64(pair_seed), anti)
        tp = None
        if taps is not None:
            tp = ModelTaps(*[(taps[n].ctypes.data if n in taps else None) for n, _ in ModelTaps._fields_])
        return lib().orc_model_forward(vp(self.h), P(tokens), P(targets), cu64(pair_seed), anti,
                                       C.byref(tp) if tp is not None else None)

    def __del__(self):
        try:
            lib().orc_model_destroy(vp(self.h))
        except Exception:
            pass

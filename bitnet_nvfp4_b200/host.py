"""Host-side mirror of the reference's kernel-entry interface (namespaces bitnet_cuda / efla_lm_cuda of
the reference's src/cuda_kernels.h and src/efla_lm_kernels.h), on torch device tensors.

Function names and argument meaning follow the reference; every call goes through the C ABI of
libbnf4.so on the current CUDA stream. torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as _l

FE_INT8, FE_WQKV, FE_EMBED_DENSE, FE_EMBED_LOWRANK, FE_POS_GELU, FE_POS_GELU_ABSMEAN, FE_ACT, FE_ABSMEAN, FE_ADD_ABSMEAN = range(9)
EPI_F32, EPI_GELU_I8, EPI_GELU_FP4, EPI_ADD_I8, EPI_F16 = range(5)

C_RANK_BASE = 0.6123724356957945  # sqrt(3/8)


def c_rank(rank: int) -> float:
    """Normalisation of a rank-r perturbation: sqrt(3/8)/sqrt(r), evaluated in fp32 like the library does."""
    import numpy as np
    return 0.0 if rank <= 0 else float(np.float32(C_RANK_BASE) / np.sqrt(np.float32(rank)))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def sf_bytes(rows: int, k: int) -> int:
    return _l.load().bnf4_nvfp4_sfa_bytes(rows, 1, k)


def matrix_bytes(rows: int, cols: int) -> int:
    return _l.load().bnf4_nvfp4_matrix_bytes(rows, cols)


def _alloc_q(rows: int, cols: int, device, want_q=True):
    q = torch.zeros((rows, cols), dtype=torch.int8, device=device) if want_q else None
    codes = torch.zeros(matrix_bytes(rows, cols), dtype=torch.uint8, device=device)
    sf = torch.zeros(sf_bytes(rows, cols), dtype=torch.uint8, device=device)
    return q, codes, sf


def device_error() -> int:
    code = C.c_int(0)
    _l.check(_l.load().bnf4_device_error(_stream(), C.byref(code)))
    return code.value


# ------------------------------------------------------------------------------------------ quantisers
def nvfp4_quantize_a(x: torch.Tensor, k_out: int | None = None):
    m, k_in = x.shape
    k_out = k_out or k_in
    _, codes, sf = _alloc_q(m, k_out, x.device, want_q=False)
    _l.check(_l.load().bnf4_nvfp4_quantize_a(_p(x), m, 1, k_in, k_out, _p(codes), _p(sf), _stream()))
    return codes, sf


def nvfp4_quantize_b(w: torch.Tensor, k_out: int | None = None):
    n, k_in = w.shape
    k_out = k_out or k_in
    _, codes, sf = _alloc_q(n, k_out, w.device, want_q=False)
    _l.check(_l.load().bnf4_nvfp4_quantize_b(_p(w), 1, n, k_in, k_out, _p(codes), _p(sf), _stream()))
    return codes, sf


def nvfp4_quantize_f32(x: torch.Tensor, k_out: int | None = None):
    """fp32 rows straight to NVFP4 (no int8 stage)."""
    m, k_in = x.shape
    k_out = k_out or k_in
    _, codes, sf = _alloc_q(m, k_out, x.device, want_q=False)
    _l.check(_l.load().bnf4_nvfp4_quantize_f32(_p(x), m, k_in, k_out, _p(codes), _p(sf), _stream()))
    return codes, sf


def nvfp4_quantize_wqkv_fused(wq, wk, wv, wb, hidden: int, rows_total: int, scale: float):
    codes = torch.zeros(matrix_bytes(rows_total, hidden), dtype=torch.uint8, device=wq.device)
    sf = torch.zeros(sf_bytes(rows_total, hidden), dtype=torch.uint8, device=wq.device)
    _l.check(_l.load().bnf4_nvfp4_quantize_wqkv_fused(_p(wq), _p(wk), _p(wv), _p(wb), 1, hidden, hidden, rows_total, scale,
                                                      scale, scale, scale, _p(codes), _p(sf), _stream()))
    return codes, sf


def embedding_lookup_noise_quantize_nvfp4(tokens_t, token_stride, emb_w, emb_noise, hidden, batch, noise_scale, anti_sign):
    q, codes, sf = _alloc_q(batch, hidden, emb_w.device)
    _l.check(_l.load().bnf4_embedding_lookup_noise_quantize_nvfp4(_p(tokens_t), token_stride, _p(emb_w), _p(emb_noise), hidden,
                                                                  batch, noise_scale, anti_sign, _p(q), _p(codes), _p(sf),
                                                                  _stream()))
    return q, codes, sf


def add_pos_gelu_quantize_nvfp4(x, pos_t, act_scale):
    batch, hidden = x.shape
    q, codes, sf = _alloc_q(batch, hidden, x.device)
    _l.check(_l.load().bnf4_add_pos_gelu_quantize_nvfp4(_p(x), _p(pos_t), hidden, batch, act_scale, _p(q), _p(codes), _p(sf),
                                                        _stream()))
    return q, codes, sf


def activation_quantize_nvfp4(x, cols_out, activation):
    rows, cols_in = x.shape
    q, codes, sf = _alloc_q(rows, cols_out, x.device)
    _l.check(_l.load().bnf4_activation_quantize_nvfp4(_p(x), rows, cols_in, cols_out, activation, _p(q), _p(codes), _p(sf),
                                                      _stream()))
    return q, codes, sf


def gelu_quantize_nvfp4(x, cols_out, act_scale):
    rows, cols_in = x.shape
    q, codes, sf = _alloc_q(rows, cols_out, x.device)
    _l.check(_l.load().bnf4_gelu_quantize_nvfp4(_p(x), rows, cols_in, cols_out, act_scale, _p(q), _p(codes), _p(sf), _stream()))
    return q, codes, sf


def absmean_norm_q_nvfp4(x8, scale):
    batch, hidden = x8.shape
    q, codes, sf = _alloc_q(batch, hidden, x8.device)
    _l.check(_l.load().bnf4_absmean_norm_q_nvfp4(_p(x8), hidden, batch, hidden, scale, _p(q), _p(codes), _p(sf), _stream()))
    return q, codes, sf


def add_scaled_to_int8_absmean_norm_q_nvfp4(x8_inout, y, add_scale, norm_scale):
    batch, hidden = x8_inout.shape
    q, codes, sf = _alloc_q(batch, hidden, y.device)
    _l.check(_l.load().bnf4_add_scaled_to_int8_absmean_norm_q_nvfp4(_p(x8_inout), _p(y), hidden, batch, hidden, add_scale,
                                                                    norm_scale, _p(q), _p(codes), _p(sf), _stream()))
    return q, codes, sf


def rowquant(front_end: int, **kw):
    """Generic row quantiser (bnf4_rowquant); keyword names are the fields of bnf4_rowquant_desc,
    tensors are converted to device pointers."""
    d = _l.RowQuantDesc()
    for k, v in kw.items():
        setattr(d, k, _p(v) if isinstance(v, torch.Tensor) else v)
    _l.check(_l.load().bnf4_rowquant(front_end, C.byref(d), _stream()))


# ------------------------------------------------------------------------------------------ GEMM
def gemm_ternary_f_nvfp4(a, b, sfa, sfb, m, n, k, alpha, beta=0.0, c=None, d=None):
    if d is None:
        d = torch.empty((m, n), dtype=torch.float32, device=a.device)
    _l.check(_l.load().bnf4_gemm_ternary_f_nvfp4(_p(a), _p(b), _p(sfa), _p(sfb), m, n, k, alpha, beta, _p(c), _p(d), _stream()))
    return d


def gemm_ternary_f_nvfp4_gelu_i8(a, b, sfa, sfb, m, n, k, alpha, beta, c, act_scale):
    d = torch.empty((m, n), dtype=torch.int8, device=a.device)
    _l.check(_l.load().bnf4_gemm_ternary_f_nvfp4_gelu_i8(_p(a), _p(b), _p(sfa), _p(sfb), m, n, k, alpha, beta, _p(c), act_scale,
                                                         _p(d), _stream()))
    return d


def gemm_nvfp4_ex(**kw):
    """Full-form GEMM (bnf4_gemm_nvfp4_ex); keyword names are the fields of bnf4_gemm_desc."""
    g = _l.GemmDesc()
    for k, v in kw.items():
        setattr(g, k, _p(v) if isinstance(v, torch.Tensor) else v)
    _l.check(_l.load().bnf4_gemm_nvfp4_ex(C.byref(g), _stream()))


# ------------------------------------------------------------------------------------------ ternary GEMM / rank-r helpers
def gemm_ternary_f(x, w, scale_x, out_scale):
    batch, cols = x.shape
    rows = w.shape[0]
    out = torch.empty((batch, rows), dtype=torch.float32, device=x.device)
    _l.check(_l.load().bnf4_gemm_ternary_f(_p(x), _p(w), _p(scale_x), rows, cols, batch, out_scale, _p(out), _stream()))
    return out


def lora_compute_t(x, B, rank):
    batch, cols = x.shape
    t = torch.empty((batch, rank), dtype=torch.int32, device=x.device)
    _l.check(_l.load().bnf4_lora_compute_t(_p(x), _p(B), cols, batch, rank, _p(t), _stream()))
    return t


def lora_add(t, A, rows, scale, out):
    batch, rank = t.shape
    _l.check(_l.load().bnf4_lora_add(_p(t), _p(A), rows, batch, rank, scale, _p(out), _stream()))
    return out


def split_qkvb_fused(qkv, hidden, beta_bias):
    batch, fused_cols = qkv.shape
    q, k, v = (torch.empty((batch, hidden), dtype=torch.float32, device=qkv.device) for _ in range(3))
    beta = torch.empty(batch, dtype=torch.float32, device=qkv.device)
    _l.check(_l.load().bnf4_split_qkvb_fused(_p(qkv), batch, hidden, fused_cols, _p(q), _p(k), _p(v), _p(beta), beta_bias,
                                             _stream()))
    return q, k, v, beta


# ------------------------------------------------------------------------------------------ EFLA
def efla_scan(**kw):
    """Whole-sequence scan / generic recurrence (bnf4_efla_scan); keyword names are the fields of bnf4_efla_desc."""
    d = _l.EflaDesc()
    for k, v in kw.items():
        setattr(d, k, _p(v) if isinstance(v, torch.Tensor) else v)
    _l.check(_l.load().bnf4_efla_scan(C.byref(d), _stream()))


def efla_step_half_qkv_fused(S, qkv, fused_cols, beta_bias, hidden, batch, method, eps):
    out = torch.empty((batch, hidden), dtype=torch.float32, device=qkv.device)
    _l.check(_l.load().bnf4_efla_step_half_qkv_fused(_p(S), _p(qkv), fused_cols, beta_bias, hidden, batch, method, eps, _p(out),
                                                     _stream()))
    return out


def efla_step_qkv_fused(S, qkv, fused_cols, beta_bias, hidden, batch, method, eps):
    out = torch.empty((batch, hidden), dtype=torch.float32, device=qkv.device)
    _l.check(_l.load().bnf4_efla_step_qkv_fused(_p(S), _p(qkv), fused_cols, beta_bias, hidden, batch, method, eps, _p(out),
                                                _stream()))
    return out


# ------------------------------------------------------------------------------------------ loss / noise / update
def cross_entropy_loss(logits, bias, bias_noise, bias_noise_scale, targets_t, token_stride, loss_accum):
    batch, vocab = logits.shape
    _l.check(_l.load().bnf4_cross_entropy_loss(_p(logits), _p(bias), _p(bias_noise), bias_noise_scale, _p(targets_t),
                                               token_stride, vocab, batch, _p(loss_accum), _stream()))


def cross_entropy_population(logits, ld, bias, bias_noise_i8, sigma, targets, vocab, members, rows_per_member):
    partial = torch.empty(members * 16, dtype=torch.float32, device=logits.device)
    loss = torch.empty(members, dtype=torch.float32, device=logits.device)
    _l.check(_l.load().bnf4_cross_entropy_population(_p(logits), ld, _p(bias), _p(bias_noise_i8), sigma, _p(targets), vocab,
                                                     members, rows_per_member, _p(partial), _p(loss), _stream()))
    return loss


def fill_ternary_noise(n, seed, use_clt=True, clt_k=4, device="cuda"):
    out = torch.empty(n, dtype=torch.int8, device=device)
    _l.check(_l.load().bnf4_fill_ternary_noise(_p(out), n, seed, int(use_clt), clt_k, _stream()))
    return out


def fill_pair_seeds(base_seed, epoch, pairs, device="cuda"):
    out = torch.empty(pairs, dtype=torch.int64, device=device)
    _l.check(_l.load().bnf4_fill_pair_seeds(base_seed, epoch, pairs, _p(out), _stream()))
    return out


def compute_z_sumsq(pair_weights, pair_seeds, salt, n, use_clt=True, clt_k=4):
    Z = torch.empty(n, dtype=torch.float32, device=pair_weights.device)
    sumsq = torch.zeros(1, dtype=torch.float32, device=pair_weights.device)
    _l.check(_l.load().bnf4_compute_z_sumsq(_p(pair_weights), _p(pair_seeds), salt, pair_weights.numel(), n, int(use_clt),
                                            clt_k, _p(Z), _p(sumsq), _stream()))
    return Z, sumsq


def compute_z_sumsq_lowrank(pair_weights, A, B, rows, cols, rank, cscale):
    pairs = pair_weights.numel()
    Z = torch.empty(rows * cols, dtype=torch.float32, device=pair_weights.device)
    sumsq = torch.zeros(1, dtype=torch.float32, device=pair_weights.device)
    _l.check(_l.load().bnf4_compute_z_sumsq_lowrank(_p(pair_weights), _p(A), rows * rank, _p(B), rank * cols, pairs, rows, cols,
                                                    rank, cscale, _p(Z), _p(sumsq), _stream()))
    return Z, sumsq


def update_inv_rms(sumsq, rms_ema, use_adaptive, beta, eps, n):
    inv = torch.empty(1, dtype=torch.float32, device=sumsq.device)
    _l.check(_l.load().bnf4_update_inv_rms(_p(sumsq), _p(rms_ema), int(use_adaptive), beta, eps, n, _p(inv), _stream()))
    return inv


def update_shadow_ternary_device(w, shadow, Z, inv_rms, lr, thresh):
    _l.check(_l.load().bnf4_update_shadow_ternary_device(_p(w), _p(shadow), _p(Z), Z.numel(), _p(inv_rms), lr, thresh, _stream()))


FITNESS_SIGN, FITNESS_ZSCORE, FITNESS_CENTERED_RANK = 0, 1, 2  # the reference's TrainConfig::FitnessMode values


def shape_pair_weights(w_host, mode=FITNESS_CENTERED_RANK, clip=3.0):
    """Host-side fitness shaping on a float32 numpy array (in place); mode as in the reference's FitnessMode enum."""
    import numpy as np
    assert w_host.dtype == np.float32 and w_host.flags["C_CONTIGUOUS"]
    _l.check(_l.load().bnf4_shape_pair_weights(w_host.ctypes.data, w_host.size, mode, clip))
    return w_host

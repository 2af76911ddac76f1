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
EPI_F32, EPI_GELU_I8, EPI_GELU_FP4 = range(3)

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

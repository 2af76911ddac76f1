"""GPU test of bnf4_compute_z_sumsq_static, the variant of the dense Z / sum-of-squares step that allocates nothing
(its block partials live in an array built into the library's device image).

The file name sorts last so that the test also runs after every other GPU test has used the library; it passes
alone as well. Both entry points run the same kernels in the same order, so the comparison is bit-exact (the
tolerance of the integer/ordered-float update tests).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

STATIC_MAX_N = 256 * 262144


def _run(fn, L, pw, seeds, salt, n, torch):
    Z = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    sumsq = torch.zeros(1, dtype=torch.float32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = fn(C.c_void_p(pw.data_ptr()), C.c_void_p(seeds.data_ptr()), C.c_uint64(salt), pw.numel(), n, 1, 4,
            C.c_void_p(Z.data_ptr()), C.c_void_p(sumsq.data_ptr()), stream)
    assert rc == 0, L.bnf4_last_error().decode()
    torch.cuda.synchronize()
    return Z.cpu().numpy(), sumsq.item()


def test_static_scratch_variant_matches_allocating_variant():
    import torch
    from bitnet_nvfp4_b200 import lib
    assert torch.cuda.is_available()
    L = lib.load()
    rng = np.random.default_rng(77)
    pairs = 48
    pw = torch.from_numpy(rng.standard_normal(pairs).astype(np.float32)).cuda()
    seeds = torch.from_numpy(rng.integers(0, 2**63 - 1, pairs, dtype=np.int64)).cuda()
    # two calls in a row on the same stream: a long vector first, so that the second, shorter call finds the
    # scratch array full of the first call's partials
    for salt, n in ((0x222222, 512 * 1024 + 77), (0x999999, 5000)):
        z_ref, ss_ref = _run(L.bnf4_compute_z_sumsq, L, pw, seeds, salt, n, torch)
        z_new, ss_new = _run(L.bnf4_compute_z_sumsq_static, L, pw, seeds, salt, n, torch)
        assert not np.isnan(z_new).any()
        assert np.array_equal(z_new, z_ref)
        assert ss_new == ss_ref and ss_new > 0.0


def test_static_scratch_variant_rejects_oversized_vectors():
    import torch
    from bitnet_nvfp4_b200 import lib
    L = lib.load()
    buf = torch.zeros(16, dtype=torch.float32, device="cuda")
    seeds = torch.zeros(2, dtype=torch.int64, device="cuda")
    p = C.c_void_p(buf.data_ptr())
    # the size check comes before any launch, so the short buffers are never touched
    rc = L.bnf4_compute_z_sumsq_static(p, C.c_void_p(seeds.data_ptr()), C.c_uint64(1), 2, STATIC_MAX_N + 1, 1, 4, p, p, None)
    assert rc == 1  # BNF4_ERR_INVALID
    assert b"capacity" in L.bnf4_last_error()
    torch.cuda.synchronize()
    assert float(buf.abs().sum()) == 0.0

"""The allocation-free GEMM entry point against the regular operator entry point.

Collected last on purpose (pytest orders files by name): if it fails, a run that stops at the first
failure has already run everything else. It must pass both in a fresh process and after the other
GPU tests, because the scratch array it uses lives in the library image and keeps whatever the
previous call left there.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _q4k_matrix(rb, rng, n_out, n_in):
    w = rng.normal(0, 0.02, (n_out, n_in)).astype(np.float32)
    return np.frombuffer(b"".join(rb.quantize_row(12, w[r]) for r in range(n_out)), dtype=np.uint8)


def test_no_alloc_gemm_matches_the_regular_entry_point_on_two_calls_in_a_row(rb, oracle):
    import torch

    lib = rb.load_library()
    rng = np.random.default_rng(99)
    stream = torch.cuda.current_stream().cuda_stream
    # the second call is smaller than the first, so it runs over scratch the first one left behind
    for n_out, n_in, T in ((384, 1024, 200), (256, 512, 37)):
        raw = _q4k_matrix(rb, rng, n_out, n_in)
        x = rng.normal(0, 1.5, (T, n_in)).astype(np.float32)
        want, _ = rb.op_gemm(12, raw, n_out, n_in, x, path=3)
        d_w = torch.from_numpy(raw.copy()).cuda()
        d_x = torch.from_numpy(x).cuda()
        d_y = torch.full((T, n_out), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        status = lib.retro_b200_gemm_q4k_noalloc(d_w.data_ptr(), n_out, n_in, d_x.data_ptr(), T, d_y.data_ptr(), stream)
        assert status == 0, lib.retro_last_error()
        torch.cuda.synchronize()
        got = d_y.cpu().numpy()
        scale = float(np.abs(want).max())
        assert float(np.abs(got - want).max()) / scale < 4e-6
        # and against the float64 product of the decoded weights, the yardstick of the other GEMM tests
        w64 = oracle.dequantize_row(oracle.T_Q4_K, raw, n_out * n_in).reshape(n_out, n_in).astype(np.float64)
        exact = x.astype(np.float64) @ w64.T
        assert float(np.abs(got - exact).max()) / float(np.abs(exact).max()) < 4e-6


def test_no_alloc_gemm_refuses_shapes_beyond_its_scratch(rb):
    import torch

    lib = rb.load_library()
    d = torch.zeros(16, dtype=torch.float32, device="cuda")
    # 4096 tokens x 4096 columns is sixteen times the fixed scratch
    assert lib.retro_b200_gemm_q4k_noalloc(d.data_ptr(), 256, 4096, d.data_ptr(), 4096, d.data_ptr(), None) == -3
    assert b"exceeds the fixed scratch" in lib.retro_last_error()
    assert lib.retro_b200_gemm_q4k_noalloc(d.data_ptr(), 256, 100, d.data_ptr(), 4, d.data_ptr(), None) == -3
    assert lib.retro_b200_gemm_q4k_noalloc(None, 256, 256, d.data_ptr(), 4, d.data_ptr(), None) == -3
    # a weight pointer off the 16-byte grid would fault inside the kernel: refused on the host, nothing launched
    assert lib.retro_b200_gemm_q4k_noalloc(d.data_ptr() + 4, 256, 256, d.data_ptr(), 4, d.data_ptr(), None) == -3
    assert b"16-byte aligned" in lib.retro_last_error()

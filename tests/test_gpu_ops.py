"""Single kernels through their operator entry points against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _q4k_matrix(rb, rng, n_out, n_in):
    w = rng.normal(0, 0.02, (n_out, n_in)).astype(np.float32)
    raw = b"".join(rb.quantize_row(12, w[r]) for r in range(n_out))
    return np.frombuffer(raw, dtype=np.uint8)


@pytest.mark.parametrize("n_out,n_in,T", [(256, 512, 5), (384, 1024, 16), (200, 768, 33), (512, 2048, 100), (256, 4096, 300)])
def test_q4k_gemm_kernels_against_the_oracle(rb, oracle, n_out, n_in, T):
    rng = np.random.default_rng(n_out + T)
    raw = _q4k_matrix(rb, rng, n_out, n_in)
    x = rng.normal(0, 1.5, (T, n_in)).astype(np.float32)
    serial = np.stack([oracle.mul_mat_vec(oracle.T_Q4_K, raw, n_out, n_in, x[t]) for t in range(T)])
    # the yardstick is the exact product of the decoded weights; the oracle's serial f32 sum is itself ~1e-6 away from it
    w = oracle.dequantize_row(oracle.T_Q4_K, raw, n_out * n_in).reshape(n_out, n_in).astype(np.float64)
    want = x.astype(np.float64) @ w.T
    scale = float(np.abs(want).max())
    assert float(np.abs(serial - want).max()) / scale < 4e-6
    rows, _ = rb.op_gemm(12, raw, n_out, n_in, x, path=1)
    exact, _ = rb.op_gemm(12, raw, n_out, n_in, x, path=3)
    e_rows, e_exact = (float(np.abs(y - want).max()) / scale for y in (rows, exact))
    print(f"q4k {n_out}x{n_in} T={T}: rel err rows={e_rows:.2e} exact={e_exact:.2e}")
    assert e_rows < 4e-6 and e_exact < 4e-6


@pytest.mark.parametrize("n_out,n_in,T", [(128, 256, 128), (256, 512, 130), (200, 768, 33), (512, 2048, 100), (256, 4096, 300), (384, 2816, 40),
                                          (1536, 1024, 1664), (1500, 1280, 1601)])
def test_q4k_tcgen05_gemm_against_float64(rb, oracle, n_out, n_in, T):
    """The tcgen05 / tensor-memory kernel computes the same exact products as the mma.sync one; shapes three to six
    have few output tiles and run as splits of the reduction (the sixth with a short final split); the last two have a
    few more tiles than the GPU has SMs (156 on 148: a second, nearly empty wave), ragged rows and tokens in the second."""
    rng = np.random.default_rng(7 * n_out + T)
    raw = _q4k_matrix(rb, rng, n_out, n_in)
    x = rng.normal(0, 1.5, (T, n_in)).astype(np.float32)
    w = oracle.dequantize_row(oracle.T_Q4_K, raw, n_out * n_in).reshape(n_out, n_in).astype(np.float64)
    want = x.astype(np.float64) @ w.T
    got, _ = rb.op_gemm(12, raw, n_out, n_in, x, path=4)
    err = float(np.abs(got - want).max()) / float(np.abs(want).max())
    print(f"q4k tcgen05 {n_out}x{n_in} T={T}: rel err {err:.2e}")
    assert err < 4e-6


@pytest.mark.parametrize("n_out,n_in,T", [(256, 512, 1), (384, 1024, 3), (200, 768, 8), (512, 2816, 5), (1040, 4096, 8), (128, 14336, 2)])
def test_q4k_streaming_gemm_against_float64(rb, oracle, n_out, n_in, T):
    """The weight-streaming kernel for at most eight tokens: exact products, ragged row counts, and
    reduction lengths that leave a partial chunk of super-blocks."""
    rng = np.random.default_rng(11 * n_out + T)
    raw = _q4k_matrix(rb, rng, n_out, n_in)
    x = rng.normal(0, 1.5, (T, n_in)).astype(np.float32)
    w = oracle.dequantize_row(oracle.T_Q4_K, raw, n_out * n_in).reshape(n_out, n_in).astype(np.float64)
    want = x.astype(np.float64) @ w.T
    got, _ = rb.op_gemm(12, raw, n_out, n_in, x, path=5)
    err = float(np.abs(got - want).max()) / float(np.abs(want).max())
    print(f"q4k stream {n_out}x{n_in} T={T}: rel err {err:.2e}")
    assert err < 4e-6
    again, _ = rb.op_gemm(12, raw, n_out, n_in, x, path=5)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("n_out,n_in,T", [(256, 512, 1), (384, 1024, 3), (200, 768, 8), (40, 256, 5), (1040, 4096, 8), (128, 14336, 2)])
def test_q8_0_streaming_gemm_against_float64(rb, oracle, n_out, n_in, T):
    """The Q8_0 weight-streaming kernel for at most eight tokens against the exact product of the
    decoded weights, and against the f32 row kernel on the same bytes."""
    rng = np.random.default_rng(13 * n_out + T)
    w = rng.normal(0, 0.02, (n_out, n_in)).astype(np.float32)
    raw = np.frombuffer(b"".join(rb.quantize_row(8, w[r]) for r in range(n_out)), dtype=np.uint8)
    x = rng.normal(0, 1.5, (T, n_in)).astype(np.float32)
    wd = oracle.dequantize_row(oracle.T_Q8_0, raw, n_out * n_in).reshape(n_out, n_in).astype(np.float64)
    want = x.astype(np.float64) @ wd.T
    got, _ = rb.op_gemm(8, raw, n_out, n_in, x, path=5)
    rows, _ = rb.op_gemm(8, raw, n_out, n_in, x, path=1)
    scale = float(np.abs(want).max())
    err, err_rows = float(np.abs(got - want).max()) / scale, float(np.abs(rows - want).max()) / scale
    print(f"q8_0 stream {n_out}x{n_in} T={T}: rel err {err:.2e} (row kernel {err_rows:.2e})")
    assert err < 4e-6 and err_rows < 4e-6
    again, _ = rb.op_gemm(8, raw, n_out, n_in, x, path=5)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("n_out,n_in,T", [(256, 512, 9), (384, 1024, 16), (200, 768, 33), (512, 2048, 100), (256, 4096, 300), (130, 192, 70)])
def test_q8_0_tensor_core_gemm_against_float64(rb, oracle, n_out, n_in, T):
    """The exact Q8_0 tensor-core kernel (more than 8 tokens): per-block scales applied in f32."""
    rng = np.random.default_rng(17 * n_out + T)
    w = rng.normal(0, 0.02, (n_out, n_in)).astype(np.float32)
    raw = np.frombuffer(b"".join(rb.quantize_row(8, w[r]) for r in range(n_out)), dtype=np.uint8)
    x = rng.normal(0, 1.5, (T, n_in)).astype(np.float32)
    wd = oracle.dequantize_row(oracle.T_Q8_0, raw, n_out * n_in).reshape(n_out, n_in).astype(np.float64)
    want = x.astype(np.float64) @ wd.T
    got, _ = rb.op_gemm(8, raw, n_out, n_in, x, path=3)
    err = float(np.abs(got - want).max()) / float(np.abs(want).max())
    print(f"q8_0 mma {n_out}x{n_in} T={T}: rel err {err:.2e}")
    assert err < 4e-6


@pytest.mark.parametrize("n_out,n_in,T", [(256, 512, 17), (384, 1024, 64), (200, 768, 65), (512, 2048, 130), (130, 192, 70), (256, 4096, 300),
                                          (38016, 256, 600)])
def test_q8_0_tcgen05_gemm_against_float64(rb, oracle, n_out, n_in, T):
    """The Q8_0 tcgen05 kernel: weights as exact f16 pairs, three MMAs per product, one accumulator over the row.
    Tiles of at most 64 tokens (N = 64 MMAs), ragged row and token counts, a reduction of three stages only, and a
    shape with enough row tiles for the 256-token tile form. One matrix carries tiny and large block scales
    (subnormal f16 products, and products near the top of the f16 range)."""
    rng = np.random.default_rng(19 * n_out + T)
    w = rng.normal(0, 0.02, (n_out, n_in)).astype(np.float32)
    if n_out == 384:
        w[::3] *= 1e-4          # block scales down to ~1e-8: w_hi and w_lo are f16 subnormals
        w[1::3] *= 1e5          # block scales up to ~100: |d q| up to ~1e4
    raw = np.frombuffer(b"".join(rb.quantize_row(8, w[r]) for r in range(n_out)), dtype=np.uint8)
    x = rng.normal(0, 1.5, (T, n_in)).astype(np.float32)
    wd = oracle.dequantize_row(oracle.T_Q8_0, raw, n_out * n_in).reshape(n_out, n_in).astype(np.float64)
    want = x.astype(np.float64) @ wd.T
    got, _ = rb.op_gemm(8, raw, n_out, n_in, x, path=4)
    # row-wise yardstick: rows of very different scales share the matrix
    scale = np.abs(wd).max(axis=1) * np.abs(x).max() * np.sqrt(n_in) + 1e-30
    err = float((np.abs(got - want) / scale[None, :]).max())
    print(f"q8_0 tcgen05 {n_out}x{n_in} T={T}: scaled err {err:.2e}")
    # one accumulator runs over the whole row inside the tensor core (no per-block f32 sums outside it): the error
    # grows with the row length, to about 1e-5 of the scale at 4096 columns
    assert err < 2e-5
    again, _ = rb.op_gemm(8, raw, n_out, n_in, x, path=4)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("n_expert,n_out,n_in,counts", [(4, 256, 128, (5, 0, 130, 40)), (3, 200, 576, (128, 1, 257)), (8, 2880, 2880, (70, 3, 0, 129, 12, 64, 300, 9)),
                                                        (4, 256, 128, (300, 5, 257, 128)), (3, 300, 2880, (513, 0, 255))])
def test_mxfp4_grouped_tcgen05_gemm_against_float64(rb, oracle, n_expert, n_out, n_in, counts):
    """The grouped MXFP4 expert GEMM: empty experts, experts of more than one token tile, a ragged last row tile,
    the 20B-class MoE's own widths; the last two cases average more than 96 pairs per expert and take the 256-pair
    tile form (tiles of 256 + 44, 256 + 1, 2 x 256 + 1 and 255 pairs). Against the exact product of the decoded weights."""
    rng = np.random.default_rng(23 * n_out + n_in)
    w = rng.normal(0, 0.02, (n_expert * n_out, n_in)).astype(np.float32)
    raw = np.frombuffer(b"".join(rb.quantize_row(39, w[r]) for r in range(n_expert * n_out)), dtype=np.uint8)
    wd = oracle.dequantize_row(oracle.T_MXFP4, raw, n_expert * n_out * n_in).reshape(n_expert, n_out, n_in).astype(np.float64)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    x = rng.normal(0, 1.5, (int(offsets[-1]), n_in)).astype(np.float32)
    got = rb.op_gemm_mxfp4_grouped(raw, n_expert, n_out, n_in, x, offsets)
    worst = 0.0
    for e in range(n_expert):
        rows = slice(int(offsets[e]), int(offsets[e + 1]))
        if rows.start == rows.stop:
            continue
        want = x[rows].astype(np.float64) @ wd[e].T
        worst = max(worst, float(np.abs(got[rows] - want).max()) / float(np.abs(want).max()))
    print(f"mxfp4 grouped tcgen05 {n_expert}x{n_out}x{n_in} rows={counts}: rel err {worst:.2e}")
    assert worst < 2e-5         # one tensor-core accumulator over the whole row, as for Q8_0 above

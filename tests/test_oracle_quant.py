"""The oracle's block decoders against the reference's known answers and an independent decoder.

Known answers restate crates/rir-core/src/quant.rs:533-581 (half conversion, E8M0 half scale,
Q8_0 scale-times-byte). The random-block comparison follows quant.rs:169-214 (LCG bytes, F16
scales pinned to 2^-6 / 2^-7) and checks every element against gguf-py's numpy decoders.
"""
import struct

import numpy as np
import pytest


def test_half_conversion_is_exact(oracle):
    h = oracle.lib().ora_half_to_f32
    assert h(0x3C00) == 1.0
    assert h(0xBC00) == -1.0
    assert h(0x0000) == 0.0
    assert h(0x0001) == 2.0 ** -24
    assert h(0x0400) == 2.0 ** -14
    assert h(0x7BFF) == 65504.0


def test_half_conversion_whole_input_space(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = oracle.dequantize_row(oracle.T_F16, bits.view(np.uint8), 65536)
    finite = np.isfinite(want)
    assert np.array_equal(got[finite], want[finite])
    assert np.array_equal(np.isnan(got), np.isnan(want))


def test_e8m0_half_scale_matches_ggml(oracle):
    e = oracle.lib().ora_e8m0_half
    assert e(127) == 0.5 and e(128) == 1.0 and e(129) == 2.0
    assert struct.pack("<f", e(1)) == struct.pack("<I", 0x00400000)
    assert struct.pack("<f", e(0)) == struct.pack("<I", 0x00200000)


def test_q8_0_decodes_scale_times_byte(oracle):
    blk = bytearray(34)
    blk[0:2] = struct.pack("<H", 0x3C00)
    for j in range(32):
        blk[2 + j] = (j - 16) & 0xFF
    v = oracle.dequantize_row(oracle.T_Q8_0, bytes(blk), 32)
    assert np.array_equal(v, np.arange(32, dtype=np.float32) - 16)


def test_partial_block_is_rejected(oracle):
    with pytest.raises(ValueError):
        oracle.dequantize_row(oracle.T_Q8_0, bytes(34), 16)


def test_round_to_half_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.normal(0, 1, 4096), rng.normal(0, 1e-5, 1024), rng.normal(0, 3e4, 256), [0.0, 65504.0, 65520.0, 1e-8]]).astype(np.float32)
    r = oracle.lib().ora_round_to_half
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).astype(np.float32)
    got = np.array([r(float(v)) for v in vals], dtype=np.float32)
    assert np.array_equal(got, want)


def _random_blocks(block_bytes: int, n_blocks: int, f16_offsets, seed: int) -> np.ndarray:
    state = seed
    raw = bytearray(block_bytes * n_blocks)
    for i in range(len(raw)):
        state = (state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        raw[i] = (state >> 33) & 0xFF
    for b in range(n_blocks):
        for i, off in enumerate(f16_offsets):
            raw[b * block_bytes + off : b * block_bytes + off + 2] = struct.pack("<H", 0x2400 if i == 0 else 0x2000)
    return np.frombuffer(bytes(raw), dtype=np.uint8)


@pytest.mark.parametrize(
    "name,block_elems,block_bytes,f16_offsets",
    [("Q8_0", 32, 34, [0]), ("Q4_K", 256, 144, [0, 2]), ("MXFP4", 32, 17, [])],
)
def test_decoders_match_gguf_py_on_random_blocks(oracle, name, block_elems, block_bytes, f16_offsets):
    gguf = pytest.importorskip("gguf")
    qt = getattr(gguf.GGMLQuantizationType, name)
    n_blocks = 64
    raw = _random_blocks(block_bytes, n_blocks, f16_offsets, seed=0x1234 + block_bytes)
    if name == "MXFP4":
        raw = raw.copy()
        raw[0::17] = 100 + (raw[0::17] % 56)  # keep the exponent away from the subnormal / overflow ends
    want = gguf.quants.dequantize(raw.reshape(n_blocks, block_bytes), qt).reshape(-1).astype(np.float32)
    got = oracle.dequantize_row(int(qt.value), raw, n_blocks * block_elems)
    assert np.array_equal(got, want)


def test_mul_mat_vec_is_serial_f32(oracle):
    """dst[row] = sum over columns, in column order, of deq(a)[row][col] * b[col], all in f32
    (generated/rir/mul_mat_vec_q8_0/cpu.rs:52-81)."""
    raw = _random_blocks(34, 8 * 4, [0], seed=99)  # 4 rows of 256
    b = np.random.default_rng(1).normal(0, 1, 256).astype(np.float32)
    got = oracle.mul_mat_vec(oracle.T_Q8_0, raw, 4, 256, b)
    w = oracle.dequantize_row(oracle.T_Q8_0, raw, 4 * 256).reshape(4, 256)
    want = np.zeros(4, dtype=np.float32)
    for r in range(4):
        acc = np.float32(0)
        for c in range(256):
            acc = np.float32(acc + np.float32(w[r, c] * b[c]))
        want[r] = acc
    assert np.array_equal(got, want)


def test_rms_norm_formula(oracle):
    rng = np.random.default_rng(3)
    x = rng.normal(0, 2, 256).astype(np.float32)
    w = rng.normal(1, 0.02, 256).astype(np.float32)
    got = oracle.rms_norm(x, w, 1e-5)
    want = x.astype(np.float64) / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5) * w
    assert np.allclose(got, want, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("name,code", [("Q8_0", 2), ("Q4_0", 3)])
def test_kv_cache_rounding_is_the_published_row_quantiser(oracle, name, code):
    """A quantised KV pool stores rows through ggml's reference quantisers (absent with the llama.cpp fork; the
    reference selects the type at `crates/retrograd-ffi/runtime/src/retro_engine.cpp:84-90`). gguf-py carries the
    same published arithmetic in numpy: quantise-then-dequantise there must equal the oracle's cache, value for value."""
    import gguf
    from gguf import quants

    t = getattr(gguf.GGMLQuantizationType, name)
    rng = np.random.default_rng(11 + code)
    rows = [rng.standard_normal(256).astype(np.float32) * s for s in (1.0, 1e-3, 37.5)]
    rows.append(np.zeros(64, dtype=np.float32))                               # d = 0: every quant decodes to 0
    rows.append(np.array([1.0, -1.0] * 16 + [0.5, -2.0, 2.0] + [0.0] * 29, dtype=np.float32))   # equal magnitudes: the first one sets the sign
    rows.append((np.arange(-64, 64, dtype=np.float32) + 0.5) / 7.0)              # values on rounding boundaries
    for row in rows:
        want = quants.dequantize(quants.quantize(row[None, :], t), t)[0]
        got = oracle.kv_round(code, row)
        assert np.array_equal(got, want)
    # F16 and F32 pools
    x = rows[0]
    assert np.array_equal(oracle.kv_round(1, x), x.astype(np.float16).astype(np.float32))
    assert np.array_equal(oracle.kv_round(0, x), x)

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


def _q8_0_act(x):
    """Activation rows as ggml's quantize_row_q8_0_ref leaves them: per 32 values an f16 scale and round-half-away quants."""
    x = x.reshape(-1, 32).astype(np.float32)
    amax = np.abs(x).max(axis=1)
    d = (amax / np.float32(127)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1) / np.where(d != 0, d, 1), 0).astype(np.float32)
    v = x * inv[:, None]
    q = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int32)
    return d.astype(np.float16).astype(np.float32), q


def _scale_min_k4(j, s):
    if j < 4:
        return s[j] & 63, s[j + 4] & 63
    return (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4)


@pytest.mark.parametrize("name", ["Q8_0", "MXFP4", "Q4_K"])
def test_act_q8_gemv_is_the_integer_dot_over_requantised_activations(oracle, name):
    """The oracle's optional act = q8 mode (what the reference's CPU backend does to activations, `tests/lora_rows.rs:16-20`)
    against an independent numpy restatement of the published block arithmetic: activations to Q8_0 (32) or Q8_K (256),
    integer products, per-block scales, f32 accumulation over blocks. It stays near the f32 GEMV and is not equal to it."""
    rng = np.random.default_rng(5)
    n_row, n_col = 6, 512
    b = rng.normal(0, 1, n_col).astype(np.float32)
    kvalues = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], dtype=np.int32)
    want = np.zeros(n_row, dtype=np.float32)
    if name == "Q8_0":
        t, raw = oracle.T_Q8_0, _random_blocks(34, n_row * n_col // 32, [0], seed=7)
        ad, aq = _q8_0_act(b)
        blocks = raw.reshape(n_row, n_col // 32, 34)
        for r in range(n_row):
            acc = np.float32(0)
            for k in range(n_col // 32):
                dw = np.frombuffer(blocks[r, k, :2].tobytes(), dtype=np.float16)[0].astype(np.float32)
                qw = blocks[r, k, 2:].view(np.int8).astype(np.int32)
                acc = np.float32(acc + np.float32(np.float32(int((qw * aq[k]).sum())) * np.float32(dw * ad[k])))
            want[r] = acc
    elif name == "MXFP4":
        raw = _random_blocks(17, n_row * n_col // 32, [], seed=8).copy()
        raw[0::17] = 120 + (raw[0::17] % 12)
        t = oracle.T_MXFP4
        ad, aq = _q8_0_act(b)
        blocks = raw.reshape(n_row, n_col // 32, 17)
        for r in range(n_row):
            acc = np.float32(0)
            for k in range(n_col // 32):
                scale = np.float32(oracle.lib().ora_e8m0_half(int(blocks[r, k, 0])))
                nib = blocks[r, k, 1:]
                w = np.concatenate([kvalues[nib & 0xF], kvalues[nib >> 4]])
                acc = np.float32(acc + np.float32(np.float32(ad[k] * scale) * np.float32(int((w * aq[k]).sum()))))
            want[r] = acc
    else:
        t, raw = oracle.T_Q4_K, _random_blocks(144, n_row * n_col // 256, [0, 2], seed=9)
        x = b.reshape(-1, 256)
        idx = np.abs(x).argmax(axis=1)
        mx = x[np.arange(x.shape[0]), idx]
        iscale = (np.float32(-127) / mx).astype(np.float32)
        aq = np.minimum(127, np.rint(x * iscale[:, None])).astype(np.int32)          # np.rint: ties to even, as nearest_int
        ad = (np.float32(1) / iscale).astype(np.float32)
        bsums = aq.reshape(-1, 16, 16).sum(axis=2)
        blocks = raw.reshape(n_row, n_col // 256, 144)
        for r in range(n_row):
            acc = np.float32(0)
            for k in range(n_col // 256):
                blk = blocks[r, k]
                d, dmin = np.frombuffer(blk[:4].tobytes(), dtype=np.float16).astype(np.float32)
                scales, qs = blk[4:16].astype(np.int32), blk[16:].astype(np.int32)
                main = mins = 0
                for g in range(4):
                    sc1, m1 = _scale_min_k4(2 * g, scales)
                    sc2, m2 = _scale_min_k4(2 * g + 1, scales)
                    q = qs[g * 32:(g + 1) * 32]
                    main += int(sc1) * int(((q & 0xF) * aq[k, g * 64:g * 64 + 32]).sum()) + int(sc2) * int(((q >> 4) * aq[k, g * 64 + 32:g * 64 + 64]).sum())
                    mins += int(m1) * int(bsums[k, 4 * g] + bsums[k, 4 * g + 1]) + int(m2) * int(bsums[k, 4 * g + 2] + bsums[k, 4 * g + 3])
                acc = np.float32(acc + np.float32(np.float32(np.float32(ad[k] * d) * np.float32(main)) - np.float32(np.float32(ad[k] * dmin) * np.float32(mins))))
            want[r] = acc
    got = oracle.mul_mat_vec_act_q8(t, raw, n_row, n_col, b)
    assert np.allclose(got, want, rtol=2e-6, atol=1e-6), (got, want)
    exact = oracle.mul_mat_vec(t, raw, n_row, n_col, b)
    scale = float(np.abs(exact).max())
    assert 0 < float(np.abs(got - exact).max()) < 0.03 * scale

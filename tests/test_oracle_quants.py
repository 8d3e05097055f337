"""Pins the oracle's block decoders to the reference's own known-answer tests and to the
`gguf` package's independent numpy decoders."""
import struct

import numpy as np
import pytest

import orc


def f16_bytes(v):
    return struct.pack("<e", v)


def test_storage_sizes():
    # crates/qwen-llm/src/tensor.rs:159 storage_layout / codec.rs:393-407
    assert orc.storage_bytes(orc.Q8_0, 32) == 34
    assert orc.storage_bytes(orc.Q4_K, 256) == 144
    assert orc.storage_bytes(orc.Q5_K, 256) == 176
    assert orc.storage_bytes(orc.Q6_K, 256) == 210
    assert orc.storage_bytes(orc.BF16, 7) == 14
    assert orc.storage_bytes(orc.Q8_0, 16) == 0  # rows must be block aligned (codec.rs:580-591)


@pytest.mark.parametrize("scale,offset", [(0.25, 16), (0.5, 8), (0.125, 4)])
def test_q8_0_known_blocks(scale, offset):
    # codec.rs:474-538: block = f16 scale + bytes (index - offset); value == (index - offset) * scale
    block = bytearray(34)
    block[:2] = f16_bytes(scale)
    for i in range(32):
        block[2 + i] = (i - offset) & 0xFF
    got = orc.dequant(orc.Q8_0, np.frombuffer(bytes(block), dtype=np.uint8), 32)
    want = ((np.arange(32, dtype=np.float32) - offset) * np.float32(scale)).astype(np.float32)
    assert got.tobytes() == want.tobytes()


def test_q4_k_known_block_matches_reference_formula():
    # codec.rs:541-577
    scales = [1, 3, 5, 7, 9, 17, 33, 49]
    mins = [2, 4, 6, 8, 10, 18, 34, 50]
    block = bytearray(144)
    block[0:2] = f16_bytes(0.5)
    block[2:4] = f16_bytes(0.25)
    for j in range(4):
        block[4 + j] = scales[j] | ((scales[j + 4] >> 4) << 6)
        block[8 + j] = mins[j] | ((mins[j + 4] >> 4) << 6)
        block[12 + j] = (scales[j + 4] & 0x0F) | ((mins[j + 4] & 0x0F) << 4)
    expected = np.zeros(256, dtype=np.float32)
    for chunk in range(4):
        even, odd = chunk * 2, chunk * 2 + 1
        for lane in range(32):
            low = (chunk * 3 + lane) & 0x0F
            high = (15 + chunk * 5 - (lane & 0x0F)) & 0x0F
            block[16 + chunk * 32 + lane] = low | (high << 4)
            expected[chunk * 64 + lane] = np.float32(0.5) * np.float32(scales[even]) * np.float32(low) - np.float32(0.25) * np.float32(mins[even])
            expected[chunk * 64 + 32 + lane] = np.float32(0.5) * np.float32(scales[odd]) * np.float32(high) - np.float32(0.25) * np.float32(mins[odd])
    got = orc.dequant(orc.Q4_K, np.frombuffer(bytes(block), dtype=np.uint8), 256)
    assert got.tobytes() == expected.tobytes()


def q6_k_block(d, scales, q):
    """ggml Q6_K layout from 6-bit quants (metal/tests/q6_k_f32_tile.rs:27-45)."""
    block = bytearray(210)
    for n in range(2):
        for l in range(32):
            q1, q2, q3, q4 = (q[128 * n + l + o] for o in (0, 32, 64, 96))
            block[64 * n + l] = (q1 & 0xF) | ((q3 & 0xF) << 4)
            block[64 * n + l + 32] = (q2 & 0xF) | ((q4 & 0xF) << 4)
            block[128 + 32 * n + l] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    for i, s in enumerate(scales):
        block[192 + i] = s & 0xFF
    block[208:210] = f16_bytes(d)
    return bytes(block)


def test_q6_k_layout_decodes_to_d_scale_q_minus_32():
    # q6_k_f32_tile.rs:73-108: signed / extreme scales and every quant incl. 31..33
    rng = np.random.default_rng(7)
    for ordinal in range(12):
        d = [1.0 / 64.0, 3.0e-3, 0.25, 7.5e-4][ordinal % 4]
        scales = []
        for i in range(16):
            k = (ordinal + i) % 6
            scales.append({0: -128, 1: 127, 2: 0, 3: -1}.get(k, int(rng.integers(-127, 128))))
        q = []
        for i in range(256):
            k = (ordinal * 7 + i) % 9
            q.append({0: 31, 1: 32, 2: 33}.get(k, int(rng.integers(0, 64))))
        raw = np.frombuffer(q6_k_block(d, scales, q), dtype=np.uint8)
        got = orc.dequant(orc.Q6_K, raw, 256)
        stored_d = np.float32(struct.unpack("<e", f16_bytes(d))[0])
        want = np.array([stored_d * np.float32(scales[i // 16]) * (np.float32(q[i]) - np.float32(32.0)) for i in range(256)],
                        dtype=np.float32)
        assert got.tobytes() == want.tobytes()


@pytest.mark.parametrize("dtype,name", [(orc.Q4_K, "Q4_K"), (orc.Q5_K, "Q5_K"), (orc.Q6_K, "Q6_K"), (orc.Q8_0, "Q8_0")])
def test_decoders_agree_with_gguf_package_on_random_bytes(dtype, name):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.default_rng(123 + dtype)
    n = 256 * 8
    nbytes = orc.storage_bytes(dtype, n)
    raw = rng.integers(0, 256, size=nbytes, dtype=np.uint8)
    # keep the f16 scale fields finite: overwrite them with small normal values
    blk_bytes = {orc.Q4_K: 144, orc.Q5_K: 176, orc.Q6_K: 210, orc.Q8_0: 34}[dtype]
    view = raw.reshape(-1, blk_bytes)
    for b in range(view.shape[0]):
        if dtype in (orc.Q4_K, orc.Q5_K):
            view[b, 0:2] = np.frombuffer(f16_bytes(rng.uniform(0.001, 0.1)), dtype=np.uint8)
            view[b, 2:4] = np.frombuffer(f16_bytes(rng.uniform(0.001, 0.1)), dtype=np.uint8)
        elif dtype == orc.Q6_K:
            view[b, 208:210] = np.frombuffer(f16_bytes(rng.uniform(-0.1, 0.1)), dtype=np.uint8)
        else:
            view[b, 0:2] = np.frombuffer(f16_bytes(rng.uniform(-0.1, 0.1)), dtype=np.uint8)
    got = orc.dequant(dtype, raw, n)
    want = quants.dequantize(raw.reshape(1, -1), getattr(gguf.GGMLQuantizationType, name)).reshape(-1).astype(np.float32)
    assert got.tobytes() == want.tobytes()


@pytest.mark.parametrize("dtype", [orc.Q4_K, orc.Q5_K, orc.Q6_K, orc.Q8_0, orc.BF16, orc.F16])
def test_quantiser_emits_decodable_blocks_with_bounded_error(dtype):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(256 * 16) * 0.02).astype(np.float32)
    raw = orc.quantize(dtype, x)
    y = orc.dequant(dtype, raw, x.size)
    rel = np.abs(y - x).max() / np.abs(x).max()
    bound = {orc.Q4_K: 0.12, orc.Q5_K: 0.06, orc.Q6_K: 0.04, orc.Q8_0: 0.01, orc.BF16: 0.005, orc.F16: 0.001}[dtype]
    assert rel < bound


def test_f16_conversion_is_ieee_exact():
    L = orc.lib()
    for bits in list(range(0, 0x7C00, 37)) + [0x0001, 0x03FF, 0x0400, 0x7BFF, 0x8001, 0xFBFF]:
        want = struct.unpack("<e", struct.pack("<H", bits))[0]
        assert L.orc_f16_to_f32(bits) == want
        assert L.orc_f32_to_f16(want) == bits
    rng = np.random.default_rng(0)
    for v in rng.standard_normal(2000).astype(np.float32) * 10:
        assert L.orc_f32_to_f16(float(v)) == struct.unpack("<H", struct.pack("<e", float(v)))[0]

"""GGUF block formats: hand-built blocks decoded by a scalar restatement of the format definitions, and
quantise -> dequantise error bounds, for the 4-bit non-linear formats (IQ4_NL, IQ4_XS) next to Q4_K / Q8_0."""
import struct

import numpy as np

from inference_b200.io import gguf_quants as gq

KV = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]


def _half(x: float) -> bytes:
    return np.float16(x).tobytes()


def test_iq4_nl_block_layout():
    rng = np.random.default_rng(0)
    qs = rng.integers(0, 256, 16, dtype=np.uint8)
    raw = _half(0.03125) + qs.tobytes()
    want = [0.03125 * KV[int(b) & 0xF] for b in qs] + [0.03125 * KV[int(b) >> 4] for b in qs]
    got = gq.dequantize(raw, "IQ4_NL", 32)
    assert got.shape == (32,) and np.allclose(got, np.array(want, dtype=np.float32))
    assert gq.type_name(20) == "IQ4_NL" and gq.nbytes("IQ4_NL", 64) == 36


def test_iq4_xs_block_layout():
    rng = np.random.default_rng(1)
    qs = rng.integers(0, 256, 128, dtype=np.uint8)
    ls = rng.integers(0, 64, 8)                                   # 6-bit scales, value - 32 is the multiplier
    sh = sum(((int(v) >> 4) & 3) << (2 * i) for i, v in enumerate(ls))
    sl = bytes((int(ls[2 * i]) & 0xF) | ((int(ls[2 * i + 1]) & 0xF) << 4) for i in range(4))
    raw = _half(0.0078125) + struct.pack("<H", sh) + sl + qs.tobytes()
    assert len(raw) == 136
    want = []
    for ib in range(8):
        dl = 0.0078125 * (int(ls[ib]) - 32)
        chunk = qs[16 * ib:16 * ib + 16]
        want += [dl * KV[int(b) & 0xF] for b in chunk] + [dl * KV[int(b) >> 4] for b in chunk]
    got = gq.dequantize(raw, "IQ4_XS", 256)
    assert np.allclose(got, np.array(want, dtype=np.float32))
    assert gq.type_name(23) == "IQ4_XS" and gq.nbytes("IQ4_XS", 512) == 272


def test_non_linear_formats_round_trip_within_their_step():
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(4096) * 0.05).astype(np.float32)
    for name, fn, bits in (("IQ4_NL", gq.quantize_iq4_nl, 4.5), ("IQ4_XS", gq.quantize_iq4_xs, 4.25)):
        raw = fn(x)
        assert raw.size * 8 / x.size == bits
        y = gq.dequantize(raw, name, x.size)
        rel = np.linalg.norm(y - x) / np.linalg.norm(x)
        assert rel < 0.09, (name, rel)                              # 4-bit non-uniform grid on Gaussian data: ~6-8 %
    q4k = gq.dequantize(gq.quantize_q4_k(x), "Q4_K", x.size)
    assert np.linalg.norm(q4k - x) / np.linalg.norm(x) < 0.09
    z = np.zeros(256, dtype=np.float32)
    assert not gq.dequantize(gq.quantize_iq4_xs(z), "IQ4_XS", 256).any()
    assert not gq.dequantize(gq.quantize_iq4_nl(z), "IQ4_NL", 256).any()

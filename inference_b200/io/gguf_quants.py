"""GGML block formats: vectorised dequantisers and the Q8_0 / Q4_K quantisers.

Layouts (bytes per block / weights per block): Q4_0 18/32, Q4_1 20/32, Q5_0 22/32, Q5_1 24/32, Q8_0 34/32,
Q2_K 84/256, Q3_K 110/256, Q4_K 144/256, Q5_K 176/256, Q6_K 210/256. Formulas follow the GGML reference
dequantisers, as restated in mlx-llm/src/gguf/dequant.rs:34-86,284-290,381-416: Q8_0 `w = qs * d`; Q4_K eight
32-weight sub-blocks with 6-bit scales/mins unpacked by `get_scale_min_k4`, low nibbles then high nibbles per
64-weight chunk, `w = d * sc * q - dmin * m`."""
from __future__ import annotations

import numpy as np

from ..contracts.errors import Unsupported

GGML_TYPES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K",
              12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 20: "IQ4_NL", 23: "IQ4_XS", 24: "I8", 25: "I16", 26: "I32", 27: "I64", 28: "F64", 30: "BF16"}
TYPE_IDS = {v: k for k, v in GGML_TYPES.items()}
BLOCK = {"F32": (4, 1), "F16": (2, 1), "BF16": (2, 1), "F64": (8, 1), "I8": (1, 1), "I16": (2, 1), "I32": (4, 1),
         "I64": (8, 1), "Q4_0": (18, 32), "Q4_1": (20, 32), "Q5_0": (22, 32), "Q5_1": (24, 32), "Q8_0": (34, 32),
         "Q2_K": (84, 256), "Q3_K": (110, 256), "Q4_K": (144, 256), "Q5_K": (176, 256), "Q6_K": (210, 256),
         "IQ4_NL": (18, 32), "IQ4_XS": (136, 256)}
# the 16 non-uniform levels of the 4-bit "non-linear" formats (ggml's kvalues_iq4nl)
IQ4_LEVELS = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def type_name(type_id: int) -> str:
    if type_id not in GGML_TYPES:
        raise Unsupported(f"GGML tensor type {type_id} is not supported (IQ / TQ / MXFP4 grids are not implemented)")
    return GGML_TYPES[type_id]


def nbytes(type_name_: str, n_elements: int) -> int:
    b, w = BLOCK[type_name_]
    return n_elements // w * b


def _f16(raw: np.ndarray) -> np.ndarray:
    return raw.copy().view(np.float16).astype(np.float32)


def _scale_min_k4(scales: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """scales uint8 [nb, 12] -> (sc, m) uint8 [nb, 8] (6-bit values)."""
    q = scales.astype(np.uint8)
    sc = np.empty((q.shape[0], 8), dtype=np.uint8)
    m = np.empty_like(sc)
    sc[:, :4] = q[:, 0:4] & 63
    m[:, :4] = q[:, 4:8] & 63
    sc[:, 4:] = (q[:, 8:12] & 0x0F) | ((q[:, 0:4] >> 6) << 4)
    m[:, 4:] = (q[:, 8:12] >> 4) | ((q[:, 4:8] >> 6) << 4)
    return sc, m


def dequantize(raw: bytes | np.ndarray, tname: str, n_elements: int) -> np.ndarray:
    """Raw tensor bytes -> float32 [n_elements]."""
    buf = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw.view(np.uint8).reshape(-1)
    if tname == "F32":
        return buf.view(np.float32)[:n_elements].astype(np.float32)
    if tname == "F16":
        return buf.view(np.float16)[:n_elements].astype(np.float32)
    if tname == "BF16":
        return (buf.view(np.uint16)[:n_elements].astype(np.uint32) << 16).view(np.float32)
    if tname == "F64":
        return buf.view(np.float64)[:n_elements].astype(np.float32)
    if tname in ("I8", "I16", "I32", "I64"):
        return buf.view({"I8": np.int8, "I16": np.int16, "I32": np.int32, "I64": np.int64}[tname])[:n_elements] \
            .astype(np.float32)
    bsz, w = BLOCK[tname]
    nb = n_elements // w
    blk = buf[: nb * bsz].reshape(nb, bsz)
    if tname == "Q8_0":
        d = _f16(blk[:, 0:2]).reshape(nb, 1)
        return (blk[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)
    if tname in ("Q4_0", "Q4_1"):
        d = _f16(blk[:, 0:2]).reshape(nb, 1)
        off = 2
        m = 0.0
        if tname == "Q4_1":
            m = _f16(blk[:, 2:4]).reshape(nb, 1)
            off = 4
        qs = blk[:, off:off + 16]
        lo, hi = (qs & 0x0F).astype(np.float32), (qs >> 4).astype(np.float32)
        q = np.concatenate([lo, hi], axis=1)
        return ((q - 8.0) * d if tname == "Q4_0" else q * d + m).reshape(-1)
    if tname in ("Q5_0", "Q5_1"):
        d = _f16(blk[:, 0:2]).reshape(nb, 1)
        off = 2
        m = 0.0
        if tname == "Q5_1":
            m = _f16(blk[:, 2:4]).reshape(nb, 1)
            off = 4
        qh = blk[:, off:off + 4].copy().view(np.uint32).reshape(nb, 1)
        qs = blk[:, off + 4:off + 20]
        j = np.arange(16, dtype=np.uint32).reshape(1, 16)
        h0 = ((qh >> j) & 1).astype(np.uint8) << 4
        h1 = ((qh >> (j + 16)) & 1).astype(np.uint8) << 4
        q = np.concatenate([(qs & 0x0F) | h0, (qs >> 4) | h1], axis=1).astype(np.float32)
        return ((q - 16.0) * d if tname == "Q5_0" else q * d + m).reshape(-1)
    if tname == "IQ4_NL":                      # fp16 d + 16 bytes: low nibbles are weights 0..15, high nibbles 16..31
        d = _f16(blk[:, 0:2]).reshape(nb, 1)
        qs = blk[:, 2:18]
        return (np.concatenate([IQ4_LEVELS[qs & 0x0F], IQ4_LEVELS[qs >> 4]], axis=1) * d).reshape(-1)
    if tname == "IQ4_XS":                      # fp16 d, u16 high scale bits, 4 bytes of low scale nibbles, 8 x 16 bytes
        d = _f16(blk[:, 0:2]).reshape(nb, 1)
        sh = blk[:, 2:4].copy().view(np.uint16).reshape(nb, 1).astype(np.int32)
        sl = blk[:, 4:8].astype(np.int32)
        ib = np.arange(8)
        ls = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)          # [nb, 8], 6 bits
        dl = d * (ls - 32).astype(np.float32)
        qs = blk[:, 8:136].reshape(nb, 8, 16)
        vals = np.concatenate([IQ4_LEVELS[qs & 0x0F], IQ4_LEVELS[qs >> 4]], axis=2)              # [nb, 8, 32]
        return (vals * dl[:, :, None]).reshape(-1)
    if tname == "Q4_K":
        d = _f16(blk[:, 0:2]).reshape(nb, 1, 1)
        dmin = _f16(blk[:, 2:4]).reshape(nb, 1, 1)
        sc, m = _scale_min_k4(blk[:, 4:16])
        qs = blk[:, 16:144].reshape(nb, 4, 32)
        q = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)
        return (d * sc.reshape(nb, 8, 1) * q - dmin * m.reshape(nb, 8, 1)).reshape(-1)
    if tname == "Q5_K":
        d = _f16(blk[:, 0:2]).reshape(nb, 1, 1)
        dmin = _f16(blk[:, 2:4]).reshape(nb, 1, 1)
        sc, m = _scale_min_k4(blk[:, 4:16])
        qh = blk[:, 16:48].reshape(nb, 1, 32)
        ql = blk[:, 48:176].reshape(nb, 4, 32)
        bits = np.arange(8, dtype=np.uint8).reshape(1, 8, 1)
        hb = ((qh >> bits) & 1).astype(np.uint8) << 4           # [nb, 8, 32]: sub-block j uses bit j
        q4 = np.stack([ql & 0x0F, ql >> 4], axis=2).reshape(nb, 8, 32)
        q = (q4 | hb).astype(np.float32)
        return (d * sc.reshape(nb, 8, 1) * q - dmin * m.reshape(nb, 8, 1)).reshape(-1)
    if tname == "Q6_K":
        ql = blk[:, 0:128].reshape(nb, 2, 64)
        qh = blk[:, 128:192].reshape(nb, 2, 32)
        sc = blk[:, 192:208].view(np.int8).reshape(nb, 2, 8).astype(np.float32)
        d = _f16(blk[:, 208:210]).reshape(nb, 1, 1)
        l0, l1 = ql[:, :, :32], ql[:, :, 32:]
        q1 = ((l0 & 0x0F) | (((qh >> 0) & 3) << 4)).astype(np.int16) - 32
        q2 = ((l1 & 0x0F) | (((qh >> 2) & 3) << 4)).astype(np.int16) - 32
        q3 = ((l0 >> 4) | (((qh >> 4) & 3) << 4)).astype(np.int16) - 32
        q4 = ((l1 >> 4) | (((qh >> 6) & 3) << 4)).astype(np.int16) - 32
        q = np.stack([q1, q2, q3, q4], axis=2).astype(np.float32)            # [nb, 2, 4, 32]
        idx = (np.arange(32) // 16).reshape(1, 1, 1, 32) + (2 * np.arange(4)).reshape(1, 1, 4, 1)  # is + 0/2/4/6
        scale = np.take_along_axis(sc.reshape(nb, 2, 1, 8).repeat(4, axis=2), np.broadcast_to(idx, (nb, 2, 4, 32)),
                                   axis=3)
        return (d.reshape(nb, 1, 1, 1) * scale * q).reshape(-1)
    if tname == "Q2_K":
        scales = blk[:, 0:16].reshape(nb, 2, 4, 2)                # [chunk n][shift j][first/second 16]
        qs = blk[:, 16:80].reshape(nb, 2, 1, 32)
        d = _f16(blk[:, 80:82]).reshape(nb, 1, 1, 1)
        dmin = _f16(blk[:, 82:84]).reshape(nb, 1, 1, 1)
        shifts = (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)
        q = ((qs >> shifts) & 3).astype(np.float32).reshape(nb, 2, 4, 2, 16)
        dl = (d.reshape(nb, 1, 1, 1) * (scales & 0x0F).astype(np.float32))[..., None]
        ml = (dmin.reshape(nb, 1, 1, 1) * (scales >> 4).astype(np.float32))[..., None]
        return (dl * q - ml).reshape(-1)
    if tname == "Q3_K":
        hm = blk[:, 0:32].reshape(nb, 1, 1, 32)
        qs = blk[:, 32:96].reshape(nb, 2, 1, 32)
        aux = blk[:, 96:108].copy().view(np.uint32).reshape(nb, 3)
        d = _f16(blk[:, 108:110]).reshape(nb, 1, 1, 1, 1)
        k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
        a0, a1, tmp = aux[:, 0], aux[:, 1], aux[:, 2]
        out = np.stack([(a0 & k2) | (((tmp >> 0) & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
                        ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)],
                       axis=1).astype(np.uint32)
        sc = out.view(np.uint8).reshape(nb, 16).view(np.int8).astype(np.float32) - 32.0   # 16 scales
        sc = sc.reshape(nb, 2, 4, 2, 1)
        shifts = (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)
        q = ((qs >> shifts) & 3).astype(np.int16)                                   # [nb, 2, 4, 32]
        mbit = np.arange(8, dtype=np.uint8).reshape(1, 2, 4, 1)                      # m = 1 << (4 n + j)
        hi = ((hm >> mbit) & 1).astype(np.int16)
        q = (q - np.where(hi == 1, 0, 4)).astype(np.float32).reshape(nb, 2, 4, 2, 16)
        return (d * sc * q).reshape(-1)
    raise Unsupported(f"dequantisation of GGML type {tname} is not implemented")


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """float32 [..., k] (k % 32 == 0) -> uint8 raw Q8_0 blocks."""
    v = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(v).max(axis=1, keepdims=True)
    d = (amax / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    q = np.where(df > 0, np.rint(v / np.where(df > 0, df, 1.0)), 0.0).clip(-127, 127).astype(np.int8)
    out = np.empty((v.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_k(x: np.ndarray) -> np.ndarray:
    """float32 [..., k] (k % 256 == 0) -> uint8 raw Q4_K super-blocks (min/max scheme, 6-bit sub-scales)."""
    v = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 8, 32)
    nb = v.shape[0]
    mins = np.maximum(0.0, -v.min(axis=2))
    scales = (v.max(axis=2) + mins) / 15.0
    d = (scales.max(axis=1, keepdims=True) / 63.0).astype(np.float16)
    dmin = (mins.max(axis=1, keepdims=True) / 63.0).astype(np.float16)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.where(df > 0, np.rint(scales / np.where(df > 0, df, 1.0)), 0).clip(0, 63).astype(np.uint8)
    m = np.where(dmf > 0, np.rint(mins / np.where(dmf > 0, dmf, 1.0)), 0).clip(0, 63).astype(np.uint8)
    eff = (df * sc)[..., None]
    q = np.where(eff > 0, np.rint((v + (dmf * m)[..., None]) / np.where(eff > 0, eff, 1.0)), 0).clip(0, 15) \
        .astype(np.uint8)
    out = np.zeros((nb, 144), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
    packed = np.zeros((nb, 12), dtype=np.uint8)
    packed[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    packed[:, 4:8] = (m[:, 0:4] & 63) | ((m[:, 4:8] >> 4) << 6)
    packed[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((m[:, 4:8] & 0x0F) << 4)
    out[:, 4:16] = packed
    q = q.reshape(nb, 4, 2, 32)
    out[:, 16:144] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(-1)


def quantize_iq4_nl(x: np.ndarray) -> np.ndarray:
    """float32 [n] (n % 32 == 0) -> IQ4_NL bytes: per block d = max-magnitude value / -127 (the largest level in
    magnitude), each weight to the nearest level."""
    b = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(b).argmax(axis=1)
    vmax = b[np.arange(len(b)), idx]
    d = (vmax / -127.0).astype(np.float16)
    inv = np.where(d.astype(np.float32) != 0, 1.0 / np.where(d == 0, 1, d).astype(np.float32), 0.0)
    q = np.abs((b * inv[:, None])[:, :, None] - IQ4_LEVELS[None, None, :]).argmin(axis=2).astype(np.uint8)
    out = np.zeros((len(b), 18), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:18] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def quantize_iq4_xs(x: np.ndarray) -> np.ndarray:
    """float32 [n] (n % 256 == 0) -> IQ4_XS bytes: one fp16 d per 256 weights, a 6-bit scale (offset 32) per 32."""
    b = np.asarray(x, dtype=np.float32).reshape(-1, 8, 32)
    nb = len(b)
    sub_max = np.abs(b).max(axis=2)                                   # [nb, 8]
    d = (sub_max.max(axis=1) / (127.0 * 31.0)).astype(np.float16)     # largest sub-block gets scale 31
    df = d.astype(np.float32)
    ls = np.where(df[:, None] > 0, np.rint(sub_max / (127.0 * np.where(df == 0, 1, df))[:, None]), 0).clip(0, 31).astype(np.int32) + 32
    dl = df[:, None] * (ls - 32)
    inv = np.where(dl != 0, 1.0 / np.where(dl == 0, 1, dl), 0.0)
    q = np.abs((b * inv[:, :, None])[..., None] - IQ4_LEVELS).argmin(axis=3).astype(np.uint8)      # [nb, 8, 32]
    out = np.zeros((nb, 136), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    sh = np.zeros(nb, dtype=np.uint16)
    for i in range(8):
        sh |= ((ls[:, i] >> 4) & 3).astype(np.uint16) << (2 * i)
        out[:, 4 + i // 2] |= ((ls[:, i] & 0xF) << (4 * (i % 2))).astype(np.uint8)
    out[:, 2:4] = sh.view(np.uint8).reshape(-1, 2)
    out[:, 8:136] = (q[:, :, :16] | (q[:, :, 16:] << 4)).reshape(nb, 128)
    return out.reshape(-1)

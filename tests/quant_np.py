"""numpy helpers for the tests: ggjt-v3 q4_0 / q8_0 quantisation of fp32
matrices with the block formulas the synthetic model writer uses
(scale = f16(absmax / 8) resp. f16(absmax / 127), round to nearest)."""
import numpy as np

Q4_0, Q8_0 = 2, 8
Q4_0_V1 = 258          # kernel type code of version-1 q4_0 blocks (the oracle calls them type 2, version 1)


def quantize_q4_0(w):
    w = np.asarray(w, np.float32).reshape(-1, 32)
    amax = np.abs(w).max(axis=1)
    d16 = (amax / np.float32(8)).astype(np.float16)
    d = d16.astype(np.float32)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0).astype(np.float32)
    q = np.clip(np.rint(w * inv[:, None]) + 8, 0, 15).astype(np.uint8)
    out = np.empty((w.shape[0], 18), np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)       # element j low nibble, j+16 high nibble
    return out.reshape(-1)


def quantize_q8_0(w):
    w = np.asarray(w, np.float32).reshape(-1, 32)
    amax = np.abs(w).max(axis=1)
    d16 = (amax / np.float32(127)).astype(np.float16)
    d = d16.astype(np.float32)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0).astype(np.float32)
    q = np.clip(np.rint(w * inv[:, None]), -127, 127).astype(np.int8)
    out = np.empty((w.shape[0], 34), np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0_v1(w):
    """ggjt version 1: f32 scale = absmax / 8, byte j = elements 2j (low nibble) and 2j + 1 (high nibble)."""
    w = np.asarray(w, np.float32).reshape(-1, 32)
    d = (np.abs(w).max(axis=1) / np.float32(8)).astype(np.float32)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0).astype(np.float32)
    q = np.clip(np.rint(w * inv[:, None]) + 8, 0, 15).astype(np.uint8)
    out = np.empty((w.shape[0], 20), np.uint8)
    out[:, 0:4] = d.view(np.uint8).reshape(-1, 4)
    out[:, 4:] = q[:, 0::2] | (q[:, 1::2] << 4)
    return out.reshape(-1)


def quantize(w, wtype):
    return quantize_q4_0(w) if wtype == Q4_0 else quantize_q8_0(w)


def dequantize_np(raw, wtype):
    """Independent numpy restatement of the v3 dequantisation formulas, used to
    cross-check the C oracle (q4_0: (nibble - 8) * d; q8_0: int8 * d)."""
    if wtype == Q4_0:
        b = np.asarray(raw, np.uint8).reshape(-1, 18)
        d = b[:, :2].copy().view(np.float16).astype(np.float32)
        lo = (b[:, 2:] & 0xF).astype(np.int32) - 8
        hi = (b[:, 2:] >> 4).astype(np.int32) - 8
        return (np.concatenate([lo, hi], axis=1).astype(np.float32) * d).reshape(-1)
    b = np.asarray(raw, np.uint8).reshape(-1, 34)
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    return (b[:, 2:].copy().view(np.int8).astype(np.float32) * d).reshape(-1)


def row_bytes(wtype, cols):
    return cols // 32 * (18 if wtype == Q4_0 else 34)

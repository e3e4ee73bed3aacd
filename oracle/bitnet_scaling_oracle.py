"""CPU restatement of the two scaling steps around the ternary product -- TEST INFRASTRUCTURE ONLY.

Parity unpinned: the reference has no implementation of these steps (its README lists activation / absmean
scaling as missing, README.md:203), so there are no reference outputs or golden vectors to pin against.  The
arithmetic below restates the published BitNet b1.58 recipe ("The Era of 1-bit LLMs", arXiv:2402.17764, and
"BitNet: Scaling 1-bit Transformers", arXiv:2310.11453: per-token absmax int8 activations, absmean ternary
weights, output rescaled by both scales) in float32, with the operation order written out, so that the GPU
path can be compared bit for bit with THIS restatement.
"""
import numpy as np


def quantize_rows(x):
    """absmax = max|x| per row; q = rint(x * (127 / absmax)) clamped to [-127, 127]; row_scale = absmax / 127.
    float32 throughout, round half to even; an all-zero row gives q = 0 and row_scale = 1."""
    x = np.asarray(x, dtype=np.float32)
    absmax = np.abs(x).max(axis=1).astype(np.float32)
    nz = absmax > 0
    s = np.zeros_like(absmax)
    s[nz] = np.float32(127.0) / absmax[nz]
    q = np.rint(x * s[:, None]).astype(np.float32)
    q = np.clip(q, -127, 127).astype(np.int8)
    row_scale = np.ones_like(absmax)
    row_scale[nz] = absmax[nz] / np.float32(127.0)
    return q, row_scale


def bf16_bits_rn(f32):
    """float32 -> bfloat16 bit pattern (uint16), round to nearest even (no NaN inputs here)."""
    u = np.asarray(f32, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def dequant_bf16_bits(c_int32, row_scale, w_scale):
    """y = bf16_rn((float32(c) * row_scale[m]) * w_scale) as uint16 bit patterns."""
    c = np.asarray(c_int32).astype(np.float32)
    y = (c * np.asarray(row_scale, dtype=np.float32)[:, None]).astype(np.float32) * np.float32(w_scale)
    return bf16_bits_rn(y.astype(np.float32))

"""Oracle: offline weight quantizers and runtime activation quantizers.

Test infrastructure only (see ``oracle/__init__.py``).  numpy restatement of
the reference's torch arithmetic.  All division is true fp32 division,
``round`` is round-half-to-even, every intermediate is float32 exactly as the
reference's ``.float()`` tensors are.

Citations are paths inside the reference project ``himikk/vllm-quant-kernels``.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32
GROUP = 32  # src/vllm_quant_kernels/_kernels.py:488,646 (MXFP8_GROUP_SIZE / MXFP4_GROUP_SIZE)

# E2M1 magnitudes and the midpoints the reference buckets on
# (src/vllm_quant_kernels/_quant.py:27-31, tests/test_mxfp4_accuracy.py:27-30).
E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=F32)
E2M1_MIDPOINTS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=F32)


def _f32(a) -> np.ndarray:
    """``tensor.float()``: fp16 / bf16-as-fp32 / fp32 input to float32."""
    return np.asarray(a).astype(F32)


# --------------------------------------------------------------------------
# float8 e4m3fn encode / decode (the arithmetic of torch's
# ``Tensor.to(torch.float8_e4m3fn)``, used at _quant.py:60,308,413)
# --------------------------------------------------------------------------

def e4m3_encode(x) -> np.ndarray:
    """fp32 -> e4m3fn byte, round-to-nearest-even, NON-saturating.

    |x| <= 464 rounds into the finite range (max 448 = 0x7e); anything larger,
    inf and NaN become NaN (0x7f / 0xff).  Subnormals go down to 2^-9; -0.0
    keeps its sign (0x80).
    """
    x = _f32(x)
    bits = x.view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    a = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)

    nan = ~np.isfinite(a)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0))).astype(np.int64)
    # guard against log2 landing one off at exact powers of two
    e = np.where(np.ldexp(1.0, e) > a, e - 1, e)
    e = np.where(np.ldexp(1.0, e + 1) <= a, e + 1, e)

    normal = a >= 2.0 ** -6
    # normal: 3 mantissa bits -> q in [8, 16]
    qn = np.rint(np.ldexp(a, 3 - e)).astype(np.int64)
    en = np.where(qn == 16, e + 1, e)
    qn = np.where(qn == 16, 8, qn)
    code_n = ((en + 7) << 3) | (qn - 8)
    overflow = (en + 7 > 15) | (((en + 7) == 15) & ((qn - 8) == 7))
    # subnormal: units of 2^-9; q == 8 lands on the smallest normal (0x08)
    qs = np.rint(np.ldexp(a, 9)).astype(np.int64)
    code = np.where(normal, code_n, qs)
    code = np.where(normal & overflow, 0x7F, code)
    code = np.where(nan, 0x7F, code)
    out = (code.astype(np.uint8) & 0x7F) | sign
    return out


def e4m3_decode(b) -> np.ndarray:
    """e4m3fn byte -> fp32 (0x7f / 0xff are NaN; there are no infinities)."""
    b = np.asarray(b).astype(np.uint8)
    s = np.where(b & 0x80, F32(-1.0), F32(1.0))
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 0x7).astype(np.int32)
    val = np.where(e == 0, np.ldexp(m.astype(np.float64), -9),
                   np.ldexp((8 + m).astype(np.float64), e - 10))
    val = np.where((e == 15) & (m == 7), np.nan, val)
    return (s * val).astype(F32)


# --------------------------------------------------------------------------
# Per-row INT8 / FP8 weight quantizers
# --------------------------------------------------------------------------

def quantize_int8_rows(w, scale_dtype=np.float16):
    """Per-row symmetric INT8.  _quant.py:248-255 (W8A16, fp16 scale) and
    :285-292 (W8A8, fp32 scale)."""
    wf = _f32(w)
    s = (np.abs(wf).max(axis=1) / F32(127.0)).astype(F32)
    s = np.maximum(s, F32(1e-12))
    q = np.clip(np.rint(wf / s[:, None]), -127, 127).astype(np.int8)
    return q, s.astype(scale_dtype)


def quantize_fp8_rows(w):
    """Per-row FP8 e4m3, scale = absmax / 448 stored as fp16.  _quant.py:306-314.
    Codes are returned as the int8 view the reference stores."""
    wf = _f32(w)
    s = (np.abs(wf).max(axis=1) / F32(448.0)).astype(F32)
    s = np.maximum(s, F32(1e-12))
    v = np.clip(wf / s[:, None], F32(-448.0), F32(448.0)).astype(F32)
    return e4m3_encode(v).view(np.int8), s.astype(np.float16)


# --------------------------------------------------------------------------
# MX quantizers
# --------------------------------------------------------------------------

def ceil_log2_f32(r) -> np.ndarray:
    """``ceil(log2(r))`` for positive normal fp32 ``r`` by the integer rule
    "exponent if the mantissa is zero, else exponent + 1".  torch's fp32
    ``log2`` agrees with it except when ``r`` sits 1-2 ulp above a power of two
    (there the float log2 rounds down to the integer); see
    :func:`ceil_log2_is_ambiguous`."""
    b = _f32(r).view(np.uint32)
    e = ((b >> 23) & 0xFF).astype(np.int32) - 127
    m = b & 0x7FFFFF
    return np.where(m == 0, e, e + 1).astype(np.int32)


def ceil_log2_is_ambiguous(r) -> np.ndarray:
    """True where float ``log2`` implementations may disagree about
    ``ceil(log2(r))``: mantissa within a few ulp above a power of two."""
    m = _f32(r).view(np.uint32) & 0x7FFFFF
    return (m != 0) & (m <= 8)


def _mx_scale(groups_absmax, fmt_max):
    g = np.maximum(groups_absmax.astype(F32), F32(1e-30))
    r = (g / F32(fmt_max)).astype(F32)
    k = np.clip(ceil_log2_f32(r), -127, 127)
    return k, r


def quantize_mxfp8(t):
    """MXFP8: e4m3 codes + one E8M0 byte per 32 elements, scale exponent chosen
    with CEIL so the group max always fits.  _quant.py:34-61."""
    tf = _f32(t)
    R, K = tf.shape
    assert K % GROUP == 0, f"K={K} must be divisible by group_size={GROUP}"
    g = tf.reshape(R, K // GROUP, GROUP)
    k, _ = _mx_scale(np.abs(g).max(axis=-1), 448.0)
    sc = np.ldexp(F32(1.0), k).astype(F32)[..., None]
    v = np.clip((g / sc).astype(F32), F32(-448.0), F32(448.0))
    codes = e4m3_encode(v).reshape(R, K)
    return codes, (k + 127).astype(np.uint8)


def quantize_mxfp4(t):
    """MXFP4: E2M1 nibbles packed two per byte (even index in the LOW nibble)
    + E8M0 byte per 32.  Exact midpoint ties go to the SMALLER magnitude
    (torch.bucketize, right=False); a negative value that rounds to zero keeps
    its sign bit; -0.0 has sign 0 because the test is ``scaled < 0``.
    _quant.py:64-105."""
    tf = _f32(t)
    R, K = tf.shape
    assert K % GROUP == 0, f"K={K} must be divisible by group_size={GROUP}"
    assert K % 2 == 0
    g = tf.reshape(R, K // GROUP, GROUP)
    k, _ = _mx_scale(np.abs(g).max(axis=-1), 6.0)
    sc = np.ldexp(F32(1.0), k).astype(F32)[..., None]
    scaled = (g / sc).astype(F32).reshape(R, K)
    sign = (scaled < 0).astype(np.uint8) << 3
    mag = np.minimum(np.abs(scaled), F32(6.0))
    # bucketize(right=False): idx = number of midpoints strictly below mag
    idx = np.searchsorted(E2M1_MIDPOINTS, mag, side="left").astype(np.uint8)
    nib = sign | idx
    packed = (nib[:, 1::2] << 4) | nib[:, 0::2]
    return np.ascontiguousarray(packed), (k + 127).astype(np.uint8)


def mx_scale_ambiguous(t, fmt_max) -> np.ndarray:
    """(R, K/32) mask of groups whose scale exponent is implementation-defined."""
    tf = _f32(t)
    R, K = tf.shape
    g = tf.reshape(R, K // GROUP, GROUP)
    _, r = _mx_scale(np.abs(g).max(axis=-1), fmt_max)
    return ceil_log2_is_ambiguous(r)


# --------------------------------------------------------------------------
# Runtime activation quantizers
# --------------------------------------------------------------------------

def act_quant_fp8(x):
    """Unscaled, unclamped, non-saturating e4m3 cast.  _quant.py:413."""
    return e4m3_encode(_f32(x))


def act_quant_int8_tensor(x):
    """Per-TENSOR symmetric INT8 over all rows of the batch.  _quant.py:536-540."""
    xf = _f32(x)
    s = F32(np.abs(xf).max() / F32(127.0)) if xf.size else F32(0.0)
    s = np.maximum(s, F32(1e-12)).astype(F32)
    q = np.clip(np.rint(xf / s), -127, 127).astype(np.int8)
    return q, s


def act_quant_mxfp8(x):
    """Activations for MXFP8 and MXFP4(W4A8) use the weight quantizer.
    _quant.py:448,495."""
    return quantize_mxfp8(x)


# --------------------------------------------------------------------------
# Dequantizers (fp32)
# --------------------------------------------------------------------------

def e8m0_decode(s) -> np.ndarray:
    """scale = 2^(byte - 127).  tests/test_mxfp4_accuracy.py:65-67."""
    return np.ldexp(F32(1.0), np.asarray(s).astype(np.int32) - 127).astype(F32)


def dequant_mxfp8(codes, scales) -> np.ndarray:
    """tests/test_mxfp4_kernel.py:64-72 (e4m3 view -> float, times 2^(s-127))."""
    R, K = codes.shape
    v = e4m3_decode(codes).reshape(R, K // GROUP, GROUP)
    return (v * e8m0_decode(scales)[..., None]).reshape(R, K).astype(F32)


def dequant_mxfp4(packed, scales) -> np.ndarray:
    """tests/test_mxfp4_accuracy.py:39-69."""
    packed = np.asarray(packed).astype(np.uint8)
    R, Kh = packed.shape
    K = Kh * 2
    nib = np.stack([packed & 0xF, (packed >> 4) & 0xF], axis=-1).reshape(R, K)
    mag = E2M1_GRID[nib & 7]
    val = np.where((nib >> 3) & 1, -mag, mag).astype(F32)
    return (val.reshape(R, K // GROUP, GROUP) * e8m0_decode(scales)[..., None]).reshape(R, K).astype(F32)

"""TEST INFRASTRUCTURE -- not product code.

Python face of the CPU checker: ctypes bindings over ``_build/liboracle.so`` (the plain-C
restatement in ``flint_oracle.c``) and, when it was built, over ``_ref/libflint_cpu.so`` -- the
reference's own CPU backend, whose float32 ``fl_matmul`` (flint/cpu/matmul.cc:306-322) then does
the heavy product. Only tests, the smoke check and the bench's CPU-baseline leg import this.

16-bit floats travel as ``numpy.uint16`` bit patterns; codes as ``numpy.uint8``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_uint8, c_uint16, c_void_p

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libflint_cpu.so")

ACT_NONE = 0
ACT_GELU_TANH = 1


def reference_dir():
    """The reference checkout to compile the checker from: $FLINT_REFERENCE_DIR, else a directory
    named `reference` beside this repository; None where neither exists (the prebuilt library under
    _ref/, if any, is then used as it is)."""
    named = os.environ.get("FLINT_REFERENCE_DIR")
    candidates = [named] if named else [os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in candidates:
        if c and os.path.isfile(os.path.join(c, "flint", "capi.h")):
            return os.path.abspath(c)
    return None


def build(ref: bool = True) -> None:
    """Compile the C restatement, and the reference's CPU library where its checkout exists."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    ref_dir = reference_dir() if ref else None
    if ref_dir:
        subprocess.run(["make", "-s", "-C", HERE, "ref", "-j8", f"REF={ref_dir}"], check=True)


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        L = ctypes.CDLL(ORACLE_SO)
        u8p, u16p, f32p, f64p = POINTER(c_uint8), POINTER(c_uint16), POINTER(c_float), POINTER(ctypes.c_double)
        L.fo_e4m3_decode.argtypes = [c_uint8]; L.fo_e4m3_decode.restype = c_float
        L.fo_e4m3_encode.argtypes = [c_float]; L.fo_e4m3_encode.restype = c_uint8
        L.fo_e2m1_decode.argtypes = [c_uint8]; L.fo_e2m1_decode.restype = c_float
        L.fo_e2m1_encode.argtypes = [c_float]; L.fo_e2m1_encode.restype = c_uint8
        L.fo_bf16_from_f32.argtypes = [c_float]; L.fo_bf16_from_f32.restype = c_uint16
        L.fo_bf16_to_f32.argtypes = [c_uint16]; L.fo_bf16_to_f32.restype = c_float
        L.fo_f16_from_f32.argtypes = [c_float]; L.fo_f16_from_f32.restype = c_uint16
        L.fo_f16_to_f32.argtypes = [c_uint16]; L.fo_f16_to_f32.restype = c_float
        L.fo_quantize_fp8_tensor.argtypes = [f32p, c_int64, u8p, f32p]
        L.fo_quantize_fp8_rows.argtypes = [f32p, c_int, c_int, u8p, f32p]
        L.fo_quantize_fp8_act.argtypes = [u16p, c_int, c_int, c_int, u8p, f32p]
        L.fo_quantize_fp8_act_amax.argtypes = [u16p, c_int, c_int, c_int, f32p, u8p, f32p]
        L.fo_quantize_nvfp4_weight.argtypes = [f32p, c_int, c_int, u8p, u8p, f32p]
        L.fo_quantize_nvfp4_act.argtypes = [u16p, c_int, c_int, c_int, u8p, u8p]
        L.fo_decode_e4m3.argtypes = [u8p, c_int64, f32p]
        L.fo_decode_nvfp4.argtypes = [u8p, u8p, c_int, c_int, f32p]
        L.fo_widen_16.argtypes = [u16p, c_int, c_int64, f32p]
        L.fo_narrow_16.argtypes = [f32p, c_int, c_int64, u16p]
        L.fo_gemm_f32_nt.argtypes = [f32p, f32p, f32p, c_int, c_int, c_int]
        L.fo_gemm_f64_nt.argtypes = [f32p, f32p, f64p, c_int, c_int, c_int]
        L.fo_epilogue.argtypes = [f32p, c_int, c_int, f32p, f32p, c_int, c_float, u16p, u16p,
                                  c_int, c_int, u16p]
        _lib = L
    return _lib


def _p(a: np.ndarray | None, ctype):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(POINTER(ctype))


# ---- codecs -------------------------------------------------------------------------------

def e4m3_decode_table() -> np.ndarray:
    return np.array([lib().fo_e4m3_decode(c) for c in range(256)], dtype=np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    L = lib()
    flat = np.ascontiguousarray(x, dtype=np.float32).ravel()
    return np.array([L.fo_e4m3_encode(float(v)) for v in flat], dtype=np.uint8).reshape(np.shape(x))


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    L = lib()
    flat = np.ascontiguousarray(x, dtype=np.float32).ravel()
    return np.array([L.fo_e2m1_encode(float(v)) for v in flat], dtype=np.uint8).reshape(np.shape(x))


def widen(x16: np.ndarray, is_bf16: bool) -> np.ndarray:
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    out = np.empty(x16.shape, dtype=np.float32)
    lib().fo_widen_16(_p(x16, c_uint16), int(is_bf16), x16.size, _p(out, c_float))
    return out


def narrow(x: np.ndarray, is_bf16: bool) -> np.ndarray:
    """float32 -> bf16/fp16 bit patterns, RNE (the C restatement's scalar helpers over the array;
    `narrow_numpy` is the independent vectorised form the pins compare it with)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().fo_narrow_16(_p(x, c_float), int(is_bf16), x.size, _p(out, c_uint16))
    return out


def narrow_numpy(x: np.ndarray, is_bf16: bool) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    if is_bf16:
        bits = x.view(np.uint32).astype(np.uint64)
        nan = (bits & 0x7FFFFFFF) > 0x7F800000
        rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
        rounded = np.where(nan, (bits >> 16) | 0x40, rounded)
        return rounded.astype(np.uint16)
    return x.astype(np.float16).view(np.uint16)  # numpy's cast is RNE


# ---- quantizers ---------------------------------------------------------------------------

def quantize_fp8_tensor(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.float32)
    codes = np.empty(w.shape, dtype=np.uint8)
    scale = np.zeros(1, dtype=np.float32)
    lib().fo_quantize_fp8_tensor(_p(w, c_float), w.size, _p(codes, c_uint8), _p(scale, c_float))
    return codes, scale


def quantize_fp8_rows(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    codes = np.empty((rows, k), dtype=np.uint8)
    scales = np.zeros(rows, dtype=np.float32)
    lib().fo_quantize_fp8_rows(_p(w, c_float), rows, k, _p(codes, c_uint8), _p(scales, c_float))
    return codes, scales


def quantize_fp8_act(x16: np.ndarray, is_bf16: bool):
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    rows, k = x16.shape
    codes = np.empty((rows, k), dtype=np.uint8)
    scales = np.zeros(rows, dtype=np.float32)
    lib().fo_quantize_fp8_act(_p(x16, c_uint16), int(is_bf16), rows, k, _p(codes, c_uint8), _p(scales, c_float))
    return codes, scales


def quantize_fp8_act_amax(x16: np.ndarray, amax: np.ndarray, is_bf16: bool):
    """quantize_fp8_act with the rows' maxima given (a column block of rows whose maxima were taken
    over the whole row): (codes, scales = amax / 448)."""
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    amax = np.ascontiguousarray(amax, dtype=np.float32)
    rows, k = x16.shape
    codes = np.empty((rows, k), dtype=np.uint8)
    scales = np.zeros(rows, dtype=np.float32)
    lib().fo_quantize_fp8_act_amax(_p(x16, c_uint16), int(is_bf16), rows, k, _p(amax, c_float), _p(codes, c_uint8),
                                   _p(scales, c_float))
    return codes, scales


def row_amax(x16: np.ndarray, is_bf16: bool) -> np.ndarray:
    """The largest magnitude of each row of a 16-bit matrix, as float32."""
    return np.abs(widen(np.ascontiguousarray(x16, dtype=np.uint16), is_bf16)).max(axis=-1).astype(np.float32)


def quantize_nvfp4_weight(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    assert k % 16 == 0
    codes = np.empty((rows, k // 2), dtype=np.uint8)
    sf = np.empty((rows, k // 16), dtype=np.uint8)
    g = np.zeros(1, dtype=np.float32)
    lib().fo_quantize_nvfp4_weight(_p(w, c_float), rows, k, _p(codes, c_uint8), _p(sf, c_uint8), _p(g, c_float))
    return codes, sf, g


def quantize_nvfp4_act(x16: np.ndarray, is_bf16: bool):
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    rows, k = x16.shape
    assert k % 16 == 0
    codes = np.empty((rows, k // 2), dtype=np.uint8)
    sf = np.empty((rows, k // 16), dtype=np.uint8)
    lib().fo_quantize_nvfp4_act(_p(x16, c_uint16), int(is_bf16), rows, k, _p(codes, c_uint8), _p(sf, c_uint8))
    return codes, sf


def layernorm_modulate(x16: np.ndarray, scale16, shift16, eps: float, is_bf16: bool) -> np.ndarray:
    """The consumer in front of a block's projection, as 16-bit values (m, k): flint's layerNorm
    without affine (float32: mean = sum / k, variance = sumsq / k - mean^2 with eps added where
    that is positive and standing alone where it is not, flint/cpu/normalizations.cc:98-140, the
    division by the deviation taken as one reciprocal per row; the two sums here are summed in
    float64 and rounded to float32 once, the value every float32 summation order approximates),
    then the reference's
    modulate, `normed * scale + normed` with each operation rounded to float32, an optional shift,
    and the cast to the narrow type (waifu/src/qwen_image/dit.rs:179-184). scale16/shift16 are
    (k) or (groups, k) bit patterns or None; row r belongs to group r // (m // groups)."""
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    m, k = x16.shape
    v = widen(x16, is_bf16)
    total = v.astype(np.float64).sum(axis=1).astype(np.float32)
    total_sq = (v.astype(np.float64) ** 2).sum(axis=1).astype(np.float32)
    mean = (total / np.float32(k)).astype(np.float32)
    var = ((total_sq / np.float32(k)).astype(np.float32) - (mean * mean).astype(np.float32)).astype(np.float32)
    var = np.where(var > 0, (var + np.float32(eps)).astype(np.float32), np.float32(eps)).astype(np.float32)
    rstd = (np.float32(1.0) / np.sqrt(var, dtype=np.float32)).astype(np.float32)
    y = ((v - mean[:, None]).astype(np.float32) * rstd[:, None]).astype(np.float32)

    def rows_of(mod):
        mod = widen(np.ascontiguousarray(mod, dtype=np.uint16).reshape(-1, k), is_bf16)
        groups = mod.shape[0]
        if m % groups:
            raise ValueError("rows do not divide into groups")
        return np.repeat(mod, m // groups, axis=0)

    if scale16 is not None:
        y = ((y * rows_of(scale16)).astype(np.float32) + y).astype(np.float32)
    if shift16 is not None:
        y = (y + rows_of(shift16)).astype(np.float32)
    return narrow(y, is_bf16)


def swiglu(x16: np.ndarray, is_bf16: bool) -> np.ndarray:
    """flint's swiglu on (m, 2 h) bit patterns -> (m, h): the first half of a row is the gate, the
    second the value; `g / (1 + exp(-g)) * v` in float32, each operation rounded, then the cast to
    the 16-bit type (flint/cpu/glu.cc:36-67)."""
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    h = x16.shape[1] // 2
    g, v = widen(x16[:, :h], is_bf16), widen(x16[:, h:], is_bf16)
    with np.errstate(over="ignore"):
        e = np.exp(-g.astype(np.float64)).astype(np.float32)  # the correctly rounded float32 exponential
        silu = (g / (np.float32(1.0) + e).astype(np.float32)).astype(np.float32)
    return narrow((silu * v).astype(np.float32), is_bf16)


def qk_norm_rope(qkv16: np.ndarray, cos: np.ndarray, sin: np.ndarray, heads: int, eps: float, is_bf16: bool,
                 q_weight16=None, k_weight16=None) -> np.ndarray:
    """The step between a fused q/k/v projection and attention on (rows, 3 * heads * head_dim) bit
    patterns: per row and q or k head flint's rmsNorm (`a * w / sqrt(mean(a^2) + eps)`, float32,
    flint/cpu/normalizations.cc:33-70; the mean of squares summed in float64 and rounded once)
    narrowed to the 16-bit type, then the even/odd pair rotation of waifu/src/krea2/dit.rs:260-275
    with every operation rounded to float32 and one final narrowing. cos, sin are float32
    (tokens, head_dim / 2); row r sits at position r % tokens. The v third is returned as it is."""
    qkv16 = np.ascontiguousarray(qkv16, dtype=np.uint16)
    rows, width = qkv16.shape
    head_dim = width // (3 * heads)
    tokens = cos.shape[0]
    out = qkv16.copy()
    x = widen(qkv16[:, :2 * heads * head_dim], is_bf16).reshape(rows, 2 * heads, head_dim)
    ms = ((x.astype(np.float64) ** 2).sum(axis=2) / head_dim).astype(np.float32)
    rms = np.sqrt(ms + np.float32(eps), dtype=np.float32)
    y = x
    if q_weight16 is not None or k_weight16 is not None:
        w = np.ones((2 * heads, head_dim), np.float32)
        if q_weight16 is not None:
            w[:heads] = widen(np.asarray(q_weight16, np.uint16), is_bf16)
        if k_weight16 is not None:
            w[heads:] = widen(np.asarray(k_weight16, np.uint16), is_bf16)
        y = (x * w[None]).astype(np.float32)
    inv = (np.float32(1.0) / rms).astype(np.float32)  # one reciprocal per head, as the GPU path takes it
    n = widen(narrow((y * inv[:, :, None]).astype(np.float32), is_bf16), is_bf16).reshape(rows, 2 * heads, head_dim // 2, 2)
    pos = np.arange(rows) % tokens
    c = np.asarray(cos, np.float32)[pos][:, None, :]
    s_ = np.asarray(sin, np.float32)[pos][:, None, :]
    even, odd = n[..., 0], n[..., 1]
    left = ((even * c).astype(np.float32) - (odd * s_).astype(np.float32)).astype(np.float32)
    right = ((even * s_).astype(np.float32) + (odd * c).astype(np.float32)).astype(np.float32)
    rot = np.stack([left, right], axis=-1).reshape(rows, 2 * heads * head_dim)
    out[:, :2 * heads * head_dim] = narrow(rot, is_bf16)
    return out


def attention_keep(mask, block_size: int, L: int, S: int):
    """Which keys each query may see (flint/capi.h:118-133, flint/cuda/attention.cu:165-179): query i
    sits at position p = i + S - L; `mask` is False/0 (every key), True/1 (causal: keys 0..p), 2
    (block causal: p's block of `block_size` keys and every block before it) or 3 (block diagonal:
    p's block alone). Returns a boolean (L, S) array, or None for no mask."""
    mask = int(mask)
    if mask == 0:
        return None
    pos = (np.arange(L) + (S - L))[:, None]
    key = np.arange(S)[None, :]
    if mask == 1:
        return key <= pos
    first = (pos // block_size) * block_size if mask == 3 else 0
    last = np.minimum(S - 1, (pos // block_size) * block_size + block_size - 1)
    return (key >= first) & (key <= last)


def attention(q16: np.ndarray, k16: np.ndarray, v16: np.ndarray, causal, is_bf16: bool, block_size: int = 0) -> np.ndarray:
    """Scaled dot product attention on 16-bit bit patterns, q (N, heads, L, D), k and v
    (N, kv_heads, S, D) with kv_heads dividing heads (query head h reads key-value head
    h // (heads / kv_heads), flint/operators.h:255-260): softmax(q k^T / sqrt(D)) v in float64,
    under the mask `causal` names (a bool, or a mask number with its `block_size`: see
    attention_keep). Returns float64; no intermediate is rounded, so a kernel that rounds its
    probabilities to 16 bits (flint/cuda/attention.cu:30-70, flint/operators.cc:170-175) agrees to
    that rounding."""
    q = widen(np.asarray(q16, np.uint16), is_bf16).astype(np.float64)
    k = widen(np.asarray(k16, np.uint16), is_bf16).astype(np.float64)
    v = widen(np.asarray(v16, np.uint16), is_bf16).astype(np.float64)
    n, heads, L, d = q.shape
    kv_heads, S = k.shape[1], k.shape[2]
    group = heads // kv_heads
    out = np.empty((n, heads, L, d), np.float64)
    keep = attention_keep(causal, block_size, L, S)
    for b in range(n):
        for h in range(heads):
            s = q[b, h] @ k[b, h // group].T / np.sqrt(float(d))
            if keep is not None:
                s = np.where(keep, s, -np.inf)
            s -= s.max(axis=1, keepdims=True)
            p = np.exp(s)
            out[b, h] = (p @ v[b, h // group]) / p.sum(axis=1, keepdims=True)
    return out


def decode_e4m3(codes: np.ndarray) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    out = np.empty(codes.shape, dtype=np.float32)
    lib().fo_decode_e4m3(_p(codes, c_uint8), codes.size, _p(out, c_float))
    return out


def decode_nvfp4(codes: np.ndarray, sf: np.ndarray) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    sf = np.ascontiguousarray(sf, dtype=np.uint8)
    rows, k = codes.shape[0], codes.shape[1] * 2
    out = np.empty((rows, k), dtype=np.float32)
    lib().fo_decode_nvfp4(_p(codes, c_uint8), _p(sf, c_uint8), rows, k, _p(out, c_float))
    return out


# ---- float32 product: the reference's own fl_matmul when built, else the C port ------------

class _Ref:
    """Minimal ctypes use of the reference's C ABI (flint/capi.h:151-234,440-446)."""

    def __init__(self):
        L = ctypes.CDLL(REF_SO)
        self.L = L
        L.fl_init.restype = None
        L.fl_get_last_error_message.restype = ctypes.c_char_p
        L.fl_operators_create.argtypes = [c_int, POINTER(c_void_p)]
        L.fl_tensor_data_borrow.argtypes = [c_void_p, c_int, c_int64, POINTER(c_void_p)]
        L.fl_tensor_data_destroy.argtypes = [c_void_p]; L.fl_tensor_data_destroy.restype = None
        L.fl_tensor_view_create.argtypes = [c_void_p, POINTER(c_int32), POINTER(c_int32), c_int32, c_int64, POINTER(c_void_p)]
        L.fl_tensor_view_destroy.argtypes = [c_void_p]; L.fl_tensor_view_destroy.restype = None
        L.fl_matmul.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p]
        L.fl_layer_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]
        L.fl_rms_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_float, c_void_p]
        L.fl_swiglu.argtypes = [c_void_p, c_void_p, c_void_p]
        L.fl_attention.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        try:
            L.fl_set_log_level.argtypes = [c_int32]
            L.fl_set_log_level.restype = None
            L.fl_set_log_level(3)  # errors only (flint/capi.h:672-690)
        except AttributeError:
            pass
        L.fl_init()
        self.ops = c_void_p()
        self._check(L.fl_operators_create(0, ctypes.byref(self.ops)))

    def _check(self, code):
        if code != 0:
            raise RuntimeError("reference flint: " + self.L.fl_get_last_error_message().decode())

    def _view(self, arr: np.ndarray, shape, stride):
        data = c_void_p()
        self._check(self.L.fl_tensor_data_borrow(arr.ctypes.data_as(c_void_p), 1, arr.size, ctypes.byref(data)))
        view = c_void_p()
        sh = (c_int32 * len(shape))(*shape)
        st = (c_int32 * len(stride))(*stride)
        self._check(self.L.fl_tensor_view_create(data, sh, st, len(shape), 0, ctypes.byref(view)))
        return data, view

    def matmul_nt(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        """a (m,k) times the transpose of b (n,k), both float32, through fl_matmul."""
        m, k = a.shape
        n = b.shape[0]
        out = np.empty((m, n), dtype=np.float32)
        da, va = self._view(a, (m, k), (k, 1))
        db, vb = self._view(b, (k, n), (1, k))  # the transpose as a view: no copy
        do, vo = self._view(out, (m, n), (n, 1))
        try:
            self._check(self.L.fl_matmul(self.ops, va, vb, vo))
        finally:
            for v in (va, vb, vo):
                self.L.fl_tensor_view_destroy(v)
            for d in (da, db, do):
                self.L.fl_tensor_data_destroy(d)
        return out


    def _unary(self, call, x: np.ndarray, out_cols: int, extra=()) -> np.ndarray:
        """Runs one of the reference's row operators on a float32 (rows, cols) array."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        out = np.empty((rows, out_cols), dtype=np.float32)
        dx, vx = self._view(x, (rows, cols), (cols, 1))
        do, vo = self._view(out, (rows, out_cols), (out_cols, 1))
        held = [(dx, vx), (do, vo)]
        try:
            args = []
            for e in extra:
                if isinstance(e, np.ndarray):
                    d, v = self._view(e, e.shape, (1,))
                    held.append((d, v))
                    args.append(v)
                else:
                    args.append(e)
            self._check(call(vx, args, vo))
        finally:
            for d, v in held:
                self.L.fl_tensor_view_destroy(v)
                self.L.fl_tensor_data_destroy(d)
        return out

    def layer_norm(self, x: np.ndarray, eps: float) -> np.ndarray:
        """fl_layer_norm without weight and bias (flint/capi.h:320-328)."""
        return self._unary(lambda vx, a, vo: self.L.fl_layer_norm(self.ops, vx, None, None, c_float(eps), vo), x, x.shape[1])

    def rms_norm(self, x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
        """fl_rms_norm (flint/capi.h:312-318); the weight is required there."""
        w = np.ascontiguousarray(weight, dtype=np.float32)
        return self._unary(lambda vx, a, vo: self.L.fl_rms_norm(self.ops, vx, a[0], c_float(eps), vo), x, x.shape[1], (w,))

    def swiglu(self, x: np.ndarray) -> np.ndarray:
        """fl_swiglu (flint/capi.h:517-519)."""
        return self._unary(lambda vx, a, vo: self.L.fl_swiglu(self.ops, vx, vo), x, x.shape[1] // 2)

    def attention(self, q: np.ndarray, k: np.ndarray, v: np.ndarray, causal, block_size: int = 0) -> np.ndarray:
        """fl_attention on the CPU device with float32 operands (flint/capi.h:532-544): q
        (N, heads, L, D), k and v (N, kv_heads, S, D), contiguous; `causal` a bool or a mask
        number (flint/capi.h:118-133) with its `block_size`."""
        arrs = [np.ascontiguousarray(t, dtype=np.float32) for t in (q, k, v)]
        out = np.empty(arrs[0].shape, dtype=np.float32)
        held = []
        try:
            for t in arrs + [out]:
                stride = [int(np.prod(t.shape[i + 1:])) for i in range(4)]
                held.append(self._view(t, t.shape, stride))
            self._check(self.L.fl_attention(self.ops, held[0][1], held[1][1], held[2][1], int(causal), int(block_size), held[3][1]))
        finally:
            for d, vw in held:
                self.L.fl_tensor_view_destroy(vw)
                self.L.fl_tensor_data_destroy(d)
        return out


_ref = None


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref() -> _Ref:
    global _ref
    if _ref is None:
        _ref = _Ref()
    return _ref


def gemm_f32_nt(a: np.ndarray, b: np.ndarray, engine: str = "auto") -> np.ndarray:
    """C = A Bt in float32. engine: "auto" (reference build if present), "reference", "port"."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    if engine == "reference" or (engine == "auto" and have_ref()):
        return ref().matmul_nt(a, b)
    m, k = a.shape
    n = b.shape[0]
    out = np.empty((m, n), dtype=np.float32)
    lib().fo_gemm_f32_nt(_p(a, c_float), _p(b, c_float), _p(out, c_float), m, n, k)
    return out


def gemm_f64_nt(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n = b.shape[0]
    out = np.empty((m, n), dtype=np.float64)
    lib().fo_gemm_f64_nt(_p(a, c_float), _p(b, c_float), _p(out, ctypes.c_double), m, n, k)
    return out


def epilogue(acc, row_scale=None, col_scale=None, global_scale=1.0, bias=None, residual=None,
             act=ACT_NONE, out_is_bf16=True) -> np.ndarray:
    acc = np.ascontiguousarray(acc, dtype=np.float32)
    m, n = acc.shape
    out = np.empty((m, n), dtype=np.uint16)
    cs = None if col_scale is None else np.ascontiguousarray(col_scale, dtype=np.float32).ravel()
    rs = None if row_scale is None else np.ascontiguousarray(row_scale, dtype=np.float32).ravel()
    if rs is not None:
        assert rs.size == m
    if cs is not None:
        assert cs.size in (1, n)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.uint16).ravel()
    r = None if residual is None else np.ascontiguousarray(residual, dtype=np.uint16).reshape(m, n)
    lib().fo_epilogue(_p(acc, c_float), m, n, _p(rs, c_float), _p(cs, c_float),
                      0 if cs is None else cs.size, float(global_scale), _p(b, c_uint16),
                      _p(r, c_uint16), int(act), int(out_is_bf16), _p(out, c_uint16))
    return out


# ---- the three linears, end to end ---------------------------------------------------------

def fp8_matmul(a16, codes, scale, addend=None, is_bf16=False, engine="auto"):
    """The reference's fl_fp8_matmul[_add] (flint/capi.cc:1047-1097): 16-bit activation, NOT
    narrowed, times the e4m3 weight's values, times one scale, plus addend, one rounding."""
    a16 = np.ascontiguousarray(a16, dtype=np.uint16)
    lead = a16.shape[:-1]
    k = a16.shape[-1]
    a = widen(a16.reshape(-1, k), is_bf16)
    w = decode_e4m3(codes)
    acc = gemm_f32_nt(a, w, engine)
    m, n = acc.shape
    bias = residual = None
    if addend is not None:
        addend = np.asarray(addend, dtype=np.uint16)
        if addend.size == n and addend.ndim == 1:
            bias = addend
        else:
            residual = np.broadcast_to(addend, lead + (n,)).reshape(m, n)
    out = epilogue(acc, None, np.asarray(scale, dtype=np.float32), 1.0, bias, residual, ACT_NONE, is_bf16)
    return out.reshape(lead + (n,))


def fp8_linear(x16, codes, scales, bias=None, residual=None, act=ACT_NONE, is_bf16=True, engine="auto"):
    """Dynamic per-token e4m3 activation x e4m3 weight (per-channel or per-tensor scale)."""
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    lead = x16.shape[:-1]
    k = x16.shape[-1]
    xc, xs = quantize_fp8_act(x16.reshape(-1, k), is_bf16)
    acc = gemm_f32_nt(decode_e4m3(xc), decode_e4m3(codes), engine)
    m, n = acc.shape
    res = None if residual is None else np.asarray(residual, dtype=np.uint16).reshape(m, n)
    out = epilogue(acc, xs, scales, 1.0, bias, res, act, is_bf16)
    return out.reshape(lead + (n,))


def fp8_linear_quantized(xc, xs, codes, scales, bias=None, residual=None, act=ACT_NONE, is_bf16=True, engine="auto"):
    """fp8_linear for an activation that is e4m3 codes (m, k) with per-row scales (m) already."""
    acc = gemm_f32_nt(decode_e4m3(np.ascontiguousarray(xc, dtype=np.uint8)), decode_e4m3(codes), engine)
    m, n = acc.shape
    res = None if residual is None else np.asarray(residual, dtype=np.uint16).reshape(m, n)
    return epilogue(acc, np.asarray(xs, dtype=np.float32), scales, 1.0, bias, res, act, is_bf16)


def nvfp4_linear(x16, codes, block_scales, global_scale, bias=None, residual=None, act=ACT_NONE,
                 is_bf16=True, engine="auto"):
    """Dynamic per-16-block e2m1 activation x NVFP4 weight, fp32 accumulate."""
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    lead = x16.shape[:-1]
    k = x16.shape[-1]
    xc, xsf = quantize_nvfp4_act(x16.reshape(-1, k), is_bf16)
    acc = gemm_f32_nt(decode_nvfp4(xc, xsf), decode_nvfp4(codes, block_scales), engine)
    m, n = acc.shape
    res = None if residual is None else np.asarray(residual, dtype=np.uint16).reshape(m, n)
    g = float(np.asarray(global_scale, dtype=np.float32).ravel()[0])
    out = epilogue(acc, None, None, g, bias, res, act, is_bf16)
    return out.reshape(lead + (n,))


# ---- error measures the parity tests use ---------------------------------------------------

def rel_l2(y: np.ndarray, ref_: np.ndarray) -> float:
    """flint/cuda/gemm_fp8_cutlass_test.cc:77-92 (relativeRmse)."""
    y = np.asarray(y, dtype=np.float64)
    ref_ = np.asarray(ref_, dtype=np.float64)
    den = float(np.sum(ref_ * ref_))
    num = float(np.sum((y - ref_) ** 2))
    if den == 0.0:
        return 0.0 if num == 0.0 else float("inf")
    return float(np.sqrt(num / den))


def ulp16_at(scale_value: float, is_bf16: bool) -> float:
    """One ulp of the 16-bit output type at the magnitude `scale_value`."""
    if scale_value <= 0 or not np.isfinite(scale_value):
        return 0.0
    e = int(np.floor(np.log2(scale_value)))
    return float(2.0 ** (e - (7 if is_bf16 else 10)))

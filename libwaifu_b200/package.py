"""Quantized weights on disk: the reference's package convention, read and written, and widened to
the two formats this library adds.

A package stores a quantized matrix as ordinary safetensors tensors paired by name
(docs/fp8.md:52-131 of the reference; reader waifu/src/tensor_file.rs:264-336, writer
tools/model_writer.py:143-182,601-618):

* ``fp8_tensor_scale`` (the reference's only FP8 format): ``"<name>"`` F8_E4M3 (rows, k) and
  ``"<name>.scale"`` F32 (1,);
* ``fp8_row_scale`` (new): the same pair with ``"<name>.scale"`` F32 (rows,), one scale per output
  channel, ``amax_row / 448`` -- what fl_fp8_linear multiplies by per channel;
* ``nvfp4`` (new): ``"<name>"`` U8 (rows, k / 2), two e2m1 codes a byte, the low nibble the even k;
  ``"<name>.block_scale"`` F8_E4M3 (rows, k / 16), unsigned e4m3; ``"<name>.scale"`` F32 (1,), the
  global scale ``amax / (448 * 6)``.

The manifest key ``weight_format`` names which one a package holds ("float" when absent); the
reader checks the pairing against it and refuses what does not fit, by name, as the reference's
reader does. The container is the safetensors layout (8-byte little-endian header length, a JSON
header of dtype / shape / data_offsets per tensor, then the bytes) written and parsed here with no
dependency.

The quantisers in this module are the exporter's arithmetic (numpy on the host, the counterpart
of tools/model_writer.py, which is torch on the host); they are not on the inference path, which
takes the stored codes as they are. ``upload_linear`` puts a stored matrix on the GPU as the
operands fl_fp8_matmul / fl_fp8_linear / fl_nvfp4_linear take.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, Iterable, Optional, Tuple

import numpy as np

SCALE_SUFFIX = ".scale"              # flint::SCALE_SUFFIX, tools/model_writer.py:184-186
BLOCK_SCALE_SUFFIX = ".block_scale"
WEIGHT_FORMATS = ("float", "fp8_tensor_scale", "fp8_row_scale", "nvfp4")
FP8_E4M3_MAX = 448.0
NVFP4_BLOCK = 16

# safetensors dtype string -> (numpy carrier dtype, bytes per element)
_CARRIER = {"F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2), "F8_E4M3": (np.uint8, 1),
            "U8": (np.uint8, 1), "I8": (np.int8, 1), "I32": (np.int32, 4), "I64": (np.int64, 8), "BOOL": (np.bool_, 1)}


class PackageError(ValueError):
    """A file or a set of tensors that is not what its weight format says."""


class StoredTensor:
    """One tensor of a file: its safetensors dtype string and a numpy array over a carrier type
    (F8_E4M3 and BF16 keep their bit patterns in uint8 / uint16)."""

    def __init__(self, dtype: str, array: np.ndarray):
        if dtype not in _CARRIER:
            raise PackageError(f"{dtype} is not an element type this reads")
        self.dtype = dtype
        self.array = np.ascontiguousarray(array, dtype=_CARRIER[dtype][0])

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self.array.shape)


# ---- the container ----------------------------------------------------------------------------

def write_safetensors(path: str, tensors: Dict[str, StoredTensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """Tensors in name order, each aligned as the format asks (the header is padded with spaces to
    a multiple of 8 bytes)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        size = t.array.size * _CARRIER[t.dtype][1]
        header[name] = {"dtype": t.dtype, "shape": list(t.shape), "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            f.write(tensors[name].array.tobytes())


def read_safetensors(path: str) -> Tuple[Dict[str, StoredTensor], Dict[str, str]]:
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise PackageError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n > 100 * 1024 * 1024:
            raise PackageError(f"{path}: a header of {n} bytes is not a safetensors file")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise PackageError(f"{path}: the header is not JSON ({e})") from None
        data = f.read()
    metadata = header.pop("__metadata__", {}) or {}
    out: Dict[str, StoredTensor] = {}
    for name, info in header.items():
        dtype, shape = info["dtype"], tuple(int(d) for d in info["shape"])
        if dtype not in _CARRIER:
            raise PackageError(f"{path}: tensor {name!r} is {dtype}, which is not an element type this reads")
        a, b = (int(v) for v in info["data_offsets"])
        carrier, width = _CARRIER[dtype]
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if a < 0 or b > len(data) or b - a != count * width:
            raise PackageError(f"{path}: tensor {name!r} has offsets {a}..{b} for {count} elements of {width} bytes")
        out[name] = StoredTensor(dtype, np.frombuffer(data, dtype=carrier, count=count, offset=a).reshape(shape))
    return out, metadata


# ---- the pairing rules ------------------------------------------------------------------------

def check_pairs(tensors: Dict[str, StoredTensor], weight_format: str, quantized: Optional[Iterable[str]] = None) -> None:
    """What the reference's check_fp8_pairs enforces (tensor_file.rs:283-336), for each format: every
    quantized matrix has the scale tensors its format needs beside it, of the right type and shape.
    Run over a whole model, since a weight and its scale may sit in different files. A tensor whose
    name merely ends in ".scale" is an ordinary tensor, as in the reference.

    NVFP4 codes are plain U8 bytes, which nothing tells apart from an ordinary uint8 tensor, so a
    package of that format names its quantized matrices (`quantized`, the "quantized" list of the
    file's metadata): each of them must be there with both companions. Without the list, every
    ".block_scale" tensor and every F32[1] ".scale" beside a U8 matrix is followed to its codes."""
    if weight_format not in WEIGHT_FORMATS:
        raise PackageError(f"weight_format {weight_format!r} is not one of {WEIGHT_FORMATS}")
    for name, t in tensors.items():
        if t.dtype != "F8_E4M3":
            continue
        if weight_format == "nvfp4" and name.endswith(BLOCK_SCALE_SUFFIX):
            continue  # the block scales of an nvfp4 weight; checked with their codes below
        if weight_format in ("float", "nvfp4"):
            raise PackageError(f"tensor {name!r} is float8_e4m3 in a package whose weight_format is {weight_format!r}")
        scale = tensors.get(name + SCALE_SUFFIX)
        if scale is None:
            raise PackageError(f"tensor {name!r} is float8_e4m3 and there is no {name + SCALE_SUFFIX!r} beside it; a "
                               "quantized weight is the elements and the scales, and the elements alone do not say "
                               "what they are worth")
        if len(t.shape) != 2:
            raise PackageError(f"tensor {name!r} is float8_e4m3 {t.shape}, and a quantized weight is a matrix")
        want = (1,) if weight_format == "fp8_tensor_scale" else (t.shape[0],)
        if scale.dtype != "F32" or scale.shape != want:
            hint = ("; a package with a scale per row is weight_format fp8_row_scale" if weight_format == "fp8_tensor_scale"
                    else "; one scale for the whole weight is weight_format fp8_tensor_scale")
            raise PackageError(f"tensor {name + SCALE_SUFFIX!r} is {scale.dtype}{list(scale.shape)}, and the scale of "
                               f"{name!r} has to be F32{list(want)} under {weight_format}{hint}")
    if weight_format != "nvfp4":
        return
    bases = set(quantized) if quantized is not None else set()
    for name, t in tensors.items():
        if name.endswith(BLOCK_SCALE_SUFFIX):
            bases.add(name[:-len(BLOCK_SCALE_SUFFIX)])
        elif name.endswith(SCALE_SUFFIX) and t.dtype == "F32" and t.shape == (1,):
            base = tensors.get(name[:-len(SCALE_SUFFIX)])
            if base is not None and base.dtype == "U8" and len(base.shape) == 2:
                bases.add(name[:-len(SCALE_SUFFIX)])
    for base in sorted(bases):
        codes, block, scale = tensors.get(base), tensors.get(base + BLOCK_SCALE_SUFFIX), tensors.get(base + SCALE_SUFFIX)
        if codes is None:
            raise PackageError(f"the nvfp4 weight {base!r} has scales but no codes tensor {base!r}")
        if block is None:
            raise PackageError(f"the nvfp4 weight {base!r} has no {base + BLOCK_SCALE_SUFFIX!r} beside it")
        if scale is None:
            raise PackageError(f"the nvfp4 weight {base!r} has no {base + SCALE_SUFFIX!r} beside it")
        if codes.dtype != "U8" or len(codes.shape) != 2:
            raise PackageError(f"the codes of the nvfp4 weight {base!r} are {codes.dtype}{list(codes.shape)}, not a U8 matrix")
        if block.dtype != "F8_E4M3":
            raise PackageError(f"{base + BLOCK_SCALE_SUFFIX!r} is {block.dtype}, and block scales are F8_E4M3")
        if scale.dtype != "F32" or scale.shape != (1,):
            raise PackageError(f"{base + SCALE_SUFFIX!r} is {scale.dtype}{list(scale.shape)}, and the global scale is F32[1]")
        if block.shape != (codes.shape[0], codes.shape[1] * 2 // NVFP4_BLOCK) or (codes.shape[1] * 2) % NVFP4_BLOCK:
            raise PackageError(f"the nvfp4 weight {base!r} has codes {list(codes.shape)} and block scales "
                               f"{list(block.shape)}; the latter has to be [rows, k / 16] for codes [rows, k / 2]")


# ---- the exporter's arithmetic ----------------------------------------------------------------

def _e4m3_codes(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn bit patterns, round to nearest even, saturating at +-448 (the clamp and the
    cast of tools/model_writer.py:170-172), NaN -> 0x7f. Pure integer arithmetic on the float32
    bits, vectorised."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    mag = np.abs(x)
    nan = np.isnan(x)
    mag = np.minimum(np.where(nan, 0, mag), np.float32(FP8_E4M3_MAX)).astype(np.float32)
    # normal e4m3: exponent >= -6; below that the step is fixed at 2^-9
    exp = np.floor(np.log2(np.maximum(mag, np.float32(2.0 ** -20)))).astype(np.int32)
    exp = np.maximum(exp, -6)
    step = np.ldexp(np.float32(1.0), exp - 3).astype(np.float32)         # 3 mantissa bits
    q = np.rint(mag / step).astype(np.int64)                             # rint is round-half-even
    # q in [0, 16]: 16 means the mantissa carried into the next exponent
    carry = q == 16
    exp = np.where(carry, exp + 1, exp)
    q = np.where(carry, 8, q)
    sub = q < 8                                                           # subnormal (only when exp == -6)
    code = np.where(sub, q, ((exp + 7) << 3) | (q - 8)).astype(np.int64)
    code = np.minimum(code, 0x7e)
    out = (code.astype(np.uint8) | sign)
    return np.where(nan, np.uint8(0x7f), out).astype(np.uint8)


_E4M3_TABLE = None


def e4m3_values() -> np.ndarray:
    """The 256 values of e4m3fn (NaN at 0x7f / 0xff)."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        c = np.arange(256, dtype=np.int64)
        e, m = (c >> 3) & 0xf, c & 7
        v = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1 + m / 8.0) * np.exp2(e - 7.0))
        v = np.where((c & 0x7f) == 0x7f, np.nan, v)
        _E4M3_TABLE = np.where(c & 0x80, -v, v).astype(np.float32)
    return _E4M3_TABLE


def quantize_fp8_tensor_scale(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """tools/model_writer.py:143-174: scale = amax / 448 (float32), data = e4m3(w / scale), divisor 1
    for an all-zero matrix."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2:
        raise PackageError(f"fp8 takes a matrix, not {w.shape}")
    scale = np.float32(np.abs(w).max() / np.float32(FP8_E4M3_MAX)) if w.size else np.float32(0)
    divisor = scale if scale > 0 else np.float32(1)
    return _e4m3_codes((w / divisor).astype(np.float32)), np.array([scale], np.float32)


def quantize_fp8_row_scale(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """The same recipe per output row."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2:
        raise PackageError(f"fp8 takes a matrix, not {w.shape}")
    scale = (np.abs(w).max(axis=1) / np.float32(FP8_E4M3_MAX)).astype(np.float32)
    divisor = np.where(scale > 0, scale, np.float32(1)).astype(np.float32)
    return _e4m3_codes((w / divisor[:, None]).astype(np.float32)), scale


_E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def _e2m1_codes(x: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit e2m1 codes (sign in bit 3), nearest with ties to the even code, saturating
    at +-6."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    mag = np.minimum(np.abs(x), np.float32(6.0))
    # midpoints between neighbouring magnitudes; a tie goes to the code with an even mantissa bit
    mids = (_E2M1_MAGNITUDES[:-1] + _E2M1_MAGNITUDES[1:]) / 2
    idx = np.zeros(x.shape, np.int64)
    for i, mid in enumerate(mids):
        up_on_tie = (i + 1) % 2 == 0  # the upper neighbour's code is even
        idx += (mag > mid) | ((mag == mid) & up_on_tie)
    return (idx | np.where(np.signbit(x), 8, 0)).astype(np.uint8)


def quantize_nvfp4(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """global = amax / (448 * 6); per 16 consecutive k: block scale = e4m3(amax_block / (6 global)),
    codes = e2m1(w * (1 / (value(block scale) * global))), a zero block -> scale 0 and codes 0.
    Returns packed codes (rows, k / 2), block scale codes (rows, k / 16), global scale (1,)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2 or w.shape[1] % NVFP4_BLOCK:
        raise PackageError(f"nvfp4 takes a matrix whose k is a multiple of 16, not {w.shape}")
    rows, k = w.shape
    g = np.float32(np.abs(w).max() / np.float32(FP8_E4M3_MAX * 6.0)) if w.size else np.float32(0)
    blocks = w.reshape(rows, k // NVFP4_BLOCK, NVFP4_BLOCK)
    amax = np.abs(blocks).max(axis=2)
    if g > 0:
        sc = _e4m3_codes((amax / (np.float32(6.0) * g).astype(np.float32)).astype(np.float32))
    else:
        sc = np.zeros(amax.shape, np.uint8)
    denom = (e4m3_values()[sc] * g).astype(np.float32)
    ok = denom > 0
    inv = np.where(ok, np.float32(1.0) / np.where(ok, denom, np.float32(1)), np.float32(0)).astype(np.float32)
    q = _e2m1_codes((blocks * inv[:, :, None]).astype(np.float32))
    q = np.where(ok[:, :, None], q, 0).astype(np.uint8).reshape(rows, k)
    sc = np.where(ok, sc, 0).astype(np.uint8)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return packed, sc, np.array([g], np.float32)


def quantize_matrices(tensors: Dict[str, np.ndarray], names: Iterable[str], weight_format: str) -> Dict[str, StoredTensor]:
    """The exporter's pass over a model: the named float32 matrices are stored in `weight_format`,
    everything else as it is (float32, or the carrier type it already has)."""
    if weight_format not in WEIGHT_FORMATS:
        raise PackageError(f"weight_format {weight_format!r} is not one of {WEIGHT_FORMATS}")
    chosen = set(names)
    out: Dict[str, StoredTensor] = {}
    for name, value in tensors.items():
        if name not in chosen or weight_format == "float":
            out[name] = value if isinstance(value, StoredTensor) else StoredTensor("F32", np.asarray(value, np.float32))
            continue
        w = np.asarray(value, np.float32)
        if weight_format == "fp8_tensor_scale":
            codes, scale = quantize_fp8_tensor_scale(w)
            out[name], out[name + SCALE_SUFFIX] = StoredTensor("F8_E4M3", codes), StoredTensor("F32", scale)
        elif weight_format == "fp8_row_scale":
            codes, scale = quantize_fp8_row_scale(w)
            out[name], out[name + SCALE_SUFFIX] = StoredTensor("F8_E4M3", codes), StoredTensor("F32", scale)
        else:
            codes, block, g = quantize_nvfp4(w)
            out[name] = StoredTensor("U8", codes)
            out[name + BLOCK_SCALE_SUFFIX] = StoredTensor("F8_E4M3", block)
            out[name + SCALE_SUFFIX] = StoredTensor("F32", g)
    return out


def write_package(path: str, tensors: Dict[str, np.ndarray], names: Iterable[str], weight_format: str) -> None:
    """One safetensors file whose metadata carries the manifest's `weight_format`."""
    names = [n for n in names]
    stored = quantize_matrices(tensors, names, weight_format)
    quantized = sorted(n for n in names if n in tensors) if weight_format != "float" else []
    check_pairs(stored, weight_format, quantized)
    write_safetensors(path, stored, {"weight_format": weight_format, "quantized": json.dumps(quantized)})


def read_package(path: str, weight_format: Optional[str] = None) -> Tuple[Dict[str, StoredTensor], str]:
    """Reads a file and checks it against its weight format (the argument, else the file's own
    metadata, else "float")."""
    tensors, metadata = read_safetensors(path)
    fmt = weight_format or metadata.get("weight_format", "float")
    quantized = None
    if "quantized" in metadata:
        try:
            quantized = [str(n) for n in json.loads(metadata["quantized"])]
        except (ValueError, TypeError):
            raise PackageError(f"{path}: the metadata's list of quantized matrices is not a JSON list") from None
    check_pairs(tensors, fmt, quantized)
    return tensors, fmt


# ---- onto the GPU -----------------------------------------------------------------------------

def upload_linear(tensors: Dict[str, StoredTensor], name: str, weight_format: str):
    """The operands of one stored matrix as device tensors of the C ABI (weights get the
    FL_ALLOC_WEIGHT hint): fp8_tensor_scale / fp8_row_scale -> (codes, scales) for fl_fp8_matmul /
    fl_fp8_linear; nvfp4 -> (codes, block_scales, global_scale) for fl_nvfp4_linear."""
    from . import flint as F
    needs = {"fp8_tensor_scale": (SCALE_SUFFIX,), "fp8_row_scale": (SCALE_SUFFIX,),
             "nvfp4": (BLOCK_SCALE_SUFFIX, SCALE_SUFFIX)}.get(weight_format, ())
    for suffix in ("",) + needs:
        if name + suffix not in tensors:
            raise PackageError(f"{name + suffix!r} is not in the package")
    t = tensors[name]
    if weight_format in ("fp8_tensor_scale", "fp8_row_scale"):
        codes = F.Tensor.from_numpy(t.array, F.DType.FP8E4M3, F.Device.CUDA)
        scales = F.Tensor.from_numpy(tensors[name + SCALE_SUFFIX].array, F.DType.FLOAT, F.Device.CUDA)
        return codes, scales
    if weight_format == "nvfp4":
        codes = F.Tensor.from_numpy(t.array, F.DType.FP4E2M1X2, F.Device.CUDA)
        block = F.Tensor.from_numpy(tensors[name + BLOCK_SCALE_SUFFIX].array, F.DType.FP8E4M3, F.Device.CUDA)
        g = F.Tensor.from_numpy(tensors[name + SCALE_SUFFIX].array, F.DType.FLOAT, F.Device.CUDA)
        return codes, block, g
    raise PackageError(f"{name!r}: weight_format {weight_format!r} holds no quantized matrix to upload")

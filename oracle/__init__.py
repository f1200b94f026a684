"""CPU oracle for the compressed data-parallel gradient path.

TEST INFRASTRUCTURE ONLY: the checker for the CUDA library, never part of the
product.  Only the test-suite, the smoke check and the benchmark's CPU-baseline
leg may import this package; the shipped package never does.

`build()` compiles `grad_oracle.c` (a plain-C restatement of the reference's
CPU codec, reducers and clip arithmetic) into `libgrad_oracle.so` next to it.
The functions below are thin numpy wrappers over that library.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SOURCE = os.path.join(_HERE, "grad_oracle.c")
_LIBRARY = os.path.join(_HERE, "libgrad_oracle.so")
_FLAGS = ["-O2", "-fno-fast-math", "-ffp-contract=off", "-fPIC", "-shared",
          "-std=c11", "-Wall", "-Wextra"]

OK, ERR_ARGUMENT, ERR_NON_FINITE, ERR_BAD_SCALE = 0, 1, 2, 3


class OracleError(ValueError):
    """Raised where the reference's CPU codec would throw."""

    def __init__(self, code: int):
        names = {ERR_ARGUMENT: "invalid argument",
                 ERR_NON_FINITE: "BFP8 encoding requires finite input values",
                 ERR_BAD_SCALE: "every BFP8 scale must be finite and positive"}
        super().__init__(names.get(code, f"oracle status {code}"))
        self.code = code


def build(force: bool = False) -> str:
    """Compile the oracle (OpenMP when a compiler that has it is found)."""
    if (not force and os.path.exists(_LIBRARY)
            and os.path.getmtime(_LIBRARY) >= os.path.getmtime(_SOURCE)):
        return _LIBRARY
    compilers = [c for c in ("/usr/bin/gcc", shutil.which("gcc"), shutil.which("cc")) if c]
    errors = []
    for openmp in (["-fopenmp"], []):
        for compiler in compilers:
            cmd = [compiler, *_FLAGS, *openmp, _SOURCE, "-o", _LIBRARY, "-lm"]
            done = subprocess.run(cmd, capture_output=True, text=True)
            if done.returncode == 0:
                return _LIBRARY
            errors.append(f"{' '.join(cmd)}\n{done.stderr}")
    raise RuntimeError("could not build the CPU oracle:\n" + "\n".join(errors))


def build_reference_kernels(reference_root: str | None = None) -> str | None:
    """Compile the reference's own CUDA kernels (unmodified) into
    oracle/_ref/libref_grad.so from the reference tree at `reference_root` (or
    $NNTRAIN_REFERENCE_ROOT); without a tree keep whatever prebuilt file is
    there.  Returns its path or None."""
    script = os.path.join(_HERE, "build_ref.sh")
    target = os.path.join(_HERE, "_ref", "libref_grad.so")
    root = reference_root or os.environ.get("NNTRAIN_REFERENCE_ROOT", "")
    if root and os.path.isdir(root) and not os.path.exists(target):
        subprocess.run(["bash", script], check=True, env=dict(os.environ, NNTRAIN_REFERENCE_ROOT=root))
    return target if os.path.exists(target) else None


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        i64, f32, f64, vp, ci = (ctypes.c_int64, ctypes.c_float, ctypes.c_double,
                                 ctypes.c_void_p, ctypes.c_int)
        sig = {
            "oracle_set_threads": (None, [ci]),
            "oracle_max_threads": (ci, []),
            "oracle_bfp8_scale_count": (i64, [i64, i64]),
            "oracle_bfp8_encode": (ci, [vp, i64, i64, vp, vp, ci]),
            "oracle_bfp8_decode": (ci, [vp, vp, i64, i64, vp, ci]),
            "oracle_bfp8_reduce": (ci, [vp, vp, ci, i64, i64, f32, vp, vp]),
            "oracle_block_transport_sum": (ci, [vp, vp, ci, i64, i64, vp, vp]),
            "oracle_pack_bfp8_block": (ci, [vp, i64, i64, vp, vp]),
            "oracle_bfp8_gradient_publish": (ci, [vp, i64, i64, vp, vp, vp, vp]),
            "oracle_bf16_encode": (ci, [vp, i64, vp, ci]),
            "oracle_bf16_decode": (ci, [vp, i64, vp]),
            "oracle_bf16_reduce": (ci, [vp, ci, i64, f32, vp, vp, vp, ci]),
            "oracle_squared_sum_f32": (f64, [vp, i64]),
            "oracle_squared_sum_bf16": (f64, [vp, i64]),
            "oracle_squared_sum_bfp8": (f64, [vp, vp, i64, i64]),
            "oracle_clip_coefficient": (f32, [f64, f32, vp]),
            "oracle_scale_f32": (None, [vp, i64, f32]),
            "oracle_scale_bf16": (None, [vp, i64, f32]),
            "oracle_scale_bfp8_scales": (None, [vp, i64, f32]),
            "oracle_generate_gradient": (None, [vp, i64, i64, i64, ctypes.c_uint64,
                                                ctypes.c_uint64, i64, f64, f64, f64, f64, ci]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = res, args
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _check(code: int) -> None:
    if code != OK:
        raise OracleError(code)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def set_threads(threads: int) -> None:
    lib().oracle_set_threads(int(threads))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def scale_count(length: int, block: int) -> int:
    return int(lib().oracle_bfp8_scale_count(length, block))


def encode(source, block: int = 0, strict: bool = True):
    """(payload int8[n], scales float32[ceil(n/block)]); block 0 = tensor-wide."""
    source = _c(source, np.float32).ravel()
    n = source.size
    payload = np.empty(n, np.int8)
    scales = np.empty(scale_count(n, block), np.float32)
    _check(lib().oracle_bfp8_encode(_p(source), n, block, _p(payload), _p(scales), int(strict)))
    return payload, scales


def decode(payload, scales, block: int = 0, strict: bool = True) -> np.ndarray:
    payload = _c(payload, np.int8).ravel()
    scales = _c(scales, np.float32).ravel()
    out = np.empty(payload.size, np.float32)
    _check(lib().oracle_bfp8_decode(_p(payload), _p(scales), payload.size, block, _p(out), int(strict)))
    return out


def _pointer_array(arrays):
    return (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])


def reduce_bfp8(payloads, scales, block: int = 0, reduction_scale: float = 1.0):
    """fp32 r = s * (rank-ordered sum of decoded shards); returns (r, non_finite)."""
    payloads = [_c(p, np.int8).ravel() for p in payloads]
    scales = [_c(s, np.float32).ravel() for s in scales]
    n = payloads[0].size
    out = np.empty(n, np.float32)
    flag = ctypes.c_int(0)
    _check(lib().oracle_bfp8_reduce(_pointer_array(payloads), _pointer_array(scales), len(payloads),
                                    n, block, reduction_scale, _p(out), ctypes.addressof(flag)))
    return out, int(flag.value)


def allreduce_bfp8(gradients, block: int = 0, reduction_scale: float = 1.0):
    """The reducer's whole result for N replicas' fp32 gradients:
    encode each, rank-ordered fp32 sum, re-encode; fp32 ends as
    decode(encode(sum)).  Returns (payload, scales, fp32, squared_sum)."""
    encoded = [encode(g, block, strict=False) for g in gradients]
    r, _ = reduce_bfp8([e[0] for e in encoded], [e[1] for e in encoded], block, reduction_scale)
    payload, scales = encode(r, block, strict=False)
    final = decode(payload, scales, block, strict=False)
    return payload, scales, final, squared_sum_bfp8(payload, scales, block)


def block_transport_sum(payloads, scales, block: int = 128):
    payloads = [_c(p, np.int8).ravel() for p in payloads]
    scales = [_c(s, np.float32).ravel() for s in scales]
    n = payloads[0].size
    out = np.empty(n, np.float32)
    sq = ctypes.c_double(0.0)
    _check(lib().oracle_block_transport_sum(_pointer_array(payloads), _pointer_array(scales),
                                            len(payloads), n, block, _p(out), ctypes.addressof(sq)))
    return out, float(sq.value)


def pack_bfp8_block(source, block: int = 128):
    source = _c(source, np.float32).ravel()
    n = source.size
    payload = np.empty(n, np.int8)
    scales = np.empty((n + block - 1) // block, np.float32)
    _check(lib().oracle_pack_bfp8_block(_p(source), n, block, _p(payload), _p(scales)))
    return payload, scales


def gradient_publish(gradient, block: int = 0, finite_status: int = 0, want_squared_sum: bool = True,
                     payload=None):
    """Returns (gradient_after, payload, scales, finite_status, squared_sum)."""
    g = np.array(gradient, dtype=np.float32, copy=True).ravel()
    n = g.size
    payload = np.zeros(n, np.int8) if payload is None else np.array(payload, np.int8, copy=True)
    scales = np.zeros(scale_count(n, block), np.float32)
    flag = ctypes.c_int(finite_status)
    sq = ctypes.c_double(0.0)
    _check(lib().oracle_bfp8_gradient_publish(_p(g), n, block, _p(payload), _p(scales),
                                              ctypes.addressof(flag),
                                              ctypes.addressof(sq) if want_squared_sum else None))
    return g, payload, scales, int(flag.value), float(sq.value)


def bf16_encode(source, rule: int = 1) -> np.ndarray:
    """rule 0 = the C# codec's NaN handling, 1 = CUDA __float2bfloat16_rn."""
    source = _c(source, np.float32).ravel()
    out = np.empty(source.size, np.uint16)
    _check(lib().oracle_bf16_encode(_p(source), source.size, _p(out), rule))
    return out


def bf16_decode(source) -> np.ndarray:
    source = _c(source, np.uint16).ravel()
    out = np.empty(source.size, np.float32)
    _check(lib().oracle_bf16_decode(_p(source), source.size, _p(out)))
    return out


def bf16_reduce(inputs, reduction_scale: float = 1.0, want_bf16: bool = False,
                square_of_bf16: bool = False):
    """Returns (fp32 sum, bf16 re-encoded or None, squared_sum)."""
    inputs = [_c(a, np.uint16).ravel() for a in inputs]
    n = inputs[0].size
    reduced = np.empty(n, np.float32)
    out16 = np.empty(n, np.uint16) if want_bf16 else None
    sq = ctypes.c_double(0.0)
    _check(lib().oracle_bf16_reduce(_pointer_array(inputs), len(inputs), n, reduction_scale,
                                    _p(reduced), _p(out16) if want_bf16 else None,
                                    ctypes.addressof(sq), int(square_of_bf16)))
    return reduced, out16, float(sq.value)


def squared_sum_f32(values) -> float:
    values = _c(values, np.float32).ravel()
    return float(lib().oracle_squared_sum_f32(_p(values), values.size))


def squared_sum_bf16(values) -> float:
    values = _c(values, np.uint16).ravel()
    return float(lib().oracle_squared_sum_bf16(_p(values), values.size))


def squared_sum_bfp8(payload, scales, block: int = 0) -> float:
    payload = _c(payload, np.int8).ravel()
    scales = _c(scales, np.float32).ravel()
    return float(lib().oracle_squared_sum_bfp8(_p(payload), _p(scales), payload.size, block))


def clip_coefficient(squared_sum: float, max_norm: float):
    """(pre-clip norm, coefficient); coefficient is 1.0 when norm <= max_norm."""
    c = ctypes.c_float(1.0)
    norm = lib().oracle_clip_coefficient(squared_sum, max_norm, ctypes.addressof(c))
    return float(norm), float(c.value)


def scale_f32(values, multiplier: float) -> np.ndarray:
    out = np.array(values, np.float32, copy=True).ravel()
    lib().oracle_scale_f32(_p(out), out.size, multiplier)
    return out


def scale_bf16(values, multiplier: float) -> np.ndarray:
    out = np.array(values, np.uint16, copy=True).ravel()
    lib().oracle_scale_bf16(_p(out), out.size, multiplier)
    return out


def scale_bfp8_scales(scales, multiplier: float) -> np.ndarray:
    out = np.array(scales, np.float32, copy=True).ravel()
    lib().oracle_scale_bfp8_scales(_p(out), out.size, multiplier)
    return out


def generate_gradient(length: int, seed: int, replica: int = 0, offset: int = 0,
                      total_length: int | None = None, slice_elements: int = 65536,
                      sigma_lo: float = 1e-5, sigma_hi: float = 1e-2,
                      outlier_fraction: float = 0.01, zero_fraction: float = 0.005,
                      subnormals: int = 8) -> np.ndarray:
    """Seeded synthetic gradient slice (counter-based; see grad_oracle.c)."""
    out = np.empty(length, np.float32)
    total = offset + length if total_length is None else total_length
    lib().oracle_generate_gradient(_p(out), length, offset, total, seed, replica, slice_elements,
                                   sigma_lo, sigma_hi, outlier_fraction, zero_fraction, subnormals)
    return out


def adamw_step(data, gradient, first_moment, second_moment, beta1, beta2, learning_rate, weight_decay,
               update_scale, scaled_epsilon, apply_weight_decay=True):
    """One AdamW step in binary32, operation by operation as the reference's
    adamw_kernel writes it (NNtrain.Cuda/native/tensor_kernels.cu:1148-1174),
    every operation rounded separately.  Returns (data, first, second)."""
    f = np.float32
    g = _c(gradient, np.float32).ravel()
    p, m, v = (np.array(a, np.float32, copy=True).ravel() for a in (data, first_moment, second_moment))
    b1, b2 = f(beta1), f(beta2)
    first = (b1 * m).astype(f) + ((f(1) - b1) * g).astype(f)
    second = (b2 * v).astype(f) + (((f(1) - b2) * g).astype(f) * g).astype(f)
    if apply_weight_decay:
        p = (p * (f(1) - f(learning_rate) * f(weight_decay))).astype(f)
    denominator = (np.sqrt(second).astype(f) + f(scaled_epsilon)).astype(f)
    p = (p - ((f(update_scale) * first).astype(f) / denominator).astype(f)).astype(f)
    return p, first.astype(f), second.astype(f)

"""Runs the reference project's own CUDA kernels (compiled unmodified into
oracle/_ref/libref_grad.so by oracle/build_ref.sh) on small inputs.  Test
infrastructure: used to pin the CPU oracle and to record golden fixtures."""
import ctypes
import os

import numpy as np
import torch

REF_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", "libref_grad.so")


def available() -> bool:
    return os.path.exists(REF_PATH) and torch.cuda.is_available()


_ref = None


def ref():
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(REF_PATH)     # RTLD_LOCAL: its symbols stay private
    return _ref


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _ok(status, what):
    if status != 0:
        raise RuntimeError(f"reference {what} returned {status}")


def codec(source: np.ndarray, block: int):
    """nntrain_cuda_bfp8_quantize_f32 + _dequantize_f32; block 0 = tensor-wide."""
    n = source.size
    eb = n if block <= 0 or block >= n else block
    src = _dev(source.astype(np.float32))
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scales = torch.zeros((n + eb - 1) // eb, dtype=torch.float32, device="cuda")
    decoded = torch.zeros(n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    _ok(ref().nntrain_cuda_bfp8_quantize_f32(0, _p(src), _p(payload), _p(scales), n, eb, None), "quantize")
    _ok(ref().nntrain_cuda_bfp8_dequantize_f32(0, _p(payload), _p(scales), _p(decoded), n, eb, None), "dequantize")
    torch.cuda.synchronize()
    return payload.cpu().numpy(), scales.cpu().numpy(), decoded.cpu().numpy()


def pack_bfp8_block(source: np.ndarray):
    n = source.size
    src = _dev(source.astype(np.float32))
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scales = torch.zeros((n + 127) // 128, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    _ok(ref().nntrain_gradient_pack_bfp8_block(0, _p(src), _p(payload), _p(scales), n, None), "pack_bfp8_block")
    torch.cuda.synchronize()
    return payload.cpu().numpy(), scales.cpu().numpy()


def pack_bf16(source: np.ndarray):
    n = source.size
    src = _dev(source.astype(np.float32))
    out = torch.zeros(n, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    _ok(ref().nntrain_gradient_pack_bf16(0, _p(src), _p(out), 0, n, None), "pack_bf16")
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint16)


def _events():
    stream, a, b = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
    _ok(ref().nntrain_gradient_comm_create(0, ctypes.byref(stream)), "comm_create")
    _ok(ref().nntrain_gradient_event_create(0, ctypes.byref(a)), "event_create")
    _ok(ref().nntrain_gradient_event_create(0, ctypes.byref(b)), "event_create")
    _ok(ref().nntrain_gradient_record_ready(0, a, None), "record_ready")
    _ok(ref().nntrain_gradient_record_ready(0, b, None), "record_ready")
    return stream, a, b


def _release(stream, a, b):
    ref().nntrain_gradient_comm_synchronize(0, stream)
    ref().nntrain_gradient_event_destroy(0, a)
    ref().nntrain_gradient_event_destroy(0, b)
    ref().nntrain_gradient_comm_destroy(0, stream)


def block_transport_sum(pa, sa, pb, sb):
    """nntrain_gradient_exchange_bfp8_block with both 'devices' = 0."""
    n = pa.size
    local, ls, remote, rs = _dev(pa), _dev(sa), _dev(pb), _dev(sb)
    staging = torch.zeros(n, dtype=torch.int8, device="cuda")
    staging_scales = torch.zeros_like(rs)
    reduced = torch.zeros(n, dtype=torch.float32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    stream, a, b = _events()
    _ok(ref().nntrain_gradient_exchange_bfp8_block(0, 0, _p(local), _p(ls), _p(remote), _p(rs), _p(staging),
                                                   _p(staging_scales), _p(reduced), n, _p(sq), stream, a, b),
        "exchange_bfp8_block")
    _release(stream, a, b)
    torch.cuda.synchronize()
    return reduced.cpu().numpy(), float(sq.item())


def bf16_transport_sum(a_bits, b_bits):
    n = a_bits.size
    local = torch.from_numpy(a_bits.view(np.int16).copy()).cuda()
    remote = torch.from_numpy(b_bits.view(np.int16).copy()).cuda()
    staging = torch.zeros(n, dtype=torch.int16, device="cuda")
    reduced = torch.zeros(n, dtype=torch.float32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    stream, a, b = _events()
    _ok(ref().nntrain_gradient_exchange_bf16(0, 0, _p(local), _p(remote), _p(staging), _p(reduced), n, _p(sq),
                                             stream, a, b), "exchange_bf16")
    _release(stream, a, b)
    torch.cuda.synchronize()
    return reduced.cpu().numpy(), float(sq.item())


def gradient_publish(source: np.ndarray):
    """nntrain_bfp8_gradient_quantize_accumulate (tensor-wide)."""
    n = source.size
    g = _dev(source.astype(np.float32))
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scale = torch.zeros(1, dtype=torch.float32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    _ok(ref().nntrain_bfp8_gradient_quantize_accumulate(0, _p(g), _p(payload), _p(scale), n, _p(flag), _p(sq), None),
        "gradient_quantize_accumulate")
    torch.cuda.synchronize()
    return g.cpu().numpy(), payload.cpu().numpy(), scale.cpu().numpy(), int(flag.item()), float(sq.item())

"""Helpers for the GPU parity tests: device buffers (torch owns the memory), layout
conversion between the boundary NCHW fp32 and the device's channels-last tensors."""
import ctypes as C

import numpy as np

from paella_b200 import capi


def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    return torch


def vec(dtype):
    return 4 if dtype == 0 else 8


def round_up(a, b):
    return (a + b - 1) // b * b


def to_device_cl(x_chw, dtype):
    """[C][H][W] fp32 numpy -> device [H][W][Cs] tensor (fp32 or bf16), padded channels zero."""
    torch = torch_cuda()
    c, h, w = x_chw.shape
    cs = round_up(c, vec(dtype))
    buf = np.zeros((h, w, cs), np.float32)
    buf[:, :, :c] = np.transpose(x_chw, (1, 2, 0))
    t = torch.from_numpy(buf).cuda()
    return (t if dtype == 0 else t.to(torch.bfloat16)).contiguous(), cs


def from_device_cl(t, c):
    """device [H][W][Cs] -> [C][H][W] fp32 numpy"""
    return np.ascontiguousarray(np.transpose(t.float().cpu().numpy()[:, :, :c], (2, 0, 1)))


def empty_cl(h, w, c, dtype, fill=0.0):
    torch = torch_cuda()
    cs = round_up(c, vec(dtype))
    t = torch.full((h, w, cs), fill, dtype=torch.float32 if dtype == 0 else torch.bfloat16, device="cuda")
    return t, cs


def dev_bytes(host_bytes: bytes):
    torch = torch_cuda()
    arr = np.frombuffer(host_bytes, dtype=np.uint8).copy()
    return torch.from_numpy(arr).cuda()


def pack_weights(kind, params, w_oihw):
    L = capi.load()
    w = np.ascontiguousarray(w_oihw, np.float32)
    n = L.pb_op_pack_weights(kind, C.byref(params), w.ctypes.data, None)
    assert n >= 0, L.pb_last_error()
    buf = (C.c_uint8 * n)()
    L.pb_op_pack_weights(kind, C.byref(params), w.ctypes.data, buf)
    return dev_bytes(bytes(buf))


def sync():
    torch_cuda().cuda.synchronize()


def error_flag(reset=True):
    L = capi.load()
    f = C.c_uint32(0)
    capi.check(L.pb_device_error_flag(0, C.byref(f), 1 if reset else 0), "pb_device_error_flag")
    return f.value

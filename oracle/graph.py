"""Oracle executor for model packs: runs a pack's operator table with the fp32 C
operators of ops.c (NCHW) and returns every tensor.

TEST INFRASTRUCTURE ONLY.  This parser reads the pack format independently of the
product's C++ loader, so a disagreement about the format shows up as a parity
failure.  The model semantics restated are those of the reference's served models
(jobs/tvm_<model>/tvm_<model>.cpp:24-47 run the compiled graph between an H2D and
a D2H copy); the reference holds no golden outputs for them (parity unpinned
upstream), so tests pin this executor against PyTorch/torchvision on CPU.
"""
from __future__ import annotations

import ctypes
import os
import struct
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

OP_CONV, OP_DENSE, OP_MAXPOOL, OP_AVGPOOL, OP_GAP, OP_ADD, OP_SOFTMAX, OP_AFFINE, OP_DETECT = 1, 2, 3, 4, 5, 6, 7, 8, 9
NONE = 0xFFFFFFFF
_f = ctypes.POINTER(ctypes.c_float)
_i = ctypes.c_int


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle_ops.so")
        if not os.path.exists(path):
            build()
        L = ctypes.CDLL(path)
        L.orc_conv2d.argtypes = [_f, _i, _i, _i, _f, _f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _i, _i]
        L.orc_conv2d_dil.argtypes = [_f, _i, _i, _i, _f, _f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _i, _i]
        L.orc_detect.argtypes = [_f, _i, _i, _i, _f, ctypes.c_float, ctypes.c_float, _i, _i, _f]
        L.orc_dense.argtypes = [_f, _i, _f, _f, _i, _i, _f]
        L.orc_maxpool.argtypes = [_f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i]
        L.orc_maxpool_pq.argtypes = [_f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i]
        L.orc_affine.argtypes = [_f, _i, ctypes.c_long, _f, _f, _i, _f]
        L.orc_avgpool.argtypes = [_f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i]
        L.orc_gap.argtypes = [_f, _i, _i, _i, _f]
        L.orc_add.argtypes = [_f, _f, ctypes.c_long, _i, _f]
        L.orc_softmax.argtypes = [_f, _i, _f]
        L.orc_round_bf16.argtypes = [_f, ctypes.c_long]
        L.orc_vec_add.argtypes = [_f, _f, ctypes.c_long]
        L.orc_quotient3.argtypes = [_f, ctypes.c_long, ctypes.c_float, _f]
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(_f)


def round_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32).copy()
    lib().orc_round_bf16(_p(a), a.size)
    return a


def conv2d(x, w, b=None, stride=(1, 1), pad=(0, 0), groups=1, act=0, residual=None, out=None, out_c_off=0, dilation=(1, 1)):
    c, h, wd = x.shape
    k, _, r, s = w.shape
    p = (h + 2 * pad[0] - dilation[0] * (r - 1) - 1) // stride[0] + 1
    q = (wd + 2 * pad[1] - dilation[1] * (s - 1) - 1) // stride[1] + 1
    if out is None:
        out = np.zeros((k, p, q), np.float32)
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    lib().orc_conv2d_dil(_p(x), c, h, wd, _p(w), _p(b), k, r, s, stride[0], stride[1], pad[0], pad[1], dilation[0], dilation[1],
                         groups, act, _p(residual), _p(out), out.shape[0], out_c_off)
    return out


def detect(head, anchors, priors, center_var, size_var, first, n_total, out):
    """Detection head over one feature map (orc_detect): writes this map's scores and boxes into `out`
    ([n_total*2 scores | n_total*4 boxes])."""
    head = np.ascontiguousarray(head, np.float32)
    priors = np.ascontiguousarray(priors, np.float32)
    assert head.shape[0] == 6 * anchors and priors.size == head.shape[1] * head.shape[2] * anchors * 4 and out.size == n_total * 6
    lib().orc_detect(_p(head), anchors, head.shape[1], head.shape[2], _p(priors), float(center_var), float(size_var), first, n_total, _p(out))
    return out


def dense(x, w, b=None, act=0):
    y = np.zeros(w.shape[0], np.float32)
    x = np.ascontiguousarray(x, np.float32).ravel()
    lib().orc_dense(_p(x), x.size, _p(np.ascontiguousarray(w, np.float32)), _p(b), w.shape[0], act, _p(y))
    return y


def pool_extent(n, k, stride, pad, ceil_mode):
    """Output extent of a pooling window sweep; ceil mode drops a last window that would start in
    the padding (torch.nn.MaxPool2d / ONNX MaxPool rule)."""
    if not ceil_mode:
        return (n + 2 * pad - k) // stride + 1
    o = -((n + 2 * pad - k) // -stride) + 1
    if (o - 1) * stride >= n + pad:
        o -= 1
    return o


def maxpool(x, k, stride, pad=(0, 0), out=None, out_c_off=0, ceil_mode=False):
    c, h, w = x.shape
    p = pool_extent(h, k[0], stride[0], pad[0], ceil_mode)
    q = pool_extent(w, k[1], stride[1], pad[1], ceil_mode)
    if out is None:
        out = np.zeros((c, p, q), np.float32)
    assert out.shape[1:] == (p, q)
    x = np.ascontiguousarray(x, np.float32)
    lib().orc_maxpool_pq(_p(x), c, h, w, k[0], k[1], stride[0], stride[1], pad[0], pad[1], p, q, _p(out), out.shape[0], out_c_off)
    return out


def avgpool(x, k, stride, pad=(0, 0), count_include_pad=True, out=None, out_c_off=0):
    c, h, w = x.shape
    p = (h + 2 * pad[0] - k[0]) // stride[0] + 1
    q = (w + 2 * pad[1] - k[1]) // stride[1] + 1
    if out is None:
        out = np.zeros((c, p, q), np.float32)
    x = np.ascontiguousarray(x, np.float32)
    lib().orc_avgpool(_p(x), c, h, w, k[0], k[1], stride[0], stride[1], pad[0], pad[1],
                      1 if count_include_pad else 0, _p(out), out.shape[0], out_c_off)
    return out


def affine(x, scale, bias, act=1):
    x = np.ascontiguousarray(x, np.float32)
    y = np.zeros_like(x)
    lib().orc_affine(_p(x), x.shape[0], x.shape[1] * x.shape[2], _p(np.ascontiguousarray(scale, np.float32)),
                     _p(np.ascontiguousarray(bias, np.float32)), act, _p(y))
    return y


def gap(x):
    x = np.ascontiguousarray(x, np.float32)
    y = np.zeros(x.shape[0], np.float32)
    lib().orc_gap(_p(x), x.shape[0], x.shape[1], x.shape[2], _p(y))
    return y


def add(a, b, act=0):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    y = np.zeros_like(a)
    lib().orc_add(_p(a), _p(b), a.size, act, _p(y))
    return y


def quotient3(v, div):
    """v / div by the reciprocal + fused-residual sequence of the average-pooling kernel (orc_quotient3)."""
    v = np.ascontiguousarray(v, np.float32)
    out = np.empty_like(v)
    lib().orc_quotient3(_p(v), v.size, float(div), _p(out))
    return out


def softmax(x):
    x = np.ascontiguousarray(x, np.float32).ravel()
    y = np.zeros_like(x)
    lib().orc_softmax(_p(x), x.size, _p(y))
    return y


class Pack:
    """Independent reader of the pack format (header 64 B, tensors 16 B, ops 96 B, names 64 B, f32 blob)."""

    def __init__(self, data: bytes):
        magic, ver, nt, no, tin, tout, prec, nfl, name = struct.unpack_from("<8s6IQ24s", data, 0)
        if magic != b"PB2PACK\0" or ver != 1:
            raise ValueError("not a model pack")
        self.name = name.split(b"\0")[0].decode()
        self.input, self.output, self.precision = tin, tout, prec
        off = 64
        self.tensors = [struct.unpack_from("<3I", data, off + 16 * i) for i in range(nt)]
        off += 16 * nt
        self.ops = [struct.unpack_from("<24I", data, off + 96 * i) for i in range(no)]
        off += 96 * no
        self.names = [data[off + 64 * i: off + 64 * i + 64].split(b"\0")[0].decode() for i in range(no)]
        off += 64 * no
        self.weights = np.frombuffer(data, dtype="<f4", count=nfl, offset=off).astype(np.float32)

    @classmethod
    def load(cls, path):
        with open(path, "rb") as f:
            return cls(f.read())


def run(pack: Pack, x: np.ndarray, emulate_bf16: bool = False, keep_all: bool = False):
    """Run the pack on input x (C,H,W fp32).  With emulate_bf16, weights and every
    activation tensor are rounded to bf16 (accumulation stays fp32), which models a
    bf16-storage / fp32-accumulate device path.  Returns the output vector (and all
    tensors when keep_all)."""
    W = pack.weights
    rb = round_bf16 if emulate_bf16 else (lambda a: a)
    bufs = [None] * len(pack.tensors)
    bufs[pack.input] = rb(np.ascontiguousarray(x, np.float32).reshape(pack.tensors[pack.input]))
    for rec in pack.ops:
        (typ, in0, in1, out, _, ooff, cin, cout, r, s, sh, sw, ph, pw, groups, act, flags, _,
         wlo, whi, blo, bhi, dh, dw) = rec
        dil = (max(dh, 1), max(dw, 1))        # 0 in packs written before dilation existed
        woff, boff = wlo | (whi << 32), blo | (bhi << 32)
        oc, oh, ow = pack.tensors[out]
        if bufs[out] is None:
            bufs[out] = np.zeros((oc, oh, ow), np.float32)
        xin = bufs[in0]
        if typ == OP_CONV:
            w = rb(W[woff: woff + cout * (cin // groups) * r * s].reshape(cout, cin // groups, r, s))
            b = np.ascontiguousarray(W[boff: boff + cout])
            res = None if in1 == NONE else np.ascontiguousarray(bufs[in1])
            if act == 3:     # PReLU: slopes follow the biases; y = v if v > 0 else slope[c] * v
                conv2d(xin, w, b, (sh, sw), (ph, pw), groups, 0, res, bufs[out], ooff, dil)
                v = bufs[out][ooff: ooff + cout]
                slope = W[boff + cout: boff + 2 * cout].reshape(-1, 1, 1)
                bufs[out][ooff: ooff + cout] = np.where(v > 0, v, v * slope).astype(np.float32)
            else:
                conv2d(xin, w, b, (sh, sw), (ph, pw), groups, act, res, bufs[out], ooff, dil)
        elif typ == OP_DENSE:
            w = rb(W[woff: woff + cout * cin].reshape(cout, cin))
            b = np.ascontiguousarray(W[boff: boff + cout])
            bufs[out][:] = dense(xin, w, b, act).reshape(oc, oh, ow)
        elif typ in (OP_MAXPOOL, OP_AVGPOOL):
            if typ == OP_MAXPOOL:
                maxpool(xin, (r, s), (sh, sw), (ph, pw), bufs[out], ooff, ceil_mode=bool(flags & 4))
            else:
                avgpool(xin, (r, s), (sh, sw), (ph, pw), bool(flags & 1), bufs[out], ooff)
            if flags & 8 or act:     # pooled value + per-channel bias, then the activation (fp32, in that order)
                sl = bufs[out][ooff: ooff + cin]
                if flags & 8:
                    sl += W[boff: boff + cin].reshape(-1, 1, 1)
                if act == 1:
                    np.maximum(sl, np.float32(0), out=sl)
                elif act == 2:
                    np.clip(sl, np.float32(0), np.float32(6), out=sl)
        elif typ == OP_GAP:
            bufs[out][:] = gap(xin).reshape(oc, 1, 1)
        elif typ == OP_ADD:
            bufs[out][:] = add(xin, bufs[in1], act)
        elif typ == OP_AFFINE:
            bufs[out][ooff: ooff + cin] = affine(xin[:cin], W[woff: woff + cin], W[boff: boff + cin], act)
        elif typ == OP_SOFTMAX:
            bufs[out][:] = softmax(xin).reshape(oc, oh, ow)
        elif typ == OP_DETECT:   # cin = anchors per position, cout = priors of the whole model, out_c_off = this map's first prior
            n_here = xin.shape[1] * xin.shape[2] * cin
            detect(xin, cin, W[woff: woff + 4 * n_here], W[boff], W[boff + 1], ooff, cout, bufs[out].reshape(-1))
        else:
            raise ValueError(f"unknown op type {typ}")
        if typ == OP_DETECT:
            continue
        if emulate_bf16 and out != pack.output:
            sl = bufs[out][ooff: ooff + cout] if typ in (OP_CONV, OP_MAXPOOL, OP_AVGPOOL, OP_AFFINE) else bufs[out]
            sl[...] = round_bf16(sl)
    y = bufs[pack.output].ravel().copy()
    return (y, bufs) if keep_all else y

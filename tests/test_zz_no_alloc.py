"""pb_conv2d_umma_noalloc: the tensor-core convolution for callers that cannot allocate (code inside an
allocator or memory-pool callback, threads that may not take the allocator's locks, hosts that have
handed out all device memory up front).  Its split-K scratch is a 4 MiB buffer built into the library.

Checked here, through the C ABI: its output equals that of the ordinary entry point
(pb_op_launch(PB_STAGE_CONV_UMMA) with caller-provided scratch) within the tolerance the other
tensor-core tests use (2^-7 relative + 2e-3 of the largest output), on two calls in a row that reuse
the built-in buffer; and a convolution whose split needs more than the buffer holds is refused with a
clear error instead of being launched.  This file sorts last so that a run stopping at the first
failure has already run everything else; it also passes when run alone in a fresh process."""
import ctypes as C

import numpy as np
import pytest

from oracle import graph as og
from paella_b200 import capi
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu


def _problem(C_, H, W, K, R, S, pad, seed):
    import torch
    rng = np.random.default_rng(seed)
    x = og.round_bf16(rng.standard_normal((C_, H, W), dtype=np.float32))
    w = og.round_bf16(rng.standard_normal((K, C_, R, S), dtype=np.float32) * np.float32(np.sqrt(2.0 / (C_ * R * S))))
    b = (rng.standard_normal(K, dtype=np.float32) * np.float32(0.1))
    P, Q = H + 2 * pad - R + 1, W + 2 * pad - S + 1
    xd, cs = gu.to_device_cl(x, 1)
    p = capi.OpParams()
    p.dtype = 1
    p.C, p.H, p.W, p.Cs = C_, H, W, cs
    p.K, p.P, p.Q = K, P, Q
    p.R, p.S, p.stride_h, p.stride_w, p.pad_h, p.pad_w, p.groups, p.act = R, S, 1, 1, pad, pad, 1, 1
    yd, ks = gu.empty_cl(P, Q, K, 1, fill=5.0)
    p.Ks = ks
    wd = gu.pack_weights(capi.STAGE_CONV_UMMA, p, w)
    bd = torch.from_numpy(b).cuda()
    p.x, p.w, p.bias, p.y = xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), yd.data_ptr()
    keep = (xd, wd, bd, yd)
    return p, yd, keep, (x, w, b, pad)


def _close(got, ref):
    scale = max(float(np.abs(ref).max()), 1e-6)
    return bool((np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 2e-3 * scale).all())


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row():
    import torch
    L = capi.load()
    # 8x8 map, 448 -> 384 channels, 3x3: 63 k-blocks, the split-K case of Inception-v3's last blocks
    p, yd, keep, (x, w, b, pad) = _problem(448, 8, 8, 384, 3, 3, 1, seed=41)
    li = capi.LaunchInfo()
    capi.check(L.pb_op_info(capi.STAGE_CONV_UMMA, C.byref(p), C.byref(li)), "pb_op_info")
    assert 0 < li.scratch_bytes <= (4 << 20), "case must split and fit the built-in buffer"

    # ordinary entry point, scratch provided by the caller
    sd = torch.zeros(li.scratch_bytes, dtype=torch.uint8, device="cuda")
    p.scratch, p.scratch_bytes = sd.data_ptr(), li.scratch_bytes
    capi.check(L.pb_op_launch(capi.STAGE_CONV_UMMA, C.byref(p), None, 0, None), "pb_op_launch")
    gu.sync()
    want = gu.from_device_cl(yd, 384)
    ref = og.conv2d(x, w, b, (1, 1), (pad, pad), 1, 1, None)
    assert _close(want, ref), "the ordinary entry point itself is off"

    # the no-allocation entry point: caller's scratch fields are ignored
    p.scratch, p.scratch_bytes = None, 0
    for call in range(2):
        yd.fill_(5.0)
        capi.check(L.pb_conv2d_umma_noalloc(C.byref(p), None, 0, None), f"pb_conv2d_umma_noalloc call {call}")
        gu.sync()
        assert gu.error_flag() == 0
        got = gu.from_device_cl(yd, 384)
        assert _close(got, want), f"call {call}: differs from the ordinary entry point by {float(np.abs(got - want).max())}"
        assert _close(got, ref)

    # a different shape that splits too, right after, through the same built-in buffer: the partial tiles the
    # first shape left behind must not leak into it
    p2, yd2, keep2, (x2, w2, b2, pad2) = _problem(512, 7, 7, 512, 3, 3, 1, seed=42)
    capi.check(L.pb_op_info(capi.STAGE_CONV_UMMA, C.byref(p2), C.byref(li)), "pb_op_info")
    assert 0 < li.scratch_bytes <= (4 << 20), "the second shape must split as well"
    capi.check(L.pb_conv2d_umma_noalloc(C.byref(p2), None, 0, None), "second shape")
    gu.sync()
    assert gu.error_flag() == 0
    assert _close(gu.from_device_cl(yd2, 512), og.conv2d(x2, w2, b2, (1, 1), (1, 1), 1, 1, None))


def test_noalloc_refuses_what_does_not_fit():
    L = capi.load()
    # 17x17 map, 3 row tiles x 8 column tiles = 24 tiles of 64 KiB partials: beyond 4 MiB once split
    p, yd, keep, _ = _problem(2048, 17, 17, 1024, 3, 3, 1, seed=43)
    li = capi.LaunchInfo()
    capi.check(L.pb_op_info(capi.STAGE_CONV_UMMA, C.byref(p), C.byref(li)), "pb_op_info")
    if li.scratch_bytes <= (4 << 20):
        pytest.skip("this build splits the shape into a buffer that fits")
    yd.fill_(5.0)
    rc = L.pb_conv2d_umma_noalloc(C.byref(p), None, 0, None)
    assert rc == -2
    assert b"built-in buffer" in L.pb_last_error()
    gu.sync()
    assert float(yd.float().min()) == 5.0 and float(yd.float().max()) == 5.0     # nothing ran

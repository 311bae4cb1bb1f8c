"""Operator kernels vs the CPU oracle, through pb_op_launch.  fp32 kernels: 1e-5 relative to the
largest output; bf16 kernels are compared with the oracle run on bf16-rounded inputs and weights
(fp32 accumulation on both sides), so the only differences are summation order and the final
bf16 rounding of the output: 2^-7 relative per element plus a small absolute term."""
import ctypes as C

import numpy as np
import pytest

from oracle import graph as og
from paella_b200 import capi
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(11)


def _params(dtype, x_shape, K, P, Q, Ks, R=1, S=1, sh=1, sw=1, ph=0, pw=0, groups=1, act=0, flags=0, out_c_off=0, Cs=None):
    p = capi.OpParams()
    p.dtype = dtype
    p.C, p.H, p.W = x_shape
    p.Cs = Cs if Cs is not None else gu.round_up(p.C, gu.vec(dtype))
    p.K, p.P, p.Q, p.Ks = K, P, Q, Ks
    p.out_c_off = out_c_off
    p.R, p.S, p.stride_h, p.stride_w, p.pad_h, p.pad_w, p.groups = R, S, sh, sw, ph, pw, groups
    p.act, p.flags = act, flags
    return p


def _assert_close(got, ref, dtype):
    scale = max(float(np.abs(ref).max()), 1e-6)
    if dtype == 0:
        assert float(np.abs(got - ref).max()) <= 1e-5 * scale
    else:
        tol = np.abs(ref) * 2.0 ** -7 + 2e-3 * scale
        bad = np.abs(got - ref) > tol
        assert not bad.any(), f"{int(bad.sum())} of {bad.size} elements off; worst {float(np.abs(got - ref).max())} (scale {scale})"


def _run_conv(kind, dtype, C_, H, W, K, R, S, sh, sw, ph, pw, groups=1, act=1, residual=False, out_total=None, off=0, bias=True,
              scratch=False, dilation=(1, 1)):
    import torch
    L = capi.load()
    x = RNG.standard_normal((C_, H, W), dtype=np.float32)
    w = (RNG.standard_normal((K, C_ // groups, R, S), dtype=np.float32) * np.float32(np.sqrt(2.0 / (C_ // groups * R * S))))
    b = RNG.standard_normal(K, dtype=np.float32) * np.float32(0.1) if bias else np.zeros(K, np.float32)
    P = (H + 2 * ph - dilation[0] * (R - 1) - 1) // sh + 1
    Q = (W + 2 * pw - dilation[1] * (S - 1) - 1) // sw + 1
    res = RNG.standard_normal((K, P, Q), dtype=np.float32) if residual else None
    if dtype == 1:
        x, w = og.round_bf16(x), og.round_bf16(w)
        res = og.round_bf16(res) if residual else None
    out_total = out_total or K
    xd, cs = gu.to_device_cl(x, dtype)
    yd, ks = gu.empty_cl(P, Q, out_total, dtype, fill=7.0)
    p = _params(dtype, (C_, H, W), K, P, Q, ks, R, S, sh, sw, ph, pw, groups, act, 0, off, cs)
    p.dil_h, p.dil_w = dilation
    if residual:
        rd, rcs = gu.to_device_cl(res, dtype)
        p.residual, p.res_Cs = rd.data_ptr(), rcs
    wd = gu.pack_weights(kind, p, w)
    bd = torch.from_numpy(b).cuda()
    p.x, p.w, p.bias, p.y = xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), yd.data_ptr()
    li = capi.LaunchInfo()
    capi.check(L.pb_op_info(kind, C.byref(p), C.byref(li)), "pb_op_info")
    assert li.flops == 2 * K * P * Q * (C_ // groups) * R * S
    unsplit_blocks = li.num_blocks
    launches = 1
    if scratch:
        if li.scratch_bytes == 0:
            pytest.skip("this shape is not split")
        sd = torch.zeros(li.scratch_bytes, dtype=torch.uint8, device="cuda")
        p.scratch, p.scratch_bytes = sd.data_ptr(), li.scratch_bytes
        capi.check(L.pb_op_info(kind, C.byref(p), C.byref(li)), "pb_op_info")
        assert li.num_blocks > unsplit_blocks
        launches = 3          # the tile counters must be back at zero after every launch
    ref = og.conv2d(x, w, b, (sh, sw), (ph, pw), groups, act, res, dilation=dilation)
    for _ in range(launches):
        yd.fill_(7.0)
        capi.check(L.pb_op_launch(kind, C.byref(p), None, 0, None), "pb_op_launch")
        gu.sync()
        assert gu.error_flag() == 0
        got_all = gu.from_device_cl(yd, out_total)
        _assert_close(got_all[off:off + K], ref, dtype)
    if scratch:
        assert int(sd[:4096].to(torch.int32).sum()) == 0
    if out_total > K:   # channels outside the slice are untouched
        mask = np.ones(out_total, bool)
        mask[off:off + K] = False
        assert (got_all[mask] == 7.0).all()


SIMT_CASES = [
    (1, 28, 28, 8, 5, 5, 1, 1, 2, 2), (8, 14, 14, 16, 5, 5, 1, 1, 2, 2), (3, 33, 31, 16, 7, 7, 2, 2, 3, 3),
    (16, 17, 17, 24, 1, 7, 1, 1, 0, 3), (12, 9, 9, 20, 3, 3, 2, 2, 0, 0), (5, 1, 1, 3, 1, 1, 1, 1, 0, 0),
]


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("case", SIMT_CASES)
def test_conv_simt(case, dtype):
    _run_conv(capi.STAGE_CONV_SIMT, dtype, *case, act=1, residual=(case[3] % 8 == 0))


# dilated filters (the receptive-field block of the face detector: 3x3 dilated by 2, 3 and 5 with equal padding)
DILATED_CASES = [
    # C, H, W, K, R, S, sh, sw, ph, pw, (dil_h, dil_w)
    (16, 30, 40, 16, 3, 3, 1, 1, 2, 2, (2, 2)), (16, 30, 40, 16, 3, 3, 1, 1, 3, 3, (3, 3)), (16, 30, 40, 16, 3, 3, 1, 1, 5, 5, (5, 5)),
    (24, 19, 23, 32, 3, 3, 2, 2, 2, 1, (2, 1)), (64, 14, 14, 64, 3, 3, 1, 1, 0, 0, (2, 3)), (8, 9, 9, 8, 2, 2, 1, 1, 0, 0, (4, 4)),
]


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("case", DILATED_CASES)
def test_conv_simt_dilated(case, dtype):
    _run_conv(capi.STAGE_CONV_SIMT, dtype, *case[:10], act=1, dilation=case[10])


@pytest.mark.parametrize("case", DILATED_CASES)
def test_conv_umma_dilated(case):
    _run_conv(capi.STAGE_CONV_UMMA, 1, *case[:10], act=0, residual=True, dilation=case[10])


def test_conv_simt_grouped_and_slice():
    _run_conv(capi.STAGE_CONV_SIMT, 0, 8, 6, 6, 8, 3, 3, 1, 1, 1, 1, groups=2, act=2)
    _run_conv(capi.STAGE_CONV_SIMT, 0, 4, 9, 9, 8, 3, 3, 1, 1, 1, 1, out_total=24, off=8)


UMMA_CASES = [
    # C, H, W, K, R, S, sh, sw, ph, pw        what it exercises
    (64, 16, 16, 64, 1, 1, 1, 1, 0, 0),       # one k-block, two row tiles
    (64, 8, 8, 32, 1, 1, 1, 1, 0, 0),         # half-empty row tile (64 of 128 rows)
    (128, 12, 12, 128, 3, 3, 1, 1, 1, 1),     # 18 k-blocks: pipeline wraps 4 stages several times
    (8, 37, 37, 32, 3, 3, 2, 2, 0, 0),        # 3 real channels padded to 8 happen here as C=8: taps share a k-block
    (16, 21, 21, 48, 5, 5, 1, 1, 2, 2),       # C < 64, 25 taps, k tail zero-filled
    (128, 17, 17, 192, 1, 7, 1, 1, 0, 3),     # asymmetric filter; two column tiles of 96
    (128, 17, 17, 160, 7, 1, 1, 1, 3, 0),     # 160 -> two tiles of 80
    (192, 9, 9, 320, 3, 3, 2, 2, 0, 0),       # 320 -> three tiles of 112 (336 padded), stride 2, single row tile of 16 rows
    (256, 14, 14, 512, 1, 1, 2, 2, 0, 0),     # strided 1x1 (down-sampling shortcut)
    (96, 7, 7, 24, 1, 1, 1, 1, 0, 0),         # K = 24: half of the second 16-column chunk is masked
    (32, 56, 56, 64, 3, 3, 1, 1, 1, 1),       # 25 row tiles
    (2048, 4, 4, 1008, 1, 1, 1, 1, 0, 0),     # long reduction (32 k-blocks), 8 column tiles
]


@pytest.mark.parametrize("case", UMMA_CASES)
def test_conv_umma(case):
    _run_conv(capi.STAGE_CONV_UMMA, 1, *case, act=1, residual=False)


@pytest.mark.parametrize("tiles_per_cta", ["1", "3"])
@pytest.mark.parametrize("case", UMMA_CASES)
def test_conv_umma_persistent_kernel(case, monkeypatch, tiles_per_cta):
    """The kernel the model launches use (a CTA walks several tiles, two accumulators in tensor memory, three
    producer threads), on the same shapes, alone and with the split reduction where the shape splits."""
    monkeypatch.setenv("PB_CONV_PERSIST", "1")
    monkeypatch.setenv("PB_CONV_PERSIST_OPS", "1")
    monkeypatch.setenv("PB_CONV_TILES_PER_CTA", tiles_per_cta)
    _run_conv(capi.STAGE_CONV_UMMA, 1, *case, act=1, residual=(case[3] % 64 == 0))
    L = capi.load()
    L.pb_set_conv_split_gain_us(0.0)
    try:
        C_, H, W, K, R, S, sh, sw, ph, pw = case
        p = _params(1, (C_, H, W), K, (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1, K, R, S, sh, sw, ph, pw)
        li = capi.LaunchInfo()
        capi.check(L.pb_op_info(capi.STAGE_CONV_UMMA, C.byref(p), C.byref(li)), "pb_op_info")
        if li.scratch_bytes:
            _run_conv(capi.STAGE_CONV_UMMA, 1, *case, act=2, residual=False, scratch=True)
    finally:
        L.pb_set_conv_split_gain_us(-1.0)


SPLIT_CASES = [c for c in UMMA_CASES if c[4] * c[5] * c[0] >= 256 and ((c[1] + 2 * c[8] - c[4]) // c[6] + 1) ** 2 <= 2048]


@pytest.mark.parametrize("case", SPLIT_CASES)
def test_conv_umma_split_reduction(case):
    """Same cases with scratch memory supplied: the reduction is split over blockIdx.z and the last
    block to arrive on a tile adds the partial tiles.  fp32 partial sums in a different order:
    same tolerance as the unsplit kernel."""
    L = capi.load()
    L.pb_set_conv_split_gain_us(0.0)        # split whenever the cost model sees any gain (the default asks for 6 us)
    try:
        _run_conv(capi.STAGE_CONV_UMMA, 1, *case, act=1, residual=(case[3] % 64 == 0), scratch=True)
    finally:
        L.pb_set_conv_split_gain_us(-1.0)


@pytest.mark.parametrize("case,residual", [((448, 8, 8, 384, 3, 3, 1, 1, 1, 1), False), ((512, 7, 7, 512, 3, 3, 1, 1, 1, 1), True),
                                           ((1024, 14, 14, 256, 3, 3, 1, 1, 1, 1), True)])
def test_conv_umma_long_reductions_do_split(case, residual):
    """Long reductions on small maps (the last blocks of Inception-v3 / ResNet): these must split at the
    library's default threshold, so the split path is exercised whatever the threshold is tuned to."""
    L = capi.load()
    p = _params(1, case[:3], case[3], case[1], case[2], case[3], case[4], case[5], 1, 1, 1, 1, 1, 1, 0, 0, case[0])
    li = capi.LaunchInfo()
    capi.check(L.pb_op_info(capi.STAGE_CONV_UMMA, C.byref(p), C.byref(li)), "pb_op_info")
    assert li.scratch_bytes > 0, "this shape should split"
    _run_conv(capi.STAGE_CONV_UMMA, 1, *case, act=1, residual=residual, scratch=True)


def test_conv_prelu_both_paths():
    """PReLU epilogue (per-channel slopes stored behind the biases): tensor-core path and direct path."""
    import torch
    L = capi.load()
    for kind, dtype in ((capi.STAGE_CONV_UMMA, 1), (capi.STAGE_CONV_SIMT, 0)):
        C_, H, W, K = 64, 14, 14, 96
        x = RNG.standard_normal((C_, H, W), dtype=np.float32)
        w = RNG.standard_normal((K, C_, 3, 3), dtype=np.float32) * np.float32(np.sqrt(2.0 / (C_ * 9)))
        b = (0.1 * RNG.standard_normal(K)).astype(np.float32)
        slope = (0.05 + 0.4 * RNG.random(K)).astype(np.float32)
        if dtype == 1:
            x, w = og.round_bf16(x), og.round_bf16(w)
        xd, cs = gu.to_device_cl(x, dtype)
        yd, ks = gu.empty_cl(H, W, K, dtype, fill=7.0)
        p = _params(dtype, (C_, H, W), K, H, W, ks, 3, 3, 1, 1, 1, 1, 1, 3, 0, 0, cs)
        wd = gu.pack_weights(kind, p, w)
        bd = torch.from_numpy(np.concatenate([b, slope])).cuda()
        p.x, p.w, p.bias, p.y = xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), yd.data_ptr()
        capi.check(L.pb_op_launch(kind, C.byref(p), None, 0, None), "prelu conv")
        gu.sync()
        v = og.conv2d(x, w, b, (1, 1), (1, 1), 1, 0, None)
        ref = np.where(v > 0, v, v * slope.reshape(-1, 1, 1)).astype(np.float32)
        assert (ref < 0).mean() > 0.2                      # the negative branch is exercised
        _assert_close(gu.from_device_cl(yd, K), ref, dtype)


def test_conv_umma_epilogue_variants():
    # residual add + relu, relu6, no activation, no bias, write into a channel slice of a wider tensor
    _run_conv(capi.STAGE_CONV_UMMA, 1, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1, act=1, residual=True)
    _run_conv(capi.STAGE_CONV_UMMA, 1, 64, 14, 14, 96, 1, 1, 1, 1, 0, 0, act=2)
    _run_conv(capi.STAGE_CONV_UMMA, 1, 64, 14, 14, 16, 1, 1, 1, 1, 0, 0, act=0, residual=True, bias=False)
    _run_conv(capi.STAGE_CONV_UMMA, 1, 64, 10, 10, 64, 3, 3, 1, 1, 1, 1, act=1, out_total=288, off=64)
    _run_conv(capi.STAGE_CONV_UMMA, 1, 48, 10, 10, 64, 5, 5, 1, 1, 2, 2, act=1, out_total=256, off=192)


def test_conv_umma_rejects_what_it_cannot_do():
    p = _params(1, (30, 8, 8), 30, 8, 8, 32, Cs=32)
    assert capi.load().pb_conv_umma_supported(C.byref(p)) == 0    # K not a multiple of 8
    p = _params(0, (64, 8, 8), 64, 8, 8, 64)
    assert capi.load().pb_conv_umma_supported(C.byref(p)) == 0    # fp32


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("case", [(32, 15, 15, 3, 3, 2, 2, 1, 1), (32, 9, 9, 3, 3, 1, 1, 1, 1), (144, 28, 28, 3, 3, 2, 2, 1, 1),
                                  (20, 7, 7, 3, 3, 1, 1, 1, 1)])
def test_dwconv(case, dtype):
    C_, H, W, R, S, sh, sw, ph, pw = case
    _run_conv(capi.STAGE_DWCONV, dtype, C_, H, W, C_, R, S, sh, sw, ph, pw, groups=C_, act=2)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("k,s,p,hw,c", [(2, 2, 0, 28, 8), (3, 3, 0, 14, 16), (3, 2, 1, 112, 64), (3, 2, 0, 35, 288), (3, 1, 1, 17, 768), (3, 2, 0, 9, 5)])
def test_pools(dtype, k, s, p, hw, c):
    L = capi.load()
    x = RNG.standard_normal((c, hw, hw), dtype=np.float32)
    if dtype == 1:
        x = og.round_bf16(x)
    P = (hw + 2 * p - k) // s + 1
    for kind, ref in ((capi.STAGE_MAXPOOL, og.maxpool(x, (k, k), (s, s), (p, p))),
                      (capi.STAGE_AVGPOOL, og.avgpool(x, (k, k), (s, s), (p, p), True))):
        xd, cs = gu.to_device_cl(x, dtype)
        yd, ks = gu.empty_cl(P, P, c + 16, dtype, fill=3.0)
        off = 8 if (c % 8 == 0) else 0
        prm = _params(dtype, (c, hw, hw), c, P, P, ks, k, k, s, s, p, p, flags=1, out_c_off=off, Cs=cs)
        prm.x, prm.y = xd.data_ptr(), yd.data_ptr()
        capi.check(L.pb_op_launch(kind, C.byref(prm), None, 0, None), "pool")
        gu.sync()
        got = gu.from_device_cl(yd, c + 16)[off:off + c]
        if kind == capi.STAGE_MAXPOOL:
            np.testing.assert_array_equal(got, ref)     # max of representable values: exact in both dtypes
        else:
            _assert_close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("k,s,p,hw,c,act", [(3, 1, 1, 17, 192, 1), (3, 1, 1, 35, 64, 1), (3, 2, 0, 9, 24, 2), (2, 2, 0, 12, 16, 0)])
def test_pools_with_a_bias_and_activation_tail(dtype, k, s, p, hw, c, act):
    """Pooling followed by a per-channel bias and an activation in the same kernel (the tail of a 1x1 convolution +
    batch-norm + ReLU that ran before an average pooling): act(pool(x) + bias), fp32, in that order."""
    import torch
    L = capi.load()
    x = RNG.standard_normal((c, hw, hw), dtype=np.float32)
    b = RNG.standard_normal(c, dtype=np.float32) * np.float32(0.3)
    if dtype == 1:
        x = og.round_bf16(x)
    P = (hw + 2 * p - k) // s + 1
    bd = torch.from_numpy(b).cuda()

    def tail(v):
        v = v + b.reshape(-1, 1, 1)
        return np.maximum(v, 0) if act == 1 else (np.clip(v, 0, 6) if act == 2 else v)

    for kind, ref in ((capi.STAGE_MAXPOOL, tail(og.maxpool(x, (k, k), (s, s), (p, p)))),
                      (capi.STAGE_AVGPOOL, tail(og.avgpool(x, (k, k), (s, s), (p, p), True)))):
        xd, cs = gu.to_device_cl(x, dtype)
        yd, ks = gu.empty_cl(P, P, c + 16, dtype, fill=3.0)
        prm = _params(dtype, (c, hw, hw), c, P, P, ks, k, k, s, s, p, p, act=act, flags=1, out_c_off=8, Cs=cs)
        prm.x, prm.y, prm.bias = xd.data_ptr(), yd.data_ptr(), bd.data_ptr()
        capi.check(L.pb_op_launch(kind, C.byref(prm), None, 0, None), "pool")
        gu.sync()
        got = gu.from_device_cl(yd, c + 16)
        _assert_close(got[8:8 + c], ref.astype(np.float32), dtype)
        assert (got[:8] == 3.0).all() and (got[8 + c:] == 3.0).all()


@pytest.mark.parametrize("dtype", [0, 1])
def test_gap_dense_add_softmax(dtype):
    import torch
    L = capi.load()
    rb = og.round_bf16 if dtype == 1 else (lambda a: a)
    # global average pool, written as the fp32 output
    x = rb(RNG.standard_normal((2048, 8, 8), dtype=np.float32))
    xd, cs = gu.to_device_cl(x, dtype)
    yd = torch.zeros(2048, dtype=torch.float32, device="cuda")
    p = _params(dtype, (2048, 8, 8), 2048, 1, 1, 2048, flags=2, Cs=cs)
    p.x, p.y = xd.data_ptr(), yd.data_ptr()
    capi.check(L.pb_op_launch(capi.STAGE_GAP, C.byref(p), None, 0, None), "gap")
    gu.sync()
    np.testing.assert_allclose(yd.cpu().numpy(), og.gap(x), rtol=1e-5, atol=1e-5)
    # dense on a flat vector
    n_in, n_out = 2048, 1000
    v = rb(RNG.standard_normal(n_in, dtype=np.float32))
    w = rb(RNG.standard_normal((n_out, n_in), dtype=np.float32) * np.float32(0.03))
    b = RNG.standard_normal(n_out, dtype=np.float32)
    vd = torch.from_numpy(v).cuda().to(torch.float32 if dtype == 0 else torch.bfloat16)
    wd = torch.from_numpy(w).cuda().to(torch.float32 if dtype == 0 else torch.bfloat16).contiguous()
    bd = torch.from_numpy(b).cuda()
    od = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    p = _params(dtype, (n_in, 1, 1), n_out, 1, 1, n_out, flags=2, Cs=n_in)
    p.x, p.w, p.bias, p.y = vd.data_ptr(), wd.data_ptr(), bd.data_ptr(), od.data_ptr()
    capi.check(L.pb_op_launch(capi.STAGE_DENSE, C.byref(p), None, 0, None), "dense")
    gu.sync()
    ref = og.dense(v, w, b)
    assert float(np.abs(od.cpu().numpy() - ref).max()) <= 2e-5 * float(np.abs(ref).max())
    # add + relu
    a1 = rb(RNG.standard_normal((64, 7, 7), dtype=np.float32))
    a2 = rb(RNG.standard_normal((64, 7, 7), dtype=np.float32))
    d1, cs = gu.to_device_cl(a1, dtype)
    d2, _ = gu.to_device_cl(a2, dtype)
    do, ks = gu.empty_cl(7, 7, 64, dtype)
    p = _params(dtype, (64, 7, 7), 64, 7, 7, ks, act=1, Cs=cs)
    p.x, p.residual, p.res_Cs, p.y = d1.data_ptr(), d2.data_ptr(), cs, do.data_ptr()
    capi.check(L.pb_op_launch(capi.STAGE_ADD, C.byref(p), None, 0, None), "add")
    gu.sync()
    _assert_close(gu.from_device_cl(do, 64), og.add(a1, a2, 1), dtype)
    # per-channel affine + relu on the first 40 of 64 channels, written at channel 8 of a 56-channel tensor
    sc = (1 + 0.1 * RNG.standard_normal(40)).astype(np.float32)
    bi = (0.1 * RNG.standard_normal(40)).astype(np.float32)
    do, ks = gu.empty_cl(7, 7, 56, dtype, fill=3.0)
    scd, bid = torch.from_numpy(sc).cuda(), torch.from_numpy(bi).cuda()
    p = _params(dtype, (40, 7, 7), 40, 7, 7, ks, act=1, out_c_off=8, Cs=cs)
    p.x, p.w, p.bias, p.y = d1.data_ptr(), scd.data_ptr(), bid.data_ptr(), do.data_ptr()
    capi.check(L.pb_op_launch(capi.STAGE_AFFINE, C.byref(p), None, 0, None), "affine")
    gu.sync()
    got = gu.from_device_cl(do, 56)
    _assert_close(got[8:48], og.affine(a1[:40], sc, bi, 1), dtype)
    assert (got[:8] == 3.0).all() and (got[48:] == 3.0).all()       # neighbours untouched
    # softmax over 1000 logits to the fp32 output
    lg = rb(RNG.standard_normal(1000, dtype=np.float32) * 3)
    ld = torch.from_numpy(lg).cuda().to(torch.float32 if dtype == 0 else torch.bfloat16)
    so = torch.zeros(1000, dtype=torch.float32, device="cuda")
    p = _params(dtype, (1000, 1, 1), 1000, 1, 1, 1000, flags=2, Cs=1000)
    p.x, p.y = ld.data_ptr(), so.data_ptr()
    capi.check(L.pb_op_launch(capi.STAGE_SOFTMAX, C.byref(p), None, 0, None), "softmax")
    gu.sync()
    np.testing.assert_allclose(so.cpu().numpy(), og.softmax(lg), rtol=2e-4, atol=1e-7)


@pytest.mark.parametrize("dtype", [0, 1])
def test_input_layout_conversion(dtype):
    import torch
    L = capi.load()
    x = RNG.standard_normal((3, 31, 29), dtype=np.float32)
    xd = torch.from_numpy(x).cuda()
    yd, ks = gu.empty_cl(31, 29, 3, dtype, fill=9.0)
    p = _params(dtype, (3, 31, 29), 3, 31, 29, ks, Cs=3)
    p.x, p.y = xd.data_ptr(), yd.data_ptr()
    capi.check(L.pb_op_launch(capi.STAGE_INPUT, C.byref(p), None, 0, None), "input")
    gu.sync()
    full = yd.float().cpu().numpy()
    ref = og.round_bf16(x) if dtype == 1 else x
    np.testing.assert_array_equal(np.transpose(full[:, :, :3], (2, 0, 1)), ref)
    assert (full[:, :, 3:] == 0).all()


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("geom", [(3, 31, 29, 3, 3, 2, 0), (3, 30, 30, 7, 7, 2, 3), (1, 12, 12, 5, 5, 1, 2), (3, 70, 75, 3, 3, 2, 0), (3, 64, 50, 7, 7, 2, 3),
                                  (4, 41, 67, 3, 3, 1, 1), (3, 33, 33, 9, 9, 1, 4)])
def test_input_patch_matrix(dtype, geom):
    """Stage 0 in its patch-matrix form: row (p, q) holds the stem convolution's receptive field,
    k = (r*S + s)*C + c, zeros outside the image and beyond R*S*C."""
    import torch
    L = capi.load()
    C_, H, W, R, S, st, pad = geom
    x = RNG.standard_normal((C_, H, W), dtype=np.float32)
    P, Q = (H + 2 * pad - R) // st + 1, (W + 2 * pad - S) // st + 1
    kp = R * S * C_
    xd = torch.from_numpy(x).cuda()
    yd, ks = gu.empty_cl(P, Q, kp, dtype, fill=9.0)
    p = _params(dtype, (C_, H, W), kp, P, Q, ks, R, S, st, st, pad, pad, Cs=C_)
    p.x, p.y = xd.data_ptr(), yd.data_ptr()
    capi.check(L.pb_op_launch(capi.STAGE_INPUT, C.byref(p), None, 0, None), "input patches")
    gu.sync()
    full = yd.float().cpu().numpy()                      # [P][Q][ks]
    xp = np.pad(x, ((0, 0), (pad, pad), (pad, pad)))
    ref = np.zeros((P, Q, kp), np.float32)
    for r in range(R):
        for s_ in range(S):
            ref[:, :, (r * S + s_) * C_:(r * S + s_ + 1) * C_] = np.transpose(xp[:, r:r + st * P:st, s_:s_ + st * Q:st], (1, 2, 0))
    np.testing.assert_array_equal(full[:, :, :kp], og.round_bf16(ref) if dtype == 1 else ref)
    assert (full[:, :, kp:] == 0).all()


# ---- tensors large enough for the strip / wide kernels (chosen by the library from the tensor's size) ----
def _strip_blocks(P, Q, cs, dtype, stride):
    strip = 4 if stride == 1 else 2          # output pixels per thread of the strip kernel
    if dtype == 1:
        # bf16: the shared-memory tile kernel takes over from 100 blocks on
        tiles = -(-cs // 64) * -(-Q // (8 * strip)) * -(-P // (13 if stride == 1 else 6))
        if tiles >= 100:
            return tiles
    return -(-(P * (-(-Q // strip)) * (cs // gu.vec(dtype))) // 256)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("case", [(64, 402, 398, 1), (64, 803, 797, 2)])
def test_dwconv_large_tensor_uses_strips(case, dtype):
    """Depthwise 3x3 on a tensor whose strips (4 pixels at stride 1, 2 at stride 2) fill the GPU: the strip kernel (or, in bf16
    on the larger case, the tile kernel) must run (block count) and agree with the oracle like the one-pixel kernel does,
    ragged last strip and borders included."""
    L = capi.load()
    C_, H, W, st = case
    P, Q = (H + 2 - 3) // st + 1, (W + 2 - 3) // st + 1
    p = _params(dtype, (C_, H, W), C_, P, Q, C_, 3, 3, st, st, 1, 1, groups=C_, act=2)
    li = capi.LaunchInfo()
    capi.check(L.pb_op_info(capi.STAGE_DWCONV, C.byref(p), C.byref(li)), "pb_op_info")
    assert li.num_blocks == _strip_blocks(P, Q, C_, dtype, st)
    _run_conv(capi.STAGE_DWCONV, dtype, C_, H, W, C_, 3, 3, st, st, 1, 1, groups=C_, act=2)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("s,pad,hw,include_pad", [(1, 1, 402, True), (1, 1, 402, False), (2, 0, 803, True), (2, 1, 805, False)])
def test_pools_large_tensor_use_strips(dtype, s, pad, hw, include_pad):
    L = capi.load()
    c = 64
    x = RNG.standard_normal((c, hw, hw), dtype=np.float32)
    if dtype == 1:
        x = og.round_bf16(x)
    P = (hw + 2 * pad - 3) // s + 1
    xd, cs = gu.to_device_cl(x, dtype)
    for kind, ref in ((capi.STAGE_MAXPOOL, og.maxpool(x, (3, 3), (s, s), (pad, pad))),
                      (capi.STAGE_AVGPOOL, og.avgpool(x, (3, 3), (s, s), (pad, pad), include_pad))):
        yd, ks = gu.empty_cl(P, P, c + 16, dtype, fill=3.0)
        prm = _params(dtype, (c, hw, hw), c, P, P, ks, 3, 3, s, s, pad, pad, flags=1 if include_pad else 0, out_c_off=8, Cs=cs)
        prm.x, prm.y = xd.data_ptr(), yd.data_ptr()
        li = capi.LaunchInfo()
        capi.check(L.pb_op_info(kind, C.byref(prm), C.byref(li)), "pb_op_info")
        assert li.num_blocks == _strip_blocks(P, P, cs, dtype, s)
        capi.check(L.pb_op_launch(kind, C.byref(prm), None, 0, None), "pool")
        gu.sync()
        full = gu.from_device_cl(yd, c + 16)
        got = full[8:8 + c]
        if kind == capi.STAGE_MAXPOOL:
            np.testing.assert_array_equal(got, ref)
        else:
            _assert_close(got, ref, dtype)
        assert (full[:8] == 3.0).all() and (full[8 + c:] == 3.0).all()     # channels outside the slice untouched


TILE_CASES = [
    # C, H, W, stride, pad: ragged strips and row chunks, fewer rows than one chunk, channel counts off the vector width
    (64, 70, 70, 1, 1), (20, 33, 41, 1, 1), (128, 15, 130, 1, 0), (64, 71, 69, 2, 1), (24, 37, 35, 2, 0), (8, 5, 300, 1, 1), (16, 100, 6, 2, 1),
]


@pytest.mark.parametrize("case", TILE_CASES)
def test_tiled_window_kernel_equals_the_strip_kernels_bit_for_bit(case, monkeypatch):
    """The 3x3 kernel for large tensors (window staged in shared memory, a thread walks down the output rows, each
    input row read and converted once) against the kernels it replaces, same launch with PB_WINDOW_TILE=0: depthwise convolution with bias and
    ReLU6, max pool, average pool with and without padding counted, into a channel slice.  Bit-identical, and within
    the usual tolerance of the oracle."""
    import torch
    L = capi.load()
    C_, H, W, st, pad = case
    P, Q = (H + 2 * pad - 3) // st + 1, (W + 2 * pad - 3) // st + 1
    x = og.round_bf16(RNG.standard_normal((C_, H, W), dtype=np.float32))
    w = og.round_bf16(RNG.standard_normal((C_, 1, 3, 3), dtype=np.float32) * np.float32(0.4))
    b = RNG.standard_normal(C_, dtype=np.float32) * np.float32(0.1)
    xd, cs = gu.to_device_cl(x, 1)
    bd = torch.from_numpy(b).cuda()
    runs = [("dw", capi.STAGE_DWCONV, 0, og.conv2d(x, w, b, (st, st), (pad, pad), C_, 2)),
            ("max", capi.STAGE_MAXPOOL, 0, og.maxpool(x, (3, 3), (st, st), (pad, pad))),
            ("avg", capi.STAGE_AVGPOOL, 1, og.avgpool(x, (3, 3), (st, st), (pad, pad), True)),
            ("avg_nopad", capi.STAGE_AVGPOOL, 0, og.avgpool(x, (3, 3), (st, st), (pad, pad), False))]
    for name, kind, flags, ref in runs:
        outs = {}
        for variant in ("tile", "0"):
            monkeypatch.setenv("PB_WINDOW_TILE", "1" if variant == "tile" else "0")
            monkeypatch.setenv("PB_WINDOW_TILE_MIN_BLOCKS", "1")
            yd, ks = gu.empty_cl(P, Q, C_ + 16, 1, fill=3.0)
            prm = _params(1, (C_, H, W), C_, P, Q, ks, 3, 3, st, st, pad, pad, groups=C_ if kind == capi.STAGE_DWCONV else 1,
                          act=2 if kind == capi.STAGE_DWCONV else 0, flags=flags, out_c_off=8, Cs=cs)
            prm.x, prm.y = xd.data_ptr(), yd.data_ptr()
            if kind == capi.STAGE_DWCONV:
                wd = gu.pack_weights(kind, prm, w)
                prm.w, prm.bias = wd.data_ptr(), bd.data_ptr()
            li = capi.LaunchInfo()
            capi.check(L.pb_op_info(kind, C.byref(prm), C.byref(li)), "pb_op_info")
            strip = 4 if st == 1 else 2
            if variant == "tile":
                assert li.num_blocks == -(-cs // 64) * -(-Q // (8 * strip)) * -(-P // (13 if st == 1 else 6)), name
            capi.check(L.pb_op_launch(kind, C.byref(prm), None, 0, None), name)
            gu.sync()
            assert gu.error_flag() == 0
            outs[variant] = gu.from_device_cl(yd, C_ + 16)
        outs["1"] = outs["tile"]
        np.testing.assert_array_equal(outs["1"], outs["0"], err_msg=name)
        got = outs["1"][8:8 + C_]
        if kind == capi.STAGE_MAXPOOL:
            np.testing.assert_array_equal(got, ref)
        else:
            _assert_close(got, ref, 1)
        # channels outside the slice are untouched (a channel count off the vector width zero-fills up to it, as the
        # kernels it replaces do)
        assert (outs["1"][:8] == 3.0).all() and (outs["1"][8 + -(-C_ // 8) * 8:] == 3.0).all()

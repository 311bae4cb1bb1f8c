"""Pins the CPU oracle's operators against PyTorch CPU fp32 (an independent
implementation of the same ONNX/Relay operator semantics)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import graph as og

RNG = np.random.default_rng(7)


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


CONV_CASES = [
    # C, H, W, K, R, S, sh, sw, ph, pw, groups
    (1, 28, 28, 8, 5, 5, 1, 1, 2, 2, 1),
    (8, 14, 14, 16, 5, 5, 1, 1, 2, 2, 1),
    (3, 33, 31, 16, 7, 7, 2, 2, 3, 3, 1),
    (16, 17, 17, 24, 1, 7, 1, 1, 0, 3, 1),
    (16, 17, 17, 24, 7, 1, 1, 1, 3, 0, 1),
    (12, 19, 19, 20, 3, 3, 2, 2, 0, 0, 1),
    (32, 15, 15, 32, 3, 3, 2, 2, 1, 1, 32),
    (32, 9, 9, 32, 3, 3, 1, 1, 1, 1, 32),
    (24, 7, 7, 40, 1, 1, 2, 2, 0, 0, 1),
    (5, 1, 1, 3, 1, 1, 1, 1, 0, 0, 1),
    (8, 6, 6, 8, 3, 3, 1, 1, 1, 1, 2),
]


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("act", [0, 1, 2])
def test_conv2d_matches_torch(oracle_lib, case, act):
    C, H, W, K, R, S, sh, sw, ph, pw, g = case
    x = RNG.standard_normal((C, H, W), dtype=np.float32)
    w = RNG.standard_normal((K, C // g, R, S), dtype=np.float32)
    b = RNG.standard_normal(K, dtype=np.float32)
    ref = F.conv2d(_t(x)[None], _t(w), _t(b), (sh, sw), (ph, pw), 1, g)[0]
    res = RNG.standard_normal(tuple(ref.shape), dtype=np.float32)
    ref = ref + _t(res)
    if act == 1:
        ref = F.relu(ref)
    elif act == 2:
        ref = F.relu6(ref)
    got = og.conv2d(x, w, b, (sh, sw), (ph, pw), g, act, res)
    np.testing.assert_allclose(got, ref.numpy(), rtol=1e-4, atol=1e-4)


DILATED_CASES = [
    # C, H, W, K, R, S, sh, sw, ph, pw, groups, (dil_h, dil_w): the receptive-field block of the face detector and odd ones
    (16, 30, 40, 16, 3, 3, 1, 1, 2, 2, 1, (2, 2)), (16, 30, 40, 16, 3, 3, 1, 1, 3, 3, 1, (3, 3)), (16, 30, 40, 16, 3, 3, 1, 1, 5, 5, 1, (5, 5)),
    (6, 19, 23, 8, 3, 3, 2, 2, 2, 1, 1, (2, 1)), (8, 14, 14, 8, 3, 3, 1, 1, 0, 0, 2, (2, 3)), (3, 9, 9, 4, 2, 2, 1, 1, 0, 0, 1, (4, 4)),
]


@pytest.mark.parametrize("case", DILATED_CASES)
def test_dilated_conv2d_matches_torch(oracle_lib, case):
    C, H, W, K, R, S, sh, sw, ph, pw, g, dil = case
    x = RNG.standard_normal((C, H, W), dtype=np.float32)
    w = RNG.standard_normal((K, C // g, R, S), dtype=np.float32)
    b = RNG.standard_normal(K, dtype=np.float32)
    ref = torch.relu(F.conv2d(_t(x)[None], _t(w), _t(b), (sh, sw), (ph, pw), dil, g)[0]).numpy()
    got = og.conv2d(x, w, b, (sh, sw), (ph, pw), g, 1, dilation=dil)
    assert got.shape == ref.shape
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)


def test_detection_head_matches_its_formula(oracle_lib):
    """orc_detect against the published post-processing written with torch tensors: softmax over the two class logits,
    centre = l[:2] * 0.1 * prior_wh + prior_centre, size = exp(l[2:] * 0.2) * prior_wh, corners = centre -+ size / 2;
    priors and head in (row, column, anchor) order, the head's channels (anchor, class) then (anchor, coordinate)."""
    A, H, W, first, n_total = 3, 5, 7, 11, 200
    head = RNG.standard_normal((6 * A, H, W), dtype=np.float32)
    priors = RNG.random((H * W * A, 4), dtype=np.float32)
    out = np.full(n_total * 6, -7.0, np.float32)
    og.detect(head, A, priors, 0.1, 0.2, first, n_total, out)
    t = _t(head)
    conf = t[:2 * A].permute(1, 2, 0).reshape(-1, 2)
    loc = t[2 * A:].permute(1, 2, 0).reshape(-1, 4)
    pr = _t(priors)
    scores = torch.softmax(conf, dim=1).numpy()
    centre = loc[:, :2] * 0.1 * pr[:, 2:] + pr[:, :2]
    size = torch.exp(loc[:, 2:] * 0.2) * pr[:, 2:]
    boxes = torch.cat([centre - size / 2, centre + size / 2], dim=1).numpy()
    n = H * W * A
    np.testing.assert_allclose(out[first * 2:(first + n) * 2].reshape(n, 2), scores, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(out[n_total * 2 + first * 4: n_total * 2 + (first + n) * 4].reshape(n, 4), boxes, rtol=1e-5, atol=1e-6)
    untouched = np.ones(n_total * 6, bool)
    untouched[first * 2:(first + n) * 2] = False
    untouched[n_total * 2 + first * 4: n_total * 2 + (first + n) * 4] = False
    assert (out[untouched] == -7.0).all()


def test_conv2d_writes_channel_slice(oracle_lib):
    x = RNG.standard_normal((4, 9, 9), dtype=np.float32)
    w = RNG.standard_normal((6, 4, 3, 3), dtype=np.float32)
    out = np.full((10, 9, 9), 7.0, np.float32)
    og.conv2d(x, w, None, (1, 1), (1, 1), 1, 0, None, out, 3)
    ref = F.conv2d(_t(x)[None], _t(w), None, 1, 1)[0].numpy()
    np.testing.assert_allclose(out[3:9], ref, rtol=1e-4, atol=1e-4)
    assert (out[:3] == 7.0).all() and (out[9:] == 7.0).all()


@pytest.mark.parametrize("k,s,p,hw", [(2, 2, 0, 28), (3, 3, 0, 14), (3, 2, 1, 112), (3, 2, 0, 35), (3, 1, 1, 17)])
def test_pools_match_torch(oracle_lib, k, s, p, hw):
    x = RNG.standard_normal((5, hw, hw), dtype=np.float32)
    got = og.maxpool(x, (k, k), (s, s), (p, p))
    ref = F.max_pool2d(_t(x)[None], k, s, p)[0].numpy()
    np.testing.assert_array_equal(got, ref)
    for cip in (True, False):
        got = og.avgpool(x, (k, k), (s, s), (p, p), cip)
        ref = F.avg_pool2d(_t(x)[None], k, s, p, count_include_pad=cip)[0].numpy()
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("k,s,p,hw", [(3, 2, 0, 111), (3, 2, 0, 112), (3, 2, 0, 13), (2, 2, 0, 14), (2, 2, 0, 7), (3, 1, 1, 14), (3, 2, 1, 8)])
def test_ceil_mode_maxpool_matches_torch(oracle_lib, k, s, p, hw):
    """SqueezeNet / GoogLeNet pooling: the last window may hang over the bottom/right edge."""
    x = RNG.standard_normal((4, hw, hw), dtype=np.float32)
    got = og.maxpool(x, (k, k), (s, s), (p, p), ceil_mode=True)
    ref = F.max_pool2d(_t(x)[None], k, s, p, ceil_mode=True)[0].numpy()
    assert got.shape == ref.shape
    np.testing.assert_array_equal(got, ref)
    from paella_b200 import packer
    assert packer._pool_extent(hw, k, s, p, True) == ref.shape[1]


def test_affine_matches_torch_batchnorm(oracle_lib):
    x = RNG.standard_normal((24, 9, 7), dtype=np.float32)
    gamma = (1 + 0.1 * RNG.standard_normal(24)).astype(np.float32)
    beta = (0.1 * RNG.standard_normal(24)).astype(np.float32)
    eps = 1e-5
    ref = F.relu(F.batch_norm(_t(x)[None], torch.zeros(24), torch.ones(24), _t(gamma), _t(beta), False, 0.0, eps))[0].numpy()
    got = og.affine(x, gamma / np.float32(np.sqrt(1 + eps)), beta, 1)
    np.testing.assert_allclose(got, ref, rtol=1e-6, atol=1e-6)


def test_dense_gap_add_softmax(oracle_lib):
    x = RNG.standard_normal(300, dtype=np.float32)
    w = RNG.standard_normal((17, 300), dtype=np.float32)
    b = RNG.standard_normal(17, dtype=np.float32)
    np.testing.assert_allclose(og.dense(x, w, b), F.linear(_t(x), _t(w), _t(b)).numpy(), rtol=1e-4, atol=1e-4)
    t = RNG.standard_normal((6, 7, 7), dtype=np.float32)
    np.testing.assert_allclose(og.gap(t), t.mean(axis=(1, 2)), rtol=1e-5, atol=1e-6)
    u = RNG.standard_normal((6, 7, 7), dtype=np.float32)
    np.testing.assert_array_equal(og.add(t, u, 1), np.maximum(t + u, 0))
    np.testing.assert_allclose(og.softmax(x), F.softmax(_t(x), 0).numpy(), rtol=1e-5, atol=1e-7)


def test_round_bf16_matches_torch(oracle_lib):
    x = RNG.standard_normal(10000, dtype=np.float32) * 100
    x[:4] = [0.0, -0.0, np.inf, 1.0000001]
    ref = _t(x).to(torch.bfloat16).to(torch.float32).numpy()
    np.testing.assert_array_equal(og.round_bf16(x), ref)


def test_average_pool_quotient_sequence_is_the_division():
    """The 3x3 average-pooling kernel replaces v / div by reciprocal, fused residual and correction
    (three instructions per element).  For every window size a 3x3 pool can have the sequence must
    return the correctly rounded quotient: compared bit for bit with numpy's fp32 division on random bit
    patterns (all normal magnitudes whose quotient is normal), zero and the largest finite values.  -0.0 is left
    out: the sequence returns +0.0 for it, and the kernel's sums start from +0.0, so they are never -0.0."""
    rng = np.random.default_rng(5)
    bits = rng.integers(0, 2 ** 32, size=4_000_000, dtype=np.uint64).astype(np.uint32)
    v = bits.view(np.float32)
    v = v[np.isfinite(v) & (np.abs(v) > 1e-30)]
    v = np.concatenate([v, np.array([0.0, 3.4028235e38, -3.4028235e38, 9.0, 1.0, 1e-30], np.float32)])
    for div in range(1, 10):
        got = og.quotient3(v, div)
        ref = v / np.float32(div)
        np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32))
    inf = np.array([np.inf, -np.inf], np.float32)
    np.testing.assert_array_equal(og.quotient3(inf, 9), inf)

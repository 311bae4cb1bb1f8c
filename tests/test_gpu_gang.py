"""Gangs: several requests of one model run as ONE set of launches (images back to back in every activation
tensor, pb_op_params.batch / pb_instance_*_batched / pb_server_config.max_gang).

Bar: a gang of n gives what n separate runs give.  Every kernel treats the images independently and the
tensor-core convolution accumulates each output row over k in the same order whatever the row's tile, so
results are BIT-IDENTICAL as long as the reduction is split the same way; with the split switched off on
both sides (pb_set_conv_split_gain_us) the tests ask for equal bits, with the default split for the usual
tolerance against the oracle."""
import ctypes as C
import os
import time

import numpy as np
import pytest

from oracle import graph as og
from paella_b200 import capi, packer
from tests import gpu_util as gu
from tests.golden.make_golden import make_input

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(23)
NEVER_SPLIT = 1e9


def _cl_batch(xs, dtype):
    """list of [C][H][W] -> device [n][H][W][Cs]"""
    import torch
    c, h, w = xs[0].shape
    cs = gu.round_up(c, gu.vec(dtype))
    buf = np.zeros((len(xs), h, w, cs), np.float32)
    for i, x in enumerate(xs):
        buf[i, :, :, :c] = np.transpose(x, (1, 2, 0))
    t = torch.from_numpy(buf).cuda()
    return (t if dtype == 0 else t.to(torch.bfloat16)).contiguous(), cs


def _op(kind, dtype, C_, H, W, K, R, S, st, pad, groups=1, act=0, flags=0, residual=False, out_total=None, off=0, nb=3):
    """Runs `kind` once with batch = nb and once per image; returns both outputs [nb][P][Q][Ks] as numpy."""
    import torch
    L = capi.load()
    xs = [RNG.standard_normal((C_, H, W), dtype=np.float32) for _ in range(nb)]
    P = (H + 2 * pad - R) // st + 1
    out_total = out_total or K
    xd, cs = _cl_batch(xs, dtype)
    tdt = torch.float32 if dtype == 0 else torch.bfloat16
    ks = gu.round_up(out_total, gu.vec(dtype))
    p = capi.OpParams()
    p.dtype = dtype
    p.C, p.H, p.W, p.Cs = C_, H, W, cs
    p.K, p.P, p.Q, p.Ks, p.out_c_off = K, P, P, ks, off
    p.R, p.S, p.stride_h, p.stride_w, p.pad_h, p.pad_w, p.groups = R, S, st, st, pad, pad, groups
    p.act, p.flags = act, flags
    keep = [xd]
    if kind in (capi.STAGE_CONV_UMMA, capi.STAGE_CONV_SIMT, capi.STAGE_DWCONV):
        w = RNG.standard_normal((K, C_ // groups, R, S), dtype=np.float32) * np.float32(0.2)
        wd = gu.pack_weights(kind, p, w)
        bd = torch.from_numpy(RNG.standard_normal(K, dtype=np.float32)).cuda()
        p.w, p.bias = wd.data_ptr(), bd.data_ptr()
        keep += [wd, bd]
    if kind == capi.STAGE_AFFINE:
        sc = torch.from_numpy(RNG.standard_normal(C_, dtype=np.float32)).cuda()
        bd = torch.from_numpy(RNG.standard_normal(C_, dtype=np.float32)).cuda()
        p.w, p.bias = sc.data_ptr(), bd.data_ptr()
        keep += [sc, bd]
    rd = None
    if residual or kind == capi.STAGE_ADD:
        rshape = (K, P, P) if kind != capi.STAGE_ADD else (C_, H, W)
        rd, rcs = _cl_batch([RNG.standard_normal(rshape, dtype=np.float32) for _ in range(nb)], dtype)
        p.res_Cs = rcs
    li = capi.LaunchInfo()

    def launch(batch, x_t, r_t, y_t):
        p.batch = batch
        p.x, p.y = x_t.data_ptr(), y_t.data_ptr()
        p.residual = r_t.data_ptr() if r_t is not None else None
        p.scratch, p.scratch_bytes = None, 0
        capi.check(L.pb_op_info(kind, C.byref(p), C.byref(li)), "pb_op_info")
        sd = None
        if li.scratch_bytes:
            sd = torch.zeros(li.scratch_bytes, dtype=torch.uint8, device="cuda")
            p.scratch, p.scratch_bytes = sd.data_ptr(), li.scratch_bytes
        capi.check(L.pb_op_launch(kind, C.byref(p), None, 0, None), "pb_op_launch")
        gu.sync()
        assert gu.error_flag() == 0
        return li.num_blocks

    y_gang = torch.full((nb, P, P, ks), 7.0, dtype=tdt, device="cuda")
    blocks_gang = launch(nb, xd, rd, y_gang)
    y_one = torch.full((nb, P, P, ks), 7.0, dtype=tdt, device="cuda")
    blocks_one = 0
    for i in range(nb):
        blocks_one = launch(1, xd[i], rd[i] if rd is not None else None, y_one[i])
    return y_gang.float().cpu().numpy(), y_one.float().cpu().numpy(), blocks_gang, blocks_one


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("kind,args", [
    (capi.STAGE_CONV_SIMT, dict(C_=8, H=9, W=9, K=16, R=3, S=3, st=1, pad=1, act=1, residual=True)),
    (capi.STAGE_DWCONV, dict(C_=32, H=11, W=11, K=32, R=3, S=3, st=2, pad=1, groups=32, act=2)),
    (capi.STAGE_DWCONV, dict(C_=16, H=9, W=9, K=16, R=5, S=5, st=1, pad=2, groups=16, act=1)),
    (capi.STAGE_MAXPOOL, dict(C_=24, H=13, W=13, K=24, R=3, S=3, st=2, pad=0, out_total=40, off=8)),
    (capi.STAGE_MAXPOOL, dict(C_=8, H=12, W=12, K=8, R=2, S=2, st=2, pad=0)),
    (capi.STAGE_AVGPOOL, dict(C_=24, H=9, W=9, K=24, R=3, S=3, st=1, pad=1, flags=1)),
    (capi.STAGE_ADD, dict(C_=24, H=7, W=7, K=24, R=1, S=1, st=1, pad=0, act=1)),
    (capi.STAGE_AFFINE, dict(C_=20, H=7, W=7, K=20, R=1, S=1, st=1, pad=0, act=1)),
])
def test_memory_bound_kernels_batch_equals_separate_launches(kind, args, dtype):
    g, o, bg, bo = _op(kind, dtype, **args)
    np.testing.assert_array_equal(g, o)
    assert bg >= bo            # one launch carries every image's blocks


@pytest.mark.parametrize("case", [
    dict(C_=64, H=8, W=8, K=32, R=1, S=1, st=1, pad=0, act=1),                       # 64 rows per image: two images share a tile
    dict(C_=128, H=17, W=17, K=192, R=3, S=3, st=1, pad=1, act=1, residual=True),    # 289 rows per image: tiles straddle images
    dict(C_=96, H=9, W=9, K=48, R=3, S=3, st=2, pad=0, act=2, out_total=80, off=16), # stride 2, channel slice
    dict(C_=16, H=21, W=21, K=48, R=5, S=5, st=1, pad=2, act=0),
])
@pytest.mark.parametrize("nb", [2, 5])
def test_tensor_core_convolution_batch_equals_separate_launches(case, nb):
    L = capi.load()
    L.pb_set_conv_split_gain_us(NEVER_SPLIT)
    try:
        g, o, bg, bo = _op(capi.STAGE_CONV_UMMA, 1, nb=nb, **case)
    finally:
        L.pb_set_conv_split_gain_us(-1.0)
    np.testing.assert_array_equal(g, o)
    P = g.shape[1]
    assert bg <= nb * bo and (nb * P * P > 128 or bg == bo)      # images share row tiles


class Batched:
    def __init__(self, path, precision, cap):
        self.L = capi.load()
        self.m, self.i = C.c_void_p(), C.c_void_p()
        capi.check(self.L.pb_model_load(path.encode(), 0, precision, C.byref(self.m)), "pb_model_load")
        capi.check(self.L.pb_instance_create_batched(self.m, cap, 0, C.byref(self.i)), "pb_instance_create_batched")
        self.n_out = self.L.pb_model_output_bytes(self.m) // 4

    def run(self, xs, by_groups):
        x = np.ascontiguousarray(np.stack(xs), np.float32)
        y = np.zeros((len(xs), self.n_out), np.float32)
        capi.check(self.L.pb_instance_run_batch_sync(self.i, len(xs), 1 if by_groups else 0, x.ctypes.data, y.ctypes.data), "run batch")
        assert gu.error_flag() == 0
        return y

    def close(self):
        self.L.pb_instance_destroy(self.i)
        self.L.pb_model_destroy(self.m)


@pytest.mark.parametrize("model,precision,shape", [("mnist", 0, (1, 28, 28)), ("resnet18", 1, (3, 224, 224)), ("inception_v3", 1, (3, 299, 299)),
                                                   ("mobilenet", 1, (3, 224, 224)), ("ultraface320", 1, (3, 240, 320))])
def test_gang_of_four_equals_four_single_runs_bit_for_bit(models_dir, model, precision, shape):
    """With the reduction split switched off on both sides, a gang's logits are the bits of the single runs,
    kernel by kernel and as stage-group graphs, for every gang size up to the capacity."""
    L = capi.load()
    L.pb_set_conv_split_gain_us(NEVER_SPLIT)
    try:
        b = Batched(os.path.join(models_dir, packer.pack_file_name(model)), precision, 4)
        rng = np.random.default_rng(31)
        xs = [(rng.random(shape, dtype=np.float32) if model == "mnist" else rng.standard_normal(shape, dtype=np.float32) * np.float32(0.6 + 0.3 * i))
              for i in range(4)]
        single = np.stack([b.run([x], False)[0] for x in xs])
        assert not np.array_equal(single[0], single[1])
        for n in (4, 3, 2):
            np.testing.assert_array_equal(b.run(xs[:n], False), single[:n])
            np.testing.assert_array_equal(b.run(xs[:n], True), single[:n])
        np.testing.assert_array_equal(b.run(xs[2:3], True)[0], single[2])       # and back to one image
        li1, li4 = capi.LaunchInfo(), capi.LaunchInfo()
        g_last = L.pb_model_num_groups(b.m) - 1
        capi.check(L.pb_model_group_info_batched(b.m, g_last, 1, C.byref(li1)), "group info")
        capi.check(L.pb_model_group_info_batched(b.m, g_last, 4, C.byref(li4)), "group info")
        assert li4.num_blocks > li1.num_blocks and li4.flops == 4 * li1.flops
        b.close()
    finally:
        L.pb_set_conv_split_gain_us(-1.0)


def test_gang_with_default_split_matches_the_oracle(models_dir):
    """Default split threshold: a gang of three Inception-v3 requests against the fp32 oracle
    (<= 1e-2 of the largest logit, same argmax)."""
    b = Batched(os.path.join(models_dir, packer.pack_file_name("inception_v3")), 1, 4)
    pack = og.Pack(packer.inception_v3(seed=1234).to_bytes())
    xs = [make_input("inception_v3", s) for s in (5, 6, 7)]
    y = b.run(xs, True)
    for i, x in enumerate(xs):
        ref = og.run(pack, x)
        assert float(np.abs(y[i] - ref).max()) <= 1e-2 * float(np.abs(ref).max())
        assert int(y[i].argmax()) == int(ref.argmax())
    b.close()


def _server(models_dir, monkeypatch, gang, streams=128):
    monkeypatch.setenv("LLIS_MODELS_DIR", models_dir)
    L = capi.load()
    cfg = capi.ServerConfig()
    L.pb_server_config_default(C.byref(cfg))
    cfg.num_streams = streams
    cfg.max_gang = gang
    s = C.c_void_p()
    capi.check(L.pb_server_create(C.byref(cfg), C.byref(s)), "pb_server_create")
    return L, s


def _pinned(nbytes):
    import torch
    return torch.zeros(nbytes, dtype=torch.uint8).pin_memory()


def _run_until(L, s, n, timeout=120.0):
    done = {}
    cookies, errs = (C.c_uint64 * 64)(), (C.c_int32 * 64)()
    t0 = time.time()
    while len(done) < n and time.time() - t0 < timeout:
        assert L.pb_server_step(s, 256) >= 0, L.pb_last_error()
        k = L.pb_server_poll_done(s, cookies, errs, 64)
        for i in range(k):
            done[cookies[i]] = errs[i]
    return done


@pytest.mark.parametrize("gang", [4, 8])
def test_server_forms_gangs_and_every_slot_gets_its_own_result(tmp_path, monkeypatch, gang):
    """The headline mix through a server that may gang requests: 12 Inception-v3 + 36 MNIST requests submitted
    at once (so the queue holds many fresh jobs of each type when the first is dispatched), host buffers, two
    rounds.  Every slot's output is checked against the oracle on that slot's own input, and the number of
    dispatches shows that gangs were formed."""
    d = tmp_path / f"models_gang{gang}"       # own directory: plugins cache loaded models by path
    d.mkdir()
    packer.write_all(str(d), ["mnist", "inception_v3"])
    monkeypatch.delenv("PB_PRECISION", raising=False)
    L, s = _server(str(d), monkeypatch, gang)
    ids, sizes = {}, {}
    for job in ["tvm_mnist", "tvm_inception_v3"]:
        j = C.c_uint32()
        capi.check(L.pb_server_register_job(s, capi.plugin_path(job).encode(), C.byref(j)), "register " + job)
        ids[job] = j.value
        ib, ob, sb = C.c_size_t(), C.c_size_t(), C.c_size_t()
        L.pb_server_job_io_bytes(s, j, C.byref(ib), C.byref(ob), C.byref(sb))
        sizes[job] = (ib.value, ob.value, sb.value)
    reqs = []
    for i in range(48):
        job = "tvm_inception_v3" if i % 4 == 0 else "tvm_mnist"
        rng = np.random.default_rng(7000 + i)
        x = (rng.standard_normal((3, 299, 299), dtype=np.float32) * np.float32(0.5 + 0.1 * (i // 4))
             if job == "tvm_inception_v3" else rng.random((1, 28, 28), dtype=np.float32))
        t = _pinned(sizes[job][2])
        t.numpy()[:x.nbytes] = np.frombuffer(x.tobytes(), np.uint8)
        reqs.append((job, x, t))
    inc = og.Pack(packer.inception_v3(seed=1234).to_bytes())
    mn = og.Pack(packer.mnist_cnn(seed=1234).to_bytes())
    refs = [og.run(inc if job == "tvm_inception_v3" else mn, x) for job, x, _ in reqs]
    for rnd in range(2):
        for job, x, t in reqs:
            ib, ob, sb = sizes[job]
            t.numpy()[(ib + 7) // 8 * 8:] = 0
        d0 = L.pb_server_num_decisions(s)
        for i, (job, x, t) in enumerate(reqs):
            capi.check(L.pb_server_launch(s, ids[job], t.data_ptr(), 1000 * rnd + i), "launch")
        done = _run_until(L, s, len(reqs))
        assert len(done) == len(reqs) and all(e == 0 for e in done.values()), done
        assert gu.error_flag() == 0
        for (job, x, t), ref in zip(reqs, refs):
            ib, ob, sb = sizes[job]
            off = (ib + 7) // 8 * 8
            y = np.frombuffer(t.numpy()[off: off + ob].tobytes(), np.float32)
            rel = float(np.abs(y - ref).max() / np.abs(ref).max())
            if job == "tvm_inception_v3":
                assert rel <= 1e-2, (rnd, rel)
                assert int(y.argmax()) == int(ref.argmax())
            else:
                assert rel <= 1e-5, (rnd, rel)
        if rnd == 1:
            # one request per launch would take 36 x 1 + 12 x 3 = 72 dispatches; with gangs allowed the scheduler
            # dispatches once per pb_server_step, when all 48 requests are queued
            assert L.pb_server_num_decisions(s) - d0 < 72 * 0.6
    assert L.pb_server_jobs_in_flight(s) == 0
    L.pb_server_destroy(s)

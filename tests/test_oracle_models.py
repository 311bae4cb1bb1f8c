"""Pins the model packs + oracle executor against torchvision's definitions of the
same topologies (CPU fp32), loading the pack's weights into the torch modules."""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torchvision

from oracle import graph as og
from paella_b200 import packer


def _load_into_torch(model, g, bn_eps, folded=lambda name: True):
    """Copies the pack's weights into the torch modules.  `folded(name)`: the convolution is followed by a
    batch-norm that the pack folded into its weights (undone here, the torch model keeps its own)."""
    pack = og.Pack(g.to_bytes())
    mods = dict(model.named_modules())
    scale = np.sqrt(1.0 + bn_eps)
    loaded_bn = set()
    for rec, name in zip(pack.ops, pack.names):
        typ, cin, cout, r, s, groups = rec[0], rec[6], rec[7], rec[8], rec[9], rec[14]
        woff, boff = rec[18] | (rec[19] << 32), rec[20] | (rec[21] << 32)
        if typ == og.OP_CONV:
            m = mods[name]
            assert isinstance(m, nn.Conv2d), name
            w = pack.weights[woff: woff + cout * (cin // groups) * r * s].reshape(cout, cin // groups, r, s)
            with torch.no_grad():
                if rec[15] == 3:             # PReLU: the slopes follow the biases in the pack
                    mods[name + "_prelu"].weight.copy_(torch.from_numpy(pack.weights[boff + cout: boff + 2 * cout]))
                if m.bias is None:           # conv + batch-norm: the pack holds the folded weight
                    m.weight.copy_(torch.from_numpy(w * np.float32(scale if folded(name) else 1.0)))
                    if name + "_bn" in mods:     # a non-zero folded bias is the batch-norm's beta (mean 0)
                        mods[name + "_bn"].bias.copy_(torch.from_numpy(pack.weights[boff: boff + cout]))
                        loaded_bn.add(name + "_bn")
                else:                        # plain biased convolution
                    m.weight.copy_(torch.from_numpy(w))
                    m.bias.copy_(torch.from_numpy(pack.weights[boff: boff + cout]))
        elif typ == og.OP_AFFINE:        # a batch-norm kept as an operator: gamma = scale * sqrt(1 + eps), beta = bias
            m = mods[name]
            assert isinstance(m, nn.BatchNorm2d), name
            with torch.no_grad():
                m.weight.copy_(torch.from_numpy(pack.weights[woff: woff + cin] * np.float32(scale)))
                m.bias.copy_(torch.from_numpy(pack.weights[boff: boff + cin]))
                m.running_mean.zero_(); m.running_var.fill_(1.0)
            loaded_bn.add(name)
        elif typ == og.OP_DENSE:
            m = mods[name]
            assert isinstance(m, nn.Linear), name
            with torch.no_grad():
                m.weight.copy_(torch.from_numpy(pack.weights[woff: woff + cout * cin].reshape(cout, cin)))
                m.bias.copy_(torch.from_numpy(pack.weights[boff: boff + cout]))
    for name, m in model.named_modules():   # freshly initialised batch-norm statistics
        if isinstance(m, nn.BatchNorm2d) and name not in loaded_bn:
            nn.init.ones_(m.weight); nn.init.zeros_(m.bias)
            m.running_mean.zero_(); m.running_var.fill_(1.0)
    return pack


class ArcFaceR100(nn.Module):
    """LResNet100E-IR written out in torch (insightface's fresnet, version_unit 3, output "E") with modules
    named after the pack's operators; convolution batch-norms are separate modules here."""

    def __init__(self):
        super().__init__()
        eps = 2e-5

        def conv_bn(name, cin, cout, k, stride, pad, prelu):
            setattr(self, name, nn.Conv2d(cin, cout, k, stride, pad, bias=False))
            setattr(self, name + "_bn", nn.BatchNorm2d(cout, eps=eps))
            if prelu:
                setattr(self, name + "_prelu", nn.PReLU(cout))

        conv_bn("conv0", 3, 64, 3, 1, 1, True)
        self.plan = []
        cin = 64
        for si, (units, ch) in enumerate(zip([3, 13, 30, 3], [64, 128, 256, 512])):
            for ui in range(units):
                n = f"stage{si + 1}_unit{ui + 1}"
                first = ui == 0
                if first:
                    conv_bn(n + "_conv1sc", cin, ch, 1, 2, 0, False)
                setattr(self, n + "_bn1", nn.BatchNorm2d(cin, eps=eps))
                conv_bn(n + "_conv1", cin, ch, 3, 1, 1, True)
                conv_bn(n + "_conv2", ch, ch, 3, 2 if first else 1, 1, False)
                self.plan.append((n, first))
                cin = ch
        self.bn1 = nn.BatchNorm2d(512, eps=eps)
        self.pre_fc1 = nn.Linear(512 * 7 * 7, 512)          # the feature batch-norm is folded into it by the packer

    def _cb(self, name, x):
        x = getattr(self, name + "_bn")(getattr(self, name)(x))
        return getattr(self, name + "_prelu")(x) if hasattr(self, name + "_prelu") else x

    def forward(self, x):
        x = self._cb("conv0", x)
        for n, first in self.plan:
            sc = self._cb(n + "_conv1sc", x) if first else x
            y = getattr(self, n + "_bn1")(x)
            y = self._cb(n + "_conv1", y)
            x = self._cb(n + "_conv2", y) + sc
        return self.pre_fc1(torch.flatten(self.bn1(x), 1))


class UltraFaceRFB320(nn.Module):
    """The 320x240 receptive-field-block face detector written out in torch, modules named after the pack's
    operators; its post-processing (softmax scores, prior decoding to corner-form boxes) as torch tensor code with
    priors generated here.  Returns [4420*2 scores | 4420*4 boxes] flattened."""

    def __init__(self):
        super().__init__()
        eps = 1e-5
        self.relu_of = {}

        def cb(name, cin, cout, k, stride=1, pad=0, dil=1, groups=1, relu=True):
            setattr(self, name, nn.Conv2d(cin, cout, k, stride, pad, dilation=dil, groups=groups, bias=False))
            setattr(self, name + "_bn", nn.BatchNorm2d(cout, eps=eps))
            self.relu_of[name] = relu

        def dw(name, cin, cout, stride):
            cb(name + "_dw", cin, cin, 3, stride, 1, groups=cin)
            cb(name + "_pw", cin, cout, 1)

        cb("base_0", 3, 16, 3, 2, 1)
        chans = [(16, 32, 1), (32, 32, 2), (32, 32, 1), (32, 64, 2), (64, 64, 1), (64, 64, 1)]
        for i, (ci, co, st) in enumerate(chans):
            dw(f"base_{i + 1}", ci, co, st)
        n, inter = "base_7", 8
        cb(n + "_b0_0", 64, inter, 1, relu=False); cb(n + "_b0_1", inter, 16, 3, 1, 1); cb(n + "_b0_2", 16, 16, 3, 1, 2, 2, relu=False)
        cb(n + "_b1_0", 64, inter, 1, relu=False); cb(n + "_b1_1", inter, 16, 3, 1, 1); cb(n + "_b1_2", 16, 16, 3, 1, 3, 3, relu=False)
        cb(n + "_b2_0", 64, inter, 1, relu=False); cb(n + "_b2_1", inter, 12, 3, 1, 1); cb(n + "_b2_2", 12, 16, 3, 1, 1)
        cb(n + "_b2_3", 16, 16, 3, 1, 5, 5, relu=False)
        cb(n + "_shortcut", 64, 64, 1, relu=False); cb(n + "_linear", 48, 64, 1, relu=False)
        dw("base_8", 64, 128, 2); dw("base_9", 128, 128, 1); dw("base_10", 128, 128, 1)
        dw("base_11", 128, 256, 2); dw("base_12", 256, 256, 1)
        self.extras_0 = nn.Conv2d(256, 64, 1)
        self.extras_1_dw = nn.Conv2d(64, 64, 3, 2, 1, groups=64)
        self.extras_1_pw = nn.Conv2d(64, 256, 1)
        for i, (c, a) in enumerate(zip((64, 128, 256), (3, 2, 2))):
            for kind, per in (("cls", 2), ("reg", 4)):
                setattr(self, f"{kind}_{i}_dw", nn.Conv2d(c, c, 3, 1, 1, groups=c))
                setattr(self, f"{kind}_{i}_pw", nn.Conv2d(c, a * per, 1))
        self.cls_3 = nn.Conv2d(256, 3 * 2, 3, 1, 1)
        self.reg_3 = nn.Conv2d(256, 3 * 4, 3, 1, 1)
        # priors: per feature map, rows then columns then box sizes; (cx, cy, w, h) relative to 320 x 240
        pri = []
        for (fw, fh), boxes in zip(((40, 30), (20, 15), (10, 8), (5, 4)), ((10, 16, 24), (32, 48), (64, 96), (128, 192, 256))):
            for j in range(fh):
                for i in range(fw):
                    for mb in boxes:
                        pri.append([(i + 0.5) / fw, (j + 0.5) / fh, mb / 320.0, mb / 240.0])
        self.register_buffer("priors", torch.tensor(pri, dtype=torch.float32).clamp(0.0, 1.0))

    def _c(self, name, x):
        x = getattr(self, name + "_bn")(getattr(self, name)(x))
        return torch.relu(x) if self.relu_of[name] else x

    def _dw(self, name, x):
        return self._c(name + "_pw", self._c(name + "_dw", x))

    def forward(self, x):
        x = self._c("base_0", x)
        for i in range(1, 7):
            x = self._dw(f"base_{i}", x)
        n = "base_7"
        b0 = self._c(n + "_b0_2", self._c(n + "_b0_1", self._c(n + "_b0_0", x)))
        b1 = self._c(n + "_b1_2", self._c(n + "_b1_1", self._c(n + "_b1_0", x)))
        b2 = self._c(n + "_b2_3", self._c(n + "_b2_2", self._c(n + "_b2_1", self._c(n + "_b2_0", x))))
        f0 = torch.relu(self._c(n + "_linear", torch.cat([b0, b1, b2], 1)) + self._c(n + "_shortcut", x))
        f1 = self._dw("base_10", self._dw("base_9", self._dw("base_8", f0)))
        f2 = self._dw("base_12", self._dw("base_11", f1))
        f3 = torch.relu(self.extras_1_pw(torch.relu(self.extras_1_dw(torch.relu(self.extras_0(f2))))))
        conf, loc = [], []
        for i, f in enumerate((f0, f1, f2)):
            c = getattr(self, f"cls_{i}_pw")(torch.relu(getattr(self, f"cls_{i}_dw")(f)))
            r = getattr(self, f"reg_{i}_pw")(torch.relu(getattr(self, f"reg_{i}_dw")(f)))
            conf.append(c.permute(0, 2, 3, 1).reshape(c.shape[0], -1, 2))
            loc.append(r.permute(0, 2, 3, 1).reshape(r.shape[0], -1, 4))
        conf.append(self.cls_3(f3).permute(0, 2, 3, 1).reshape(x.shape[0], -1, 2))
        loc.append(self.reg_3(f3).permute(0, 2, 3, 1).reshape(x.shape[0], -1, 4))
        conf, loc = torch.cat(conf, 1), torch.cat(loc, 1)
        scores = torch.softmax(conf, dim=2)
        centre = loc[..., :2] * 0.1 * self.priors[..., 2:] + self.priors[..., :2]
        size = torch.exp(loc[..., 2:] * 0.2) * self.priors[..., 2:]
        boxes = torch.cat([centre - size / 2, centre + size / 2], dim=2)
        return torch.cat([scores.reshape(x.shape[0], -1), boxes.reshape(x.shape[0], -1)], 1)


CASES = [
    ("ultraface320", UltraFaceRFB320, 1e-5, (240, 320)),
    ("arcfaceresnet100", ArcFaceR100, 2e-5, 112),
    ("resnet18", lambda: torchvision.models.resnet18(weights=None), 1e-5, 224),
    ("resnet34", lambda: torchvision.models.resnet34(weights=None), 1e-5, 224),
    ("resnet50", lambda: torchvision.models.resnet50(weights=None), 1e-5, 224),
    ("mobilenet", lambda: torchvision.models.mobilenet_v2(weights=None), 1e-5, 224),
    ("squeezenet1_1", lambda: torchvision.models.squeezenet1_1(weights=None), 0.0, 224),
    ("densenet121", lambda: torchvision.models.densenet121(weights=None), 1e-5, 224),
    ("googlenet", lambda: torchvision.models.googlenet(weights=None, aux_logits=False, init_weights=False), 1e-3, 224),
    ("inception_v3", lambda: torchvision.models.inception_v3(weights=None, aux_logits=False,
                                                              transform_input=False, init_weights=False), 1e-3, 299),
]


@pytest.mark.parametrize("name,ctor,eps,size", CASES, ids=[c[0] for c in CASES])
def test_pack_matches_torchvision(oracle_lib, name, ctor, eps, size):
    kw = {"bias_std": 0.1} if name in ("squeezenet1_1", "ultraface320") else {}      # the models whose convolutions carry biases
    g = packer.MODELS[name](seed=1234, **kw)
    model = ctor().eval()
    # DenseNet: only conv0 and every conv1 are followed by a batch-norm; conv2 and the transition convs are not
    folded = (lambda n: n.endswith("conv0") or n.endswith("conv1")) if name == "densenet121" else (lambda n: True)
    pack = _load_into_torch(model, g, eps, folded)
    hw = size if isinstance(size, tuple) else (size, size)
    x = np.random.default_rng(5).standard_normal((3,) + hw, dtype=np.float32)
    with torch.no_grad():
        ref = model(torch.from_numpy(x)[None])[0].numpy()
    got = og.run(pack, x)
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() <= 2e-4 * scale
    if name == "ultraface320":       # a detector: the face / background decision of every prior, not one arg-max
        assert got.size == 4420 * 6 and ((got[:8840:2] > 0.5) == (ref[:8840:2] > 0.5)).mean() > 0.999
    else:
        assert int(got.argmax()) == int(ref.argmax())


def test_mnist_pack_matches_torch(oracle_lib):
    g = packer.mnist_cnn(seed=1234, bias_std=0.1)
    pack = og.Pack(g.to_bytes())
    W = pack.weights
    m = nn.Sequential(nn.Conv2d(1, 8, 5, 1, 2), nn.ReLU(), nn.MaxPool2d(2, 2), nn.Conv2d(8, 16, 5, 1, 2), nn.ReLU(),
                      nn.MaxPool2d(3, 3), nn.Flatten(0), nn.Linear(256, 10))
    convs = [m[0], m[3], m[7]]
    k = 0
    for rec in pack.ops:
        if rec[0] in (og.OP_CONV, og.OP_DENSE):
            woff, boff = rec[18], rec[20]
            with torch.no_grad():
                convs[k].weight.copy_(torch.from_numpy(W[woff: woff + convs[k].weight.numel()].reshape(convs[k].weight.shape)))
                convs[k].bias.copy_(torch.from_numpy(W[boff: boff + convs[k].bias.numel()]))
            k += 1
    x = np.random.default_rng(0).random((1, 28, 28), dtype=np.float32)
    with torch.no_grad():
        ref = m(torch.from_numpy(x)).numpy()
    got = og.run(pack, x)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5)


def test_algorithmic_work_matches_published_counts():
    """MAC totals per request quoted for the benchmark configurations."""
    assert packer.mnist_cnn().macs() == 156800 + 627200 + 2560
    assert abs(packer.resnet18().macs() / 1e9 - 1.814) < 0.002
    assert abs(packer.inception_v3().macs() / 1e9 - 5.713) < 0.003
    assert abs(packer.resnet50().macs() / 1e9 - 4.089) < 0.003
    assert abs(packer.mobilenet_v2().macs() / 1e9 - 0.3006) < 0.001


def test_pooling_branch_with_its_convolution_first_equals_the_original_order(oracle_lib):
    """packer.pooled_pointwise writes relu(bn(conv1x1(avgpool3x3(x)))) as relu(avgpool3x3(conv1x1(x)) + bias).  With the
    same weights and a non-zero bias both orders give the same tensor (fp32, 1e-5 of its range), borders included:
    the average pooling counts its zero padding, so it is linear and commutes with the 1x1 convolution."""
    eps = 1e-3
    a = packer.Graph("a", (24, 9, 11), seed=7, precision=0, bias_std=0.3)
    a.pooled_pointwise(a.input, 16, eps, "branch_pool")
    b = packer.Graph("b", (24, 9, 11), seed=7, precision=0, bias_std=0.3)
    y = b.avgpool(b.input, 3, 1, 1, True, name="avgpool")
    b.conv(y, 16, 1, 1, 0, bn_eps=eps, name="branch_pool.conv")
    # same seed, same order of draws: convolution weights first, then the bias
    pa, pb_ = og.Pack(a.to_bytes()), og.Pack(b.to_bytes())
    wa = pa.weights[pa.ops[0][18]: pa.ops[0][18] + 16 * 24]
    wb = pb_.weights[pb_.ops[1][18]: pb_.ops[1][18] + 16 * 24]
    np.testing.assert_array_equal(wa, wb)
    np.testing.assert_array_equal(pa.weights[pa.ops[1][20]: pa.ops[1][20] + 16], pb_.weights[pb_.ops[1][20]: pb_.ops[1][20] + 16])
    assert np.abs(pa.weights[pa.ops[1][20]: pa.ops[1][20] + 16]).max() > 0.05
    x = np.random.default_rng(3).standard_normal((24, 9, 11), dtype=np.float32)
    ya, yb = og.run(pa, x), og.run(pb_, x)
    assert ya.shape == yb.shape == (16 * 9 * 11,)
    assert float(np.abs(ya - yb).max()) <= 1e-5 * float(np.abs(yb).max())
    assert (ya == 0).mean() > 0.1 and (ya > 0).mean() > 0.1        # the ReLU is at work

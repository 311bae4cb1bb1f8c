"""Model packer: builds the operator graph of a served model and writes it, with
its weights, as one binary "pack" file that the job adapters load from
``$LLIS_MODELS_DIR`` at ``full_init`` time.

This is the counterpart of the reference's offline compile step
(sosp23_artifact/setup/onnx2tvm.py:14-29 turns an ONNX file into
``<model>-cuda_llis-pack.so``, which jobs/tvm_mnist/tvm_mnist.cpp:24-33 loads).
There is no code generation here: the pack is a flat table of operators that the
C++ graph executor maps onto hand-written sm_100a kernels.

Pack layout (little endian):
  header   64 B : magic "PB2PACK\\0", u32 version, n_tensors, n_ops,
                  input_tensor, output_tensor, precision (0 fp32, 1 bf16),
                  u64 weight_floats, char name[24]
  tensors  n_tensors x 16 B : u32 C, H, W, reserved        (batch is always 1)
  ops      n_ops x 96 B     : 24 x u32, see OP_FIELDS
  names    n_ops x 64 B     : NUL padded layer names
  weights  weight_floats x f32: conv weights OIHW, dense [out][in], biases [out]

Boundary layouts are the reference's: NCHW fp32 input, fp32 output vector.  A
concatenation is expressed by several producers writing channel slices
(``out_c_off``) of one tensor.  Weights are He-normal N(0, 2/fan_in) from a
seeded generator; batch-norm layers are folded into the preceding convolution
(w' = w * gamma / sqrt(var + eps), b' = beta - mean * gamma / sqrt(var + eps)
with the freshly initialised statistics gamma=1, beta=0, mean=0, var=1).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

MAGIC = b"PB2PACK\0"
VERSION = 1
NONE = 0xFFFFFFFF

OP_CONV, OP_DENSE, OP_MAXPOOL, OP_AVGPOOL, OP_GAP, OP_ADD, OP_SOFTMAX, OP_AFFINE, OP_DETECT = 1, 2, 3, 4, 5, 6, 7, 8, 9
ACT_NONE, ACT_RELU, ACT_RELU6, ACT_PRELU = 0, 1, 2, 3   # PReLU: the conv's bias block is [bias | per-channel slope]
FLAG_COUNT_INCLUDE_PAD = 1
FLAG_CEIL_MODE = 4          # informational: the output tensor's extent already says it
FLAG_POOL_BIAS = 8          # pooling: a per-channel bias (b_off) is added to the pooled value, then `act` applies

OP_FIELDS = ("type", "in0", "in1", "out", "rsv0", "out_c_off", "cin", "cout", "r", "s",
             "stride_h", "stride_w", "pad_h", "pad_w", "groups", "act", "flags", "rsv1",
             "w_off_lo", "w_off_hi", "b_off_lo", "b_off_hi", "dil_h", "dil_w")   # dilation 0 reads as 1


@dataclass
class Op:
    type: int
    in0: int
    out: int
    in1: int = NONE
    out_c_off: int = 0
    cin: int = 0
    cout: int = 0
    r: int = 1
    s: int = 1
    stride_h: int = 1
    stride_w: int = 1
    pad_h: int = 0
    pad_w: int = 0
    groups: int = 1
    act: int = ACT_NONE
    flags: int = 0
    w_off: int = 0
    b_off: int = 0
    name: str = ""
    dil_h: int = 1
    dil_w: int = 1

    def record(self) -> bytes:
        return struct.pack(
            "<24I", self.type, self.in0, self.in1, self.out, 0, self.out_c_off, self.cin,
            self.cout, self.r, self.s, self.stride_h, self.stride_w, self.pad_h, self.pad_w,
            self.groups, self.act, self.flags, 0, self.w_off & 0xFFFFFFFF, self.w_off >> 32,
            self.b_off & 0xFFFFFFFF, self.b_off >> 32, self.dil_h, self.dil_w)


def _pool_extent(n, k, stride, pad, ceil_mode):
    """Output extent of a pooling sweep; in ceil mode the last window may hang over the edge but must
    start inside the input or its left/top padding (ONNX MaxPool ceil_mode / torch MaxPool2d rule)."""
    if not ceil_mode:
        return (n + 2 * pad - k) // stride + 1
    o = -((n + 2 * pad - k) // -stride) + 1
    if (o - 1) * stride >= n + pad:
        o -= 1
    return o


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


@dataclass
class Graph:
    """Operator graph under construction.  Tensors are (C, H, W) at batch 1."""
    name: str
    in_shape: tuple
    seed: int = 1234
    precision: int = 1
    bias_std: float = 0.0           # biases are 0 as in the benchmark configs; tests set > 0
    round_weights_bf16: bool = False
    tensors: list = field(default_factory=list)
    ops: list = field(default_factory=list)
    weights: list = field(default_factory=list)
    n_floats: int = 0
    output: int = 0

    def __post_init__(self):
        self.rng = np.random.default_rng(self.seed)
        self.input = self.tensor(*self.in_shape)
        self.output = self.input

    # -- tensors and weights -------------------------------------------------
    def tensor(self, c, h, w) -> int:
        self.tensors.append((int(c), int(h), int(w)))
        return len(self.tensors) - 1

    def shape(self, t):
        return self.tensors[t]

    def _push(self, arr) -> int:
        arr = np.ascontiguousarray(arr, dtype=np.float32).ravel()
        off = self.n_floats
        self.weights.append(arr)
        self.n_floats += arr.size
        return off

    def _he(self, shape, fan_in, scale=1.0):
        w = self.rng.standard_normal(shape, dtype=np.float32) * np.float32(np.sqrt(2.0 / fan_in))
        w = (w * np.float32(scale)).astype(np.float32)
        if self.round_weights_bf16:
            u = w.view(np.uint32).astype(np.uint64)
            u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
            w = u.view(np.float32)
        return w

    def _bias(self, n):
        if self.bias_std > 0:
            return (self.rng.standard_normal(n, dtype=np.float32) * np.float32(self.bias_std))
        return np.zeros(n, dtype=np.float32)

    # -- operators -----------------------------------------------------------
    def conv(self, x, cout, k, stride=1, pad=0, groups=1, act=ACT_RELU, residual=None,
             out=None, out_c_off=0, bn_eps=None, name="", w_scale=1.0, dilation=1):
        c, h, w = self.shape(x)
        r, s = _pair(k)
        sh, sw = _pair(stride)
        ph, pw = _pair(pad)
        dh, dw = _pair(dilation)
        p = (h + 2 * ph - dh * (r - 1) - 1) // sh + 1
        q = (w + 2 * pw - dw * (s - 1) - 1) // sw + 1
        if out is None:
            out = self.tensor(cout, p, q)
        else:
            assert self.shape(out)[1:] == (p, q), (name, self.shape(out), p, q)
        fan_in = (c // groups) * r * s
        scale = w_scale * (1.0 if bn_eps is None else 1.0 / np.sqrt(1.0 + bn_eps))
        w_off = self._push(self._he((cout, c // groups, r, s), fan_in, scale))
        b_off = self._push(self._bias(cout))
        if act == ACT_PRELU:     # slopes right behind the biases: 0.25 (the usual initial value) +- 0.1
            self._push((0.25 + 0.2 * (self.rng.random(cout, dtype=np.float32) - 0.5)).astype(np.float32))
        self.ops.append(Op(OP_CONV, x, out, NONE if residual is None else residual, out_c_off,
                           c, cout, r, s, sh, sw, ph, pw, groups, act, 0, w_off, b_off, name, dh, dw))
        self.output = out
        return out

    def dense(self, x, n_out, act=ACT_NONE, name="", out_scale=None, out_bias=None):
        """Fully connected layer; out_scale / out_bias fold a following per-output affine (a 1-D batch-norm
        on the features) into the weights and biases."""
        c, h, w = self.shape(x)
        n_in = c * h * w
        out = self.tensor(n_out, 1, 1)
        wt = self._he((n_out, n_in), n_in)
        bs = self._bias(n_out)
        if out_scale is not None:
            wt = (wt * np.asarray(out_scale, np.float32).reshape(-1, 1)).astype(np.float32)
            bs = (bs * np.asarray(out_scale, np.float32) + np.asarray(out_bias, np.float32)).astype(np.float32)
        w_off = self._push(wt)
        b_off = self._push(bs)
        self.ops.append(Op(OP_DENSE, x, out, cin=n_in, cout=n_out, act=act, w_off=w_off,
                           b_off=b_off, name=name))
        self.output = out
        return out

    def _pool(self, typ, x, k, stride, pad, out, out_c_off, flags, name, act=ACT_NONE, bias=False):
        c, h, w = self.shape(x)
        r, s = _pair(k)
        sh, sw = _pair(stride)
        ph, pw = _pair(pad)
        p = _pool_extent(h, r, sh, ph, bool(flags & FLAG_CEIL_MODE))
        q = _pool_extent(w, s, sw, pw, bool(flags & FLAG_CEIL_MODE))
        if out is None:
            out = self.tensor(c, p, q)
        else:
            assert self.shape(out)[1:] == (p, q), (name, self.shape(out), p, q)
        b_off = 0
        if bias:
            flags |= FLAG_POOL_BIAS
            b_off = self._push(self._bias(c))
        self.ops.append(Op(typ, x, out, out_c_off=out_c_off, cin=c, cout=c, r=r, s=s,
                           stride_h=sh, stride_w=sw, pad_h=ph, pad_w=pw, act=act, flags=flags, b_off=b_off, name=name))
        self.output = out
        return out

    def maxpool(self, x, k, stride, pad=0, out=None, out_c_off=0, name="", ceil_mode=False):
        return self._pool(OP_MAXPOOL, x, k, stride, pad, out, out_c_off, FLAG_CEIL_MODE if ceil_mode else 0, name)

    def avgpool(self, x, k, stride, pad=0, count_include_pad=True, out=None, out_c_off=0, name="", act=ACT_NONE, bias=False):
        """Average pooling; with `bias` / `act` the pooled value gets a per-channel bias and an activation (the tail of a
        convolution + batch-norm + ReLU whose linear part ran BEFORE the pooling, see pooled_pointwise)."""
        return self._pool(OP_AVGPOOL, x, k, stride, pad, out, out_c_off,
                          FLAG_COUNT_INCLUDE_PAD if count_include_pad else 0, name, act, bias)

    def pooled_pointwise(self, x, cout, bn_eps, name, out=None, out_c_off=0):
        """relu(bn(conv1x1(avgpool3x3(x)))) - the pooling branch of an Inception block - computed as
        relu(avgpool3x3(conv1x1(x)) + bias): a 1x1 convolution and an average pooling that counts its zero padding are
        both linear and commute, and pooling AFTER the convolution moves cout instead of cin channels (4 to 10 times
        fewer in Inception-v3).  The operators keep the names `<name>.conv` and `<name>.avgpool`."""
        saved, self.bias_std = self.bias_std, 0.0
        y = self.conv(x, cout, 1, 1, 0, act=ACT_NONE, bn_eps=bn_eps, name=name + ".conv")      # linear part only: no bias
        self.bias_std = saved
        return self.avgpool(y, 3, 1, 1, True, out=out, out_c_off=out_c_off, name=name + ".avgpool", act=ACT_RELU, bias=True)

    def gap(self, x, name=""):
        c, h, w = self.shape(x)
        out = self.tensor(c, 1, 1)
        self.ops.append(Op(OP_GAP, x, out, cin=c, cout=c, r=h, s=w, name=name))
        self.output = out
        return out

    def add(self, a, b, act=ACT_NONE, name=""):
        c, h, w = self.shape(a)
        assert self.shape(b) == (c, h, w)
        out = self.tensor(c, h, w)
        self.ops.append(Op(OP_ADD, a, out, in1=b, cin=c, cout=c, act=act, name=name))
        self.output = out
        return out

    def affine(self, x, cin=None, act=ACT_RELU, bn_eps=1e-5, name=""):
        """Batch-norm (inference form) + activation on the first `cin` channels of x, as a per-channel
        scale and bias: scale = gamma / sqrt(var + eps), bias = beta - mean * scale with mean 0, var 1,
        gamma ~ 1 + 0.1 N(0,1), beta ~ 0.1 N(0,1) from the seed."""
        c, h, w = self.shape(x)
        cin = c if cin is None else cin
        assert 0 < cin <= c
        out = self.tensor(cin, h, w)
        gamma = (1.0 + 0.1 * self.rng.standard_normal(cin, dtype=np.float32)).astype(np.float32)
        beta = (0.1 * self.rng.standard_normal(cin, dtype=np.float32)).astype(np.float32)
        w_off = self._push(gamma / np.float32(np.sqrt(1.0 + bn_eps)))
        b_off = self._push(beta)
        self.ops.append(Op(OP_AFFINE, x, out, cin=cin, cout=cin, act=act, w_off=w_off, b_off=b_off, name=name))
        self.output = out
        return out

    def softmax(self, x, name=""):
        c, h, w = self.shape(x)
        out = self.tensor(c, h, w)
        self.ops.append(Op(OP_SOFTMAX, x, out, cin=c * h * w, cout=c * h * w, name=name))
        self.output = out
        return out

    def detect(self, head, anchors, priors, first, n_total, out=None, center_variance=0.1, size_variance=0.2, name=""):
        """Detection head of a single-shot detector over one feature map.  `head` has 6*anchors channels: class
        logits (anchor, class) then box regressions (anchor, coordinate); `priors` is [H*W*anchors][4] = (cx, cy,
        w, h) in (row, column, anchor) order.  Writes the softmax scores of this map's priors to
        out[(first+i)*2 ..] and their corner-form boxes to out[n_total*2 + (first+i)*4 ..]; `out` is the fp32
        model output of n_total*6 floats that all maps of the model share."""
        c, h, w = self.shape(head)
        assert c == 6 * anchors
        priors = np.asarray(priors, np.float32).reshape(h * w * anchors, 4)
        if out is None:
            out = self.tensor(n_total * 6, 1, 1)
        w_off = self._push(priors)
        b_off = self._push(np.array([center_variance, size_variance], np.float32))
        self.ops.append(Op(OP_DETECT, head, out, out_c_off=first, cin=anchors, cout=n_total, w_off=w_off, b_off=b_off, name=name))
        self.output = out
        return out

    # -- accounting ------------------------------------------------------------
    def macs(self) -> int:
        total = 0
        for op in self.ops:
            if op.type == OP_CONV:
                _, p, q = self.shape(op.out)
                total += op.cout * p * q * (op.cin // op.groups) * op.r * op.s
            elif op.type == OP_DENSE:
                total += op.cin * op.cout
        return total

    def layer_table(self):
        """Per-op algorithmic work: (name, type, flops, bytes at fp32/bf16 element size e)."""
        rows = []
        for op in self.ops:
            ci, hi, wi = self.shape(op.in0)
            co, p, q = self.shape(op.out)
            if op.type == OP_CONV:
                flops = 2 * op.cout * p * q * (op.cin // op.groups) * op.r * op.s
                elems = ci * hi * wi + op.cout * (op.cin // op.groups) * op.r * op.s + op.cout + op.cout * p * q
                if op.in1 != NONE:
                    elems += op.cout * p * q
            elif op.type == OP_DENSE:
                flops = 2 * op.cin * op.cout
                elems = op.cin + op.cin * op.cout + 2 * op.cout
            else:
                flops = 0
                elems = ci * hi * wi + op.cout * p * q
                if op.type == OP_ADD:
                    elems += ci * hi * wi
            rows.append((op.name, op.type, flops, elems))
        return rows

    # -- serialisation ---------------------------------------------------------
    def to_bytes(self) -> bytes:
        hdr = struct.pack("<8s6IQ24s", MAGIC, VERSION, len(self.tensors), len(self.ops),
                          self.input, self.output, self.precision, self.n_floats,
                          self.name.encode()[:23])
        assert len(hdr) == 64
        parts = [hdr]
        parts += [struct.pack("<4I", c, h, w, 0) for (c, h, w) in self.tensors]
        parts += [op.record() for op in self.ops]
        parts += [struct.pack("<64s", op.name.encode()[:63]) for op in self.ops]
        blob = np.concatenate(self.weights) if self.weights else np.zeros(0, np.float32)
        parts.append(blob.astype("<f4").tobytes())
        return b"".join(parts)

    def save(self, path):
        with open(path, "wb") as f:
            f.write(self.to_bytes())
        return path


# ---------------------------------------------------------------------------
# Model zoo: the topologies named by the benchmark configurations.
# ---------------------------------------------------------------------------

def mnist_cnn(seed=1234, precision=0, **kw) -> Graph:
    """ONNX-zoo mnist-8 topology (I/O sizes in jobs/tvm_mnist/tvm_mnist.cpp:12-18)."""
    g = Graph("mnist", (1, 28, 28), seed, precision, **kw)
    x = g.conv(g.input, 8, 5, 1, 2, name="conv1")
    x = g.maxpool(x, 2, 2, name="pool1")
    x = g.conv(x, 16, 5, 1, 2, name="conv2")
    x = g.maxpool(x, 3, 3, name="pool2")
    g.dense(x, 10, name="fc")
    return g


def _basic_block(g, x, planes, stride, name):
    eps = 1e-5
    cin = g.shape(x)[0]
    idt = x
    if stride != 1 or cin != planes:
        idt = g.conv(x, planes, 1, stride, 0, act=ACT_NONE, bn_eps=eps, name=name + ".downsample.0")
    y = g.conv(x, planes, 3, stride, 1, bn_eps=eps, name=name + ".conv1")
    return g.conv(y, planes, 3, 1, 1, act=ACT_RELU, residual=idt, bn_eps=eps, name=name + ".conv2")


def _bottleneck(g, x, planes, stride, name):
    eps = 1e-5
    cin = g.shape(x)[0]
    idt = x
    if stride != 1 or cin != planes * 4:
        idt = g.conv(x, planes * 4, 1, stride, 0, act=ACT_NONE, bn_eps=eps, name=name + ".downsample.0")
    y = g.conv(x, planes, 1, 1, 0, bn_eps=eps, name=name + ".conv1")
    y = g.conv(y, planes, 3, stride, 1, bn_eps=eps, name=name + ".conv2")
    return g.conv(y, planes * 4, 1, 1, 0, act=ACT_RELU, residual=idt, bn_eps=eps, name=name + ".conv3")


def _resnet(name, block, layers, seed, precision, num_classes, **kw) -> Graph:
    g = Graph(name, (3, 224, 224), seed, precision, **kw)
    x = g.conv(g.input, 64, 7, 2, 3, bn_eps=1e-5, name="conv1")
    x = g.maxpool(x, 3, 2, 1, name="maxpool")
    planes = 64
    for li, n in enumerate(layers):
        for bi in range(n):
            stride = 2 if (li > 0 and bi == 0) else 1
            x = block(g, x, planes, stride, f"layer{li + 1}.{bi}")
        planes *= 2
    x = g.gap(x, name="avgpool")
    g.dense(x, num_classes, name="fc")
    return g


def resnet18(seed=1234, precision=1, num_classes=1000, **kw) -> Graph:
    """ResNet-18 v1 (basic blocks 2-2-2-2), batch-norm folded."""
    return _resnet("resnet18", _basic_block, [2, 2, 2, 2], seed, precision, num_classes, **kw)


def resnet34(seed=1234, precision=1, num_classes=1000, **kw) -> Graph:
    """ResNet-34 v1 (basic blocks 3-4-6-3), batch-norm folded (jobs/tvm_resnet34 of the reference)."""
    return _resnet("resnet34", _basic_block, [3, 4, 6, 3], seed, precision, num_classes, **kw)


def resnet50(seed=1234, precision=1, num_classes=1000, **kw) -> Graph:
    """ResNet-50 v1.5 bottlenecks 3-4-6-3 (stride on the 3x3), batch-norm folded."""
    return _resnet("resnet50", _bottleneck, [3, 4, 6, 3], seed, precision, num_classes, **kw)


def mobilenet_v2(seed=1234, precision=1, num_classes=1000, **kw) -> Graph:
    """MobileNetV2 width 1.0: inverted residuals with depthwise 3x3 + ReLU6."""
    eps = 1e-5
    g = Graph("mobilenet", (3, 224, 224), seed, precision, **kw)
    x = g.conv(g.input, 32, 3, 2, 1, act=ACT_RELU6, bn_eps=eps, name="features.0.0")
    cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2),
           (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
    idx = 1
    for t, c, n, s in cfg:
        for i in range(n):
            stride = s if i == 0 else 1
            cin = g.shape(x)[0]
            hidden = cin * t
            base = f"features.{idx}.conv"
            y = x
            j = 0
            if t != 1:
                y = g.conv(y, hidden, 1, 1, 0, act=ACT_RELU6, bn_eps=eps, name=f"{base}.{j}.0")
                j += 1
            y = g.conv(y, hidden, 3, stride, 1, groups=hidden, act=ACT_RELU6, bn_eps=eps,
                       name=f"{base}.{j}.0")
            j += 1
            use_res = stride == 1 and cin == c
            x = g.conv(y, c, 1, 1, 0, act=ACT_NONE, residual=x if use_res else None, bn_eps=eps,
                       name=f"{base}.{j}")
            idx += 1
    x = g.conv(x, 1280, 1, 1, 0, act=ACT_RELU6, bn_eps=eps, name=f"features.{idx}.0")
    x = g.gap(x, name="avgpool")
    g.dense(x, num_classes, name="classifier.1")
    return g


def inception_v3(seed=1234, precision=1, num_classes=1000, size=299, **kw) -> Graph:
    """Inception-v3 (A/B/C/D/E blocks), no auxiliary head, batch-norm (eps 1e-3) folded.
    Every branch writes its channel slice of the block's output tensor directly.  The pooling branch of the A, C and E
    blocks (average pool 3x3 -> 1x1 convolution -> batch-norm -> ReLU) runs its convolution first (pooled_pointwise)."""
    eps = 1e-3
    g = Graph("inception_v3", (3, size, size), seed, precision, **kw)

    def bc(x, cout, k, stride=1, pad=0, name="", out=None, off=0):
        return g.conv(x, cout, k, stride, pad, bn_eps=eps, name=name + ".conv", out=out, out_c_off=off)

    x = bc(g.input, 32, 3, 2, 0, "Conv2d_1a_3x3")
    x = bc(x, 32, 3, 1, 0, "Conv2d_2a_3x3")
    x = bc(x, 64, 3, 1, 1, "Conv2d_2b_3x3")
    x = g.maxpool(x, 3, 2, name="maxpool1")
    x = bc(x, 80, 1, 1, 0, "Conv2d_3b_1x1")
    x = bc(x, 192, 3, 1, 0, "Conv2d_4a_3x3")
    x = g.maxpool(x, 3, 2, name="maxpool2")

    def block_a(x, pool_features, n):
        _, h, w = g.shape(x)
        out = g.tensor(64 + 64 + 96 + pool_features, h, w)
        bc(x, 64, 1, name=n + ".branch1x1", out=out, off=0)
        y = bc(x, 48, 1, name=n + ".branch5x5_1")
        bc(y, 64, 5, 1, 2, n + ".branch5x5_2", out=out, off=64)
        y = bc(x, 64, 1, name=n + ".branch3x3dbl_1")
        y = bc(y, 96, 3, 1, 1, n + ".branch3x3dbl_2")
        bc(y, 96, 3, 1, 1, n + ".branch3x3dbl_3", out=out, off=128)
        g.pooled_pointwise(x, pool_features, eps, n + ".branch_pool", out=out, out_c_off=224)
        return out

    def block_b(x, n):
        c, h, w = g.shape(x)
        p = (h - 3) // 2 + 1
        out = g.tensor(384 + 96 + c, p, p)
        bc(x, 384, 3, 2, 0, n + ".branch3x3", out=out, off=0)
        y = bc(x, 64, 1, name=n + ".branch3x3dbl_1")
        y = bc(y, 96, 3, 1, 1, n + ".branch3x3dbl_2")
        bc(y, 96, 3, 2, 0, n + ".branch3x3dbl_3", out=out, off=384)
        g.maxpool(x, 3, 2, out=out, out_c_off=480, name=n + ".maxpool")
        return out

    def block_c(x, c7, n):
        _, h, w = g.shape(x)
        out = g.tensor(768, h, w)
        bc(x, 192, 1, name=n + ".branch1x1", out=out, off=0)
        y = bc(x, c7, 1, name=n + ".branch7x7_1")
        y = bc(y, c7, (1, 7), 1, (0, 3), n + ".branch7x7_2")
        bc(y, 192, (7, 1), 1, (3, 0), n + ".branch7x7_3", out=out, off=192)
        y = bc(x, c7, 1, name=n + ".branch7x7dbl_1")
        y = bc(y, c7, (7, 1), 1, (3, 0), n + ".branch7x7dbl_2")
        y = bc(y, c7, (1, 7), 1, (0, 3), n + ".branch7x7dbl_3")
        y = bc(y, c7, (7, 1), 1, (3, 0), n + ".branch7x7dbl_4")
        bc(y, 192, (1, 7), 1, (0, 3), n + ".branch7x7dbl_5", out=out, off=384)
        g.pooled_pointwise(x, 192, eps, n + ".branch_pool", out=out, out_c_off=576)
        return out

    def block_d(x, n):
        c, h, w = g.shape(x)
        p = (h - 3) // 2 + 1
        out = g.tensor(320 + 192 + c, p, p)
        y = bc(x, 192, 1, name=n + ".branch3x3_1")
        bc(y, 320, 3, 2, 0, n + ".branch3x3_2", out=out, off=0)
        y = bc(x, 192, 1, name=n + ".branch7x7x3_1")
        y = bc(y, 192, (1, 7), 1, (0, 3), n + ".branch7x7x3_2")
        y = bc(y, 192, (7, 1), 1, (3, 0), n + ".branch7x7x3_3")
        bc(y, 192, 3, 2, 0, n + ".branch7x7x3_4", out=out, off=320)
        g.maxpool(x, 3, 2, out=out, out_c_off=512, name=n + ".maxpool")
        return out

    def block_e(x, n):
        _, h, w = g.shape(x)
        out = g.tensor(2048, h, w)
        bc(x, 320, 1, name=n + ".branch1x1", out=out, off=0)
        y = bc(x, 384, 1, name=n + ".branch3x3_1")
        bc(y, 384, (1, 3), 1, (0, 1), n + ".branch3x3_2a", out=out, off=320)
        bc(y, 384, (3, 1), 1, (1, 0), n + ".branch3x3_2b", out=out, off=704)
        y = bc(x, 448, 1, name=n + ".branch3x3dbl_1")
        y = bc(y, 384, 3, 1, 1, n + ".branch3x3dbl_2")
        bc(y, 384, (1, 3), 1, (0, 1), n + ".branch3x3dbl_3a", out=out, off=1088)
        bc(y, 384, (3, 1), 1, (1, 0), n + ".branch3x3dbl_3b", out=out, off=1472)
        g.pooled_pointwise(x, 192, eps, n + ".branch_pool", out=out, out_c_off=1856)
        return out

    x = block_a(x, 32, "Mixed_5b")
    x = block_a(x, 64, "Mixed_5c")
    x = block_a(x, 64, "Mixed_5d")
    x = block_b(x, "Mixed_6a")
    x = block_c(x, 128, "Mixed_6b")
    x = block_c(x, 160, "Mixed_6c")
    x = block_c(x, 160, "Mixed_6d")
    x = block_c(x, 192, "Mixed_6e")
    x = block_d(x, "Mixed_7a")
    x = block_e(x, "Mixed_7b")
    x = block_e(x, "Mixed_7c")
    x = g.gap(x, name="avgpool")
    g.dense(x, num_classes, name="fc")
    return g


def squeezenet1_1(seed=1234, precision=1, num_classes=1000, **kw) -> Graph:
    """SqueezeNet 1.1 (jobs/tvm_squeezenet1_1 of the reference): fire modules, ceil-mode max pooling,
    convolutional classifier + global average pool.  Convolutions carry biases (no batch-norm)."""
    g = Graph("squeezenet1_1", (3, 224, 224), seed, precision, **kw)

    def fire(x, squeeze, e1, e3, n):
        _, h, w = g.shape(x)
        y = g.conv(x, squeeze, 1, name=n + ".squeeze")
        out = g.tensor(e1 + e3, h, w)
        g.conv(y, e1, 1, name=n + ".expand1x1", out=out, out_c_off=0)
        g.conv(y, e3, 3, 1, 1, name=n + ".expand3x3", out=out, out_c_off=e1)
        return out

    x = g.conv(g.input, 64, 3, 2, 0, name="features.0")
    x = g.maxpool(x, 3, 2, ceil_mode=True, name="features.2")
    x = fire(x, 16, 64, 64, "features.3")
    x = fire(x, 16, 64, 64, "features.4")
    x = g.maxpool(x, 3, 2, ceil_mode=True, name="features.5")
    x = fire(x, 32, 128, 128, "features.6")
    x = fire(x, 32, 128, 128, "features.7")
    x = g.maxpool(x, 3, 2, ceil_mode=True, name="features.8")
    x = fire(x, 48, 192, 192, "features.9")
    x = fire(x, 48, 192, 192, "features.10")
    x = fire(x, 64, 256, 256, "features.11")
    x = fire(x, 64, 256, 256, "features.12")
    x = g.conv(x, num_classes, 1, name="classifier.1")
    g.gap(x, name="classifier.3")
    return g


def densenet121(seed=1234, precision=1, num_classes=1000, **kw) -> Graph:
    """DenseNet-121 (jobs/tvm_densenet121 of the reference), growth 32, blocks 6-12-24-16.  Each dense
    layer: norm1+relu1 on the concatenated features (a stand-alone affine operator: it precedes its
    convolution and the input is shared, so it cannot be folded), conv1 1x1 with norm2+relu2 folded,
    conv2 3x3 appended to the block's tensor."""
    eps = 1e-5
    growth, bn_size = 32, 4
    g = Graph("densenet121", (3, 224, 224), seed, precision, **kw)
    x = g.conv(g.input, 64, 7, 2, 3, bn_eps=eps, name="features.conv0")          # + norm0 + relu0
    c = 64
    feats = None
    for bi, n_layers in enumerate([6, 12, 24, 16]):
        _, h, w = g.shape(x)
        if bi == 0:
            h, w = _pool_extent(h, 3, 2, 1, False), _pool_extent(w, 3, 2, 1, False)
            feats = g.tensor(c + growth * n_layers, h, w)
            g.maxpool(x, 3, 2, 1, out=feats, out_c_off=0, name="features.pool0")
        else:
            # transition: norm + relu -> 2x2 average pool -> 1x1 convolution.  The published order is convolution, then
            # pool; both are linear with nothing in between, so they commute, and pooling first leaves the convolution
            # a quarter of the pixels (8 % of the model's multiply-adds)
            feats = g.tensor(c + growth * n_layers, h // 2, w // 2)
            y = g.avgpool(x, 2, 2, 0, True, name=f"features.transition{bi}.pool")
            g.conv(y, c, 1, act=ACT_NONE, out=feats, out_c_off=0, name=f"features.transition{bi}.conv")
        for li in range(n_layers):
            n = f"features.denseblock{bi + 1}.denselayer{li + 1}"
            y = g.affine(feats, cin=c, bn_eps=eps, name=n + ".norm1")
            y = g.conv(y, bn_size * growth, 1, bn_eps=eps, name=n + ".conv1")     # + norm2 + relu2
            g.conv(y, growth, 3, 1, 1, act=ACT_NONE, out=feats, out_c_off=c, name=n + ".conv2")
            c += growth
        if bi < 3:
            x = g.affine(feats, bn_eps=eps, name=f"features.transition{bi + 1}.norm")
            c //= 2
    y = g.affine(feats, bn_eps=eps, name="features.norm5")
    y = g.gap(y, name="avgpool")
    g.dense(y, num_classes, name="classifier")
    return g


def arcface_r100(seed=1234, precision=1, **kw) -> Graph:
    """ArcFace LResNet100E-IR (jobs/tvm_arcfaceresnet100 of the reference: 3x112x112 in, 512-d embedding out):
    3x3 stem + batch-norm + PReLU; improved residual units bn -> conv3x3 -> bn -> PReLU -> conv3x3(stride) -> bn
    (+ 1x1 stride-2 projection with batch-norm on the first unit of a stage), 3-13-30-3 units of 64-128-256-512
    channels; bn -> flatten -> fc 512 -> bn.  Batch-norms that follow a convolution (or the fc) are folded;
    the one that opens a unit is an affine operator.  The input is taken as already normalised."""
    eps = 2e-5
    g = Graph("arcfaceresnet100", (3, 112, 112), seed, precision, **kw)
    x = g.conv(g.input, 64, 3, 1, 1, act=ACT_PRELU, bn_eps=eps, name="conv0")
    for si, (units, ch) in enumerate(zip([3, 13, 30, 3], [64, 128, 256, 512])):
        for ui in range(units):
            n = f"stage{si + 1}_unit{ui + 1}"
            first = ui == 0
            sc = g.conv(x, ch, 1, 2, 0, act=ACT_NONE, bn_eps=eps, name=n + "_conv1sc") if first else x
            y = g.affine(x, act=ACT_NONE, bn_eps=eps, name=n + "_bn1")
            y = g.conv(y, ch, 3, 1, 1, act=ACT_PRELU, bn_eps=eps, name=n + "_conv1")
            # the unit's last batch-norm starts small (gamma 0.25), as deep residual nets are initialised, so that
            # activations do not grow by a constant factor in each of the 49 units
            x = g.conv(y, ch, 3, 2 if first else 1, 1, act=ACT_NONE, residual=sc, bn_eps=eps, name=n + "_conv2", w_scale=0.25)
    y = g.affine(x, act=ACT_NONE, bn_eps=eps, name="bn1")
    gamma = (1.0 + 0.1 * g.rng.standard_normal(512, dtype=np.float32)).astype(np.float32)
    beta = (0.1 * g.rng.standard_normal(512, dtype=np.float32)).astype(np.float32)
    g.dense(y, 512, name="pre_fc1", out_scale=gamma / np.float32(np.sqrt(1.0 + eps)), out_bias=beta)
    return g


def ultraface_priors(image_wh=(320, 240), min_boxes=((10, 16, 24), (32, 48), (64, 96), (128, 192, 256)), strides=(8, 16, 32, 64)):
    """Prior boxes of the single-shot face detector, one list per feature map: for every cell (row, column) and
    every min box size, (cx, cy, w, h) relative to the image, clipped to [0, 1].  The feature map of stride s has
    ceil(W/s) x ceil(H/s) cells and its cell pitch is the image extent divided by that count."""
    iw, ih = image_wh
    maps = []
    for boxes, st in zip(min_boxes, strides):
        fw, fh = -(-iw // st), -(-ih // st)
        scale_w, scale_h = iw / (iw / fw), ih / (ih / fh)
        pri = []
        for j in range(fh):
            for i in range(fw):
                for mb in boxes:
                    pri.append(((i + 0.5) / scale_w, (j + 0.5) / scale_h, mb / iw, mb / ih))
        maps.append(np.clip(np.asarray(pri, np.float32), 0.0, 1.0))
    return maps


def ultraface_rfb320(seed=1234, precision=1, **kw) -> Graph:
    """The 320x240 face detector with receptive-field blocks (jobs/tvm_ultraface320 of the reference: 3x240x320 in,
    4420 priors out).  Backbone of depthwise-separable units (3x3 depthwise + 1x1, batch-norm + ReLU after each,
    folded), 16-32-32-32-64-64-64 channels down to stride 8, one receptive-field block there (three branches of
    1x1 -> 3x3 (-> 3x3) -> 3x3 dilated by 2 / 3 / 5, concatenated, 1x1, plus a 1x1 shortcut, ReLU), 128 x3 at stride
    16, 256 x2 at stride 32 and an extra 1x1 -> separable 3x3 stride 2 at stride 64.  Each of the four maps feeds a
    class head and a box head (separable 3x3; plain 3x3 on the last map) with 3, 2, 2, 3 anchors per cell.
    Output: [4420 x 2 softmax scores | 4420 x 4 corner-form boxes]; the reference's adapter returns the first
    4420 x 2 floats (tvm_ultraface320.cpp:15-17), which are the first 4420 x 2 floats here."""
    eps = 1e-5
    g = Graph("ultraface320", (3, 240, 320), seed, precision, **kw)

    def dw_unit(x, cout, stride, n):
        c = g.shape(x)[0]
        y = g.conv(x, c, 3, stride, 1, groups=c, bn_eps=eps, name=n + "_dw")
        return g.conv(y, cout, 1, 1, 0, bn_eps=eps, name=n + "_pw")

    def bconv(x, cout, k, stride=1, pad=0, dilation=1, relu=True, n="", **k2):
        return g.conv(x, cout, k, stride, pad, act=ACT_RELU if relu else ACT_NONE, bn_eps=eps, dilation=dilation, name=n, **k2)

    def rfb(x, cout, n, reduce=8):
        c, h, w = g.shape(x)
        inter = c // reduce
        cat = g.tensor(6 * inter, h, w)
        b = bconv(x, inter, 1, relu=False, n=n + "_b0_0")
        b = bconv(b, 2 * inter, 3, 1, 1, n=n + "_b0_1")
        bconv(b, 2 * inter, 3, 1, 2, dilation=2, relu=False, n=n + "_b0_2", out=cat, out_c_off=0)
        b = bconv(x, inter, 1, relu=False, n=n + "_b1_0")
        b = bconv(b, 2 * inter, 3, 1, 1, n=n + "_b1_1")
        bconv(b, 2 * inter, 3, 1, 3, dilation=3, relu=False, n=n + "_b1_2", out=cat, out_c_off=2 * inter)
        b = bconv(x, inter, 1, relu=False, n=n + "_b2_0")
        b = bconv(b, inter // 2 * 3, 3, 1, 1, n=n + "_b2_1")
        b = bconv(b, 2 * inter, 3, 1, 1, n=n + "_b2_2")
        bconv(b, 2 * inter, 3, 1, 5, dilation=5, relu=False, n=n + "_b2_3", out=cat, out_c_off=4 * inter)
        short = bconv(x, cout, 1, relu=False, n=n + "_shortcut")
        return bconv(cat, cout, 1, relu=True, n=n + "_linear", residual=short)      # relu(linear(cat) + shortcut)

    x = g.conv(g.input, 16, 3, 2, 1, bn_eps=eps, name="base_0")
    for i, (cout, stride) in enumerate([(32, 1), (32, 2), (32, 1), (64, 2), (64, 1), (64, 1)]):
        x = dw_unit(x, cout, stride, f"base_{i + 1}")
    f0 = rfb(x, 64, "base_7")
    x = dw_unit(f0, 128, 2, "base_8")
    x = dw_unit(x, 128, 1, "base_9")
    f1 = dw_unit(x, 128, 1, "base_10")
    x = dw_unit(f1, 256, 2, "base_11")
    f2 = dw_unit(x, 256, 1, "base_12")
    x = g.conv(f2, 64, 1, 1, 0, name="extras_0")
    x = g.conv(x, 64, 3, 2, 1, groups=64, name="extras_1_dw")
    f3 = g.conv(x, 256, 1, 1, 0, name="extras_1_pw")

    anchors = (3, 2, 2, 3)
    priors = ultraface_priors()
    n_total = sum(len(p) for p in priors)
    out = g.tensor(n_total * 6, 1, 1)
    first = 0
    saved_bias = g.bias_std
    g.bias_std = max(g.bias_std, 0.5)          # head biases: spread the class logits so that scores are not all 0.5
    for i, (f, a) in enumerate(zip((f0, f1, f2, f3), anchors)):
        c, h, w = g.shape(f)
        assert h * w * a == len(priors[i])
        head = g.tensor(6 * a, h, w)
        if i < 3:
            y = g.conv(f, c, 3, 1, 1, groups=c, name=f"cls_{i}_dw")
            g.conv(y, 2 * a, 1, 1, 0, act=ACT_NONE, name=f"cls_{i}_pw", out=head, out_c_off=0)
            y = g.conv(f, c, 3, 1, 1, groups=c, name=f"reg_{i}_dw")
            g.conv(y, 4 * a, 1, 1, 0, act=ACT_NONE, name=f"reg_{i}_pw", out=head, out_c_off=2 * a)
        else:
            g.conv(f, 2 * a, 3, 1, 1, act=ACT_NONE, name=f"cls_{i}", out=head, out_c_off=0)
            g.conv(f, 4 * a, 3, 1, 1, act=ACT_NONE, name=f"reg_{i}", out=head, out_c_off=2 * a)
        g.detect(head, a, priors[i], first, n_total, out=out, name=f"detect_{i}")
        first += len(priors[i])
    g.bias_std = saved_bias
    return g


def googlenet(seed=1234, precision=1, num_classes=1000, **kw) -> Graph:
    """GoogLeNet / Inception-v1 (jobs/tvm_googlenet of the reference) in torchvision's form: batch-norm
    (eps 1e-3) folded, no auxiliary heads, 3x3 in the "5x5" branch, ceil-mode max pooling."""
    eps = 1e-3
    g = Graph("googlenet", (3, 224, 224), seed, precision, **kw)

    def bc(x, cout, k, stride=1, pad=0, name="", out=None, off=0):
        return g.conv(x, cout, k, stride, pad, bn_eps=eps, name=name + ".conv", out=out, out_c_off=off)

    def inception(x, c1, c3r, c3, c5r, c5, cp, n):
        _, h, w = g.shape(x)
        out = g.tensor(c1 + c3 + c5 + cp, h, w)
        bc(x, c1, 1, name=n + ".branch1", out=out, off=0)
        y = bc(x, c3r, 1, name=n + ".branch2.0")
        bc(y, c3, 3, 1, 1, n + ".branch2.1", out=out, off=c1)
        y = bc(x, c5r, 1, name=n + ".branch3.0")
        bc(y, c5, 3, 1, 1, n + ".branch3.1", out=out, off=c1 + c3)
        y = g.maxpool(x, 3, 1, 1, ceil_mode=True, name=n + ".branch4.0")
        bc(y, cp, 1, name=n + ".branch4.1", out=out, off=c1 + c3 + c5)
        return out

    x = bc(g.input, 64, 7, 2, 3, "conv1")
    x = g.maxpool(x, 3, 2, ceil_mode=True, name="maxpool1")
    x = bc(x, 64, 1, name="conv2")
    x = bc(x, 192, 3, 1, 1, "conv3")
    x = g.maxpool(x, 3, 2, ceil_mode=True, name="maxpool2")
    x = inception(x, 64, 96, 128, 16, 32, 32, "inception3a")
    x = inception(x, 128, 128, 192, 32, 96, 64, "inception3b")
    x = g.maxpool(x, 3, 2, ceil_mode=True, name="maxpool3")
    x = inception(x, 192, 96, 208, 16, 48, 64, "inception4a")
    x = inception(x, 160, 112, 224, 24, 64, 64, "inception4b")
    x = inception(x, 128, 128, 256, 24, 64, 64, "inception4c")
    x = inception(x, 112, 144, 288, 32, 64, 64, "inception4d")
    x = inception(x, 256, 160, 320, 32, 128, 128, "inception4e")
    x = g.maxpool(x, 2, 2, ceil_mode=True, name="maxpool4")
    x = inception(x, 256, 160, 320, 32, 128, 128, "inception5a")
    x = inception(x, 384, 192, 384, 48, 128, 128, "inception5b")
    x = g.gap(x, name="avgpool")
    g.dense(x, num_classes, name="fc")
    return g


MODELS = {
    "mnist": mnist_cnn,
    "resnet18": resnet18,
    "resnet34": resnet34,
    "resnet50": resnet50,
    "mobilenet": mobilenet_v2,
    "inception_v3": inception_v3,
    "squeezenet1_1": squeezenet1_1,
    "googlenet": googlenet,
    "densenet121": densenet121,
    "arcfaceresnet100": arcface_r100,
    "ultraface320": ultraface_rfb320,
}


def pack_file_name(model: str) -> str:
    """File the job adapter for `model` opens under $LLIS_MODELS_DIR."""
    return f"{model}-b200-pack.bin"


def write_all(models_dir, models=None, seed=1234, **kw):
    import os
    os.makedirs(models_dir, exist_ok=True)
    out = {}
    for m in (models or MODELS):
        g = MODELS[m](seed=seed, **kw)
        out[m] = g.save(os.path.join(models_dir, pack_file_name(m)))
    return out


if __name__ == "__main__":
    import sys
    d = sys.argv[1] if len(sys.argv) > 1 else "models"
    for m, p in write_all(d, sys.argv[2:] or None).items():
        print(m, p)

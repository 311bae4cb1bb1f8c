"""Generates tests/golden/golden_logits.npz: oracle (fp32 CPU) logits of the benchmark models on
seeded inputs and seeded He-normal weights.  Run from the repository root:
    python tests/golden/make_golden.py
The torchvision cross-check of the same packs lives in tests/test_oracle_models.py."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import graph as og  # noqa: E402
from paella_b200 import packer  # noqa: E402

INPUTS = {"mnist": ((1, 28, 28), "uniform"), "resnet18": ((3, 224, 224), "normal"), "inception_v3": ((3, 299, 299), "normal"),
          "resnet50": ((3, 224, 224), "normal"), "mobilenet": ((3, 224, 224), "normal"), "resnet34": ((3, 224, 224), "normal"),
          "squeezenet1_1": ((3, 224, 224), "normal"), "googlenet": ((3, 224, 224), "normal"), "densenet121": ((3, 224, 224), "normal"),
          "arcfaceresnet100": ((3, 112, 112), "normal"), "ultraface320": ((3, 240, 320), "normal")}


def make_input(model, seed=5):
    shape, dist = INPUTS[model]
    rng = np.random.default_rng(seed)
    return rng.random(shape, dtype=np.float32) if dist == "uniform" else rng.standard_normal(shape, dtype=np.float32)


if __name__ == "__main__":
    out = {}
    for m in INPUTS:
        g = packer.MODELS[m](seed=1234)
        out[m] = og.run(og.Pack(g.to_bytes()), make_input(m))
        print(m, out[m][:4], int(out[m].argmax()))
    np.savez(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_logits.npz"), **out)

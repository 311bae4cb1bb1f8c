"""The oracle reproduces the committed golden logits (guards the oracle and the packer's seeded
weights against drift between the machine that made the fixtures and the one running the tests)."""
import os

import numpy as np
import pytest

from oracle import graph as og
from paella_b200 import packer
from tests.golden.make_golden import make_input

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_logits.npz"))


@pytest.mark.parametrize("model", ["mnist", "resnet18", "mobilenet"])
def test_oracle_reproduces_golden(oracle_lib, model):
    g = packer.MODELS[model](seed=1234)
    y = og.run(og.Pack(g.to_bytes()), make_input(model))
    ref = GOLDEN[model]
    assert float(np.abs(y - ref).max()) <= 1e-5 * float(np.abs(ref).max())
    assert int(y.argmax()) == int(ref.argmax())

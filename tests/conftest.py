import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); deselected on CPU-only machines")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def golden_inputs(name, weights=None):
    """Regenerates the inputs of a golden layer case from its stored parameters."""
    from fused_moe_b200 import synth
    g = load_golden(name)
    T, e_local, off, seed, hidden, inter, zipf, tseed = [int(x) for x in g["params"]]
    inp = synth.make_inputs(T=T, e_local=e_local, local_expert_offset=off, seed=seed, hidden=hidden,
                            inter=inter, zipf=bool(zipf), weights=weights, token_seed=tseed)
    return g, inp


@pytest.fixture(scope="session")
def full_weights_cpu():
    """Weights of experts 0..31 at the benchmark shape (seed 0); ~20 s to draw, 1.4 GB."""
    from fused_moe_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    return synth.make_weights(32, 0, 0)


@pytest.fixture(scope="session")
def full_weights_gpu(full_weights_cpu):
    return tuple(t.cuda() for t in full_weights_cpu)

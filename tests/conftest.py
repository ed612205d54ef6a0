import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz"), allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


def alloc_cache_np(nb, P, h, d, int8_k=False):
    ng = d // 32
    kc = np.zeros((nb, P, h, d if int8_k else d // 2), dtype=np.int8 if int8_k else np.uint8)
    vc = np.zeros((nb, P, h, d // 2), dtype=np.uint8)
    mk = lambda: np.zeros((nb, P, h, ng), dtype=np.float16)
    return kc, vc, mk(), mk(), mk(), mk()


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")

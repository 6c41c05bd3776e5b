import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402

load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # The no-allocation entry point's test file is named to sort last; keep file order otherwise.
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz"),))


class Golden:
    """tests/golden/ttir_cpu_golden.npz: outputs of the reference's own CPU code (see generate.py)."""

    def __init__(self):
        self._z = np.load(os.path.join(ROOT, "tests", "golden", "ttir_cpu_golden.npz"))

    def __getitem__(self, name):
        import torch
        if name + "@bf16" in self._z.files:
            return torch.from_numpy(self._z[name + "@bf16"].copy()).view(torch.bfloat16)
        return torch.from_numpy(self._z[name].copy())

    def names(self):
        return [n.replace("@bf16", "") for n in self._z.files]


@pytest.fixture(scope="session")
def golden():
    return Golden()


@pytest.fixture(scope="session")
def rt():
    import ttmlir_b200.runtime_api as api
    return api


@pytest.fixture(scope="session")
def device(rt):
    if rt.get_num_available_devices() == 0:
        pytest.skip("no CUDA device")
    dev = rt.open_mesh_device(rt.MeshDeviceOptions(mesh_shape=[1, 1]))
    yield dev
    rt.close_mesh_device(dev)

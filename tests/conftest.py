import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "hidream_moe_small.npz")
    with np.load(path, allow_pickle=False) as z:
        data = {k: z[k] for k in z.files}
    data["meta"] = dict(zip(data.pop("meta_keys").tolist(), data.pop("meta_vals").tolist()))
    return data


@pytest.fixture(scope="session")
def golden_hunyuan3d():
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "hunyuan3d_moe_small.npz")
    with np.load(path, allow_pickle=False) as z:
        data = {k: z[k] for k in z.files}
    data["meta"] = dict(zip(data.pop("meta_keys").tolist(), data.pop("meta_vals").tolist()))
    return data


@pytest.fixture(scope="session")
def golden_attention():
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "hidream_attention_small.npz")
    with np.load(path, allow_pickle=False) as z:
        data = {k: z[k] for k in z.files}
    data["meta"] = dict(zip(data.pop("meta_keys").tolist(), data.pop("meta_vals").tolist()))
    return data


@pytest.fixture(scope="session")
def golden_block():
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "hidream_block_small.npz")
    with np.load(path, allow_pickle=False) as z:
        data = {k: z[k] for k in z.files}
    data["meta"] = dict(zip(data.pop("meta_keys").tolist(), data.pop("meta_vals").tolist()))
    return data


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    major, _ = torch.cuda.get_device_capability(0)
    if major != 10:
        pytest.skip("the kernels are sm_100a only")
    return torch.device("cuda:0")

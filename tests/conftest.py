import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from resinfer_b200 import nvfp4
    nvfp4.ensure_loaded(required=True)          # a GPU box without the native library is an error
    return torch.device("cuda", 0)


@pytest.fixture(scope="session")
def device_rcp(cuda_device):
    """rcp.approx.ftz.f32 evaluated on the device, as a numpy -> numpy callable."""
    import numpy as np
    import torch
    from resinfer_b200 import ops

    def fn(x):
        t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(cuda_device)
        return ops.rcp_approx(t).cpu().numpy()

    return fn


@pytest.fixture(scope="session")
def ref_ops(cuda_device):
    """The reference project's own quantiser kernels (oracle/_ref), or None when not built."""
    import torch
    lib = os.path.join(ROOT, "oracle", "_ref", "libnvfp4_ref.so")
    if not os.path.exists(lib):
        return None
    torch.ops.load_library(lib)
    return torch.ops.nvfp4_ref

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (oracle/ftq_oracle.c), built on demand."""
    from tests import oracle_lib
    return oracle_lib.load()


@pytest.fixture(scope="session")
def lib_path():
    path = os.path.join(ROOT, "ft_gemm_b200", "lib", "libft_gemm_b200.so")
    if not os.path.exists(path):
        subprocess.run(["make", "-C", ROOT, "lib"], check=True, stdout=subprocess.DEVNULL)
    return path

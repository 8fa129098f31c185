import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _bounds_word_stays_clear(request):
    """Under COCCL_CHECKED_KERNELS=1 (the bounds-checked twin of the kernel library) every GPU test also asserts that no
    codec access left its chunk: the error word is read, and cleared, after the test."""
    yield
    if os.environ.get("COCCL_CHECKED_KERNELS", "") in ("", "0") or request.node.get_closest_marker("gpu") is None:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from coccl_b200 import _lib
    checked, word = _lib.bounds_word(reset=True)
    assert checked, "COCCL_CHECKED_KERNELS is set but the plain library was loaded"
    assert word[0] == 0, f"a codec access left its chunk: site {word[0] & 0xff}, element {word[1] | (word[2] << 32)}, " \
                         f"payload end {word[3]} of {word[4]}, chunk end {word[5]} of {word[6]}"

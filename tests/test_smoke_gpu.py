"""The entry point the driver runs on a GPU box: a few tokens from a tiny random model, compared
with the plain implementation."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_smoke():
    sys.path.insert(0, ROOT)
    import __graft_entry__
    __graft_entry__.smoke()

"""The entry point the build driver runs on a GPU box: one tiny layer step checked against the oracle."""
import pytest

pytestmark = pytest.mark.gpu


def test_smoke_entry_point():
    import __graft_entry__
    __graft_entry__.smoke()

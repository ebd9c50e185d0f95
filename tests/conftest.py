import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture
def isolated_rule_cache(tmp_path, monkeypatch):
    """Redirect the superoptimizer's on-disk cache into a temp dir."""
    from pccl_b200.dsl.superopt import rule_db
    monkeypatch.setattr(rule_db, "_cache_dir", lambda: tmp_path / "superopt")
    return tmp_path / "superopt"

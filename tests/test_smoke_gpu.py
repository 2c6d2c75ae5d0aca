"""The driver's smoke hook runs as a test too, so a change that breaks it shows up here first."""
import pytest

pytestmark = pytest.mark.gpu


def test_smoke_hook_runs(capsys):
    import __graft_entry__
    __graft_entry__.smoke()
    assert "smoke ok" in capsys.readouterr().out

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _own_rendezvous_port(monkeypatch):
    """In-process single-rank trainers rendezvous on MASTER_PORT: give every test its own free port so that tests can run
    side by side (pytest-xdist) and a lingering socket of the previous test never collides."""
    if "MASTER_PORT" not in os.environ:
        import socket

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            monkeypatch.setenv("MASTER_PORT", str(s.getsockname()[1]))
    yield
    # an in-process trainer test must not leave its default process group to the next test
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def _registry_snapshot():
    """repr of every model flavor registered by the model packages imported so far."""
    out = {}
    for name, mod in list(sys.modules.items()):
        if mod is None or not (name.startswith("torchtitan_b200.models.") or name.startswith("torchtitan_b200.experiments.")):
            continue
        for attr, value in list(vars(mod).items()):
            if attr.endswith("_configs") and isinstance(value, dict):
                for flavor, cfg in value.items():
                    out[(name, attr, flavor)] = repr(cfg)
    return out


@pytest.fixture(autouse=True)
def _flavor_registries_stay_untouched():
    """The flavor registries hold shared objects: a test that shrinks one in place changes what every later test builds.
    Copy first (``dataclasses.replace``) and replace nested parts instead of assigning into them."""
    before = _registry_snapshot()
    yield
    after = _registry_snapshot()
    changed = [k for k, v in before.items() if after.get(k) != v]
    assert not changed, f"this test modified registered model flavors in place: {changed}"

import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Tiny random models A and B, written once per test session into a temporary folder."""
    from tiny_configs import TINY_A, TINY_A_INIT, TINY_B, TINY_B_INIT, TINY_C, TINY_C_INIT
    from velomind_b200 import write_random_model
    root = tmp_path_factory.mktemp("models")
    return {
        "tiny_a": write_random_model(str(root / "tiny_a"), TINY_A, **TINY_A_INIT),
        "tiny_b": write_random_model(str(root / "tiny_b"), TINY_B, **TINY_B_INIT),
        "tiny_c": write_random_model(str(root / "tiny_c"), TINY_C, **TINY_C_INIT),
    }


@pytest.fixture(scope="session")
def toy_plugin(tmp_path_factory):
    """tests/cpp/toy_parts.cu built into a plug-in library and loaded: its parts and architectures are registered."""
    import toy_plugin as plugin
    return plugin.load(str(tmp_path_factory.mktemp("toy_plugin")))

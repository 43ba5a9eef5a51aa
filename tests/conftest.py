import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # tests in files named test_zz_* run last, whatever order the files were given in
    items.sort(key=lambda it: 1 if Path(str(it.fspath)).name.startswith("test_zz_") else 0)


@pytest.fixture(scope="session")
def tiny_model_dirs(tmp_path_factory):
    """The two tiny test models, written once per session into a temporary folder (bfloat16
    storage, so the float32 engine, the bfloat16 engine and the plain implementation all read the
    same values)."""
    from plain_llama import TINY_WEIGHTS, tiny_configs
    from tokasaurus_b200.weights import write_model_folder

    root = tmp_path_factory.mktemp("tiny_models")
    dirs = []
    for i, (cfg, w) in enumerate(zip(tiny_configs(), TINY_WEIGHTS)):
        dirs.append(write_model_folder(root / f"cfg{i}", cfg, seed=w["seed"], std=w["std"], norm_init=w["norm_init"]))
    return dirs

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


TINY = dict(NL=2, DM=128, NH=4, NKV=2, DH=32, DFF=256, NV=300)
# ragged on purpose: K not a multiple of 112 or 64, vocabulary not a multiple of the rows-per-warp
RAGGED = dict(NL=3, DM=192, NH=6, NKV=2, DH=32, DFF=328, NV=1001)
# GQA group of 8 and head_dim 128, the Qwen3-32B head geometry at toy width
WIDE = dict(NL=2, DM=256, NH=8, NKV=1, DH=128, DFF=512, NV=512)
# GQA group of 4 and head_dim 128, the Qwen3-8B head geometry at toy width
GQA4 = dict(NL=2, DM=256, NH=8, NKV=2, DH=128, DFF=512, NV=512)


@pytest.fixture(scope="session")
def tiny_file(tmp_path_factory):
    import oracle_lib as ol
    d = tmp_path_factory.mktemp("tiny")
    path = str(d / "tiny.weights")
    ol.write_v3(path, TINY, ol.synth_tensors(TINY, seed=3))
    return path


def make_model_file(tmp_path_factory, cfg, seed, name):
    import oracle_lib as ol
    d = tmp_path_factory.mktemp(name)
    path = str(d / (name + ".weights"))
    ol.write_v3(path, cfg, ol.synth_tensors(cfg, seed=seed))
    return path


@pytest.fixture(scope="session")
def ragged_file(tmp_path_factory):
    return make_model_file(tmp_path_factory, RAGGED, 11, "ragged")


@pytest.fixture(scope="session")
def wide_file(tmp_path_factory):
    return make_model_file(tmp_path_factory, WIDE, 12, "wide")


@pytest.fixture(scope="session")
def gqa4_file(tmp_path_factory):
    return make_model_file(tmp_path_factory, GQA4, 13, "gqa4")

import hashlib
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def dig(a):
    if isinstance(a, np.ndarray):
        a = np.ascontiguousarray(a).tobytes()
    return hashlib.sha256(bytes(a)).hexdigest()


@pytest.fixture(scope="session")
def golden():
    with open(os.path.join(ROOT, "tests", "golden", "p3_golden.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def orc():
    from oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The unmodified reference behind its C shim, where oracle/_ref was built."""
    from oracle import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libp3ref.so not built")
    return Reference()


@pytest.fixture(scope="session")
def ref_or_none():
    """Reference shim if built, else None (tests then rely on the oracle and the goldens)."""
    from oracle import Reference
    return Reference() if Reference.available() else None


@pytest.fixture(scope="session")
def zk():
    import zkh_import
    return zkh_import.load()


@pytest.fixture(scope="session")
def prover(zk):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.init()
    p = zk.Prover(0, torch.cuda.current_stream().cuda_stream)   # same stream as torch: ordered with its copies
    yield p
    p.close()


def lcg_cols(orc, n, count, seed):
    cols, s = [], seed
    for _ in range(count):
        a, s = orc.lcg(n, s)
        cols.append(a)
    return cols

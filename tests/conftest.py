"""Shared fixtures. GPU tests are marked `gpu`; everything else runs on a GPU-less host."""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device")


@pytest.fixture(scope="session")
def oracle():
    """The plain-C restatement of the reference CPU path (test infrastructure)."""
    from oracle import ref_lib
    if not ref_lib.have_oracle():
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"], check=True, capture_output=True)
    return ref_lib.OracleLib()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU code compiled in place (only where oracle/_ref was built)."""
    from oracle import ref_lib
    if not ref_lib.have_ref():
        pytest.skip("oracle/_ref/libtl_ref.so not built (needs the reference sources)")
    return ref_lib.RefLib()


@pytest.fixture(scope="session")
def tl():
    """The product library, initialised on cuda:0. GPU tests fail (not skip) without it."""
    import tensorlib_b200 as t
    if not os.path.exists(t.LIB_PATH):
        subprocess.run([sys.executable, "-m", "tensorlib_b200.build"], cwd=ROOT, check=True)
    t.init(0)
    return t


@pytest.fixture(scope="session")
def golden_tiny():
    return np.load(os.path.join(GOLDEN, "tiny_llama2.npz"))


@pytest.fixture(scope="session")
def golden_ops():
    return np.load(os.path.join(GOLDEN, "ops.npz"))


@pytest.fixture(scope="session")
def golden_sweep():
    return np.load(os.path.join(GOLDEN, "matmul_sweep.npz"))


@pytest.fixture(scope="session")
def tiny_payload():
    from tensorlib_b200 import synth
    return synth.llama2c_payload(synth.TINY, 20240229)


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint16)


def assert_bit_equal(a: np.ndarray, b: np.ndarray, what: str = ""):
    a16, b16 = bits(a), bits(b)
    assert a16.shape == b16.shape, f"{what}: shape {a16.shape} vs {b16.shape}"
    bad = np.flatnonzero(a16.reshape(-1) != b16.reshape(-1))
    assert bad.size == 0, (f"{what}: {bad.size}/{a16.size} fp16 values differ, first at {bad[:5]}: "
                           f"{a.reshape(-1)[bad[:5]]} vs {b.reshape(-1)[bad[:5]]}")

"""The oracle against the reference's own known-answer tests and against the committed golden vectors (no GPU)."""
import os
import subprocess

import numpy as np
import pytest

from katago_b200 import modelfile as mf
from tests.golden.make_golden import CASES

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KATAGO_ORACLE = os.path.join(ROOT, "oracle", "_ref", "katago_oracle")
needs_ref = pytest.mark.skipif(not os.path.exists(KATAGO_ORACLE), reason="oracle/_ref/katago_oracle not built (needs the reference checkout)")


@needs_ref
def test_reference_layer_known_answers():
    """cpp/tests/testnn.cpp:107-921: conv 1x1/3x3/5x5, batch norm with mask, residual block, gpool block."""
    r = subprocess.run([KATAGO_ORACLE, "runnnlayertests"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Test failed" not in r.stdout and "mismatch" not in r.stdout.lower(), r.stdout[-2000:]
    assert "Tested 14 configurations" in r.stdout


@needs_ref
def test_reference_tiny_net_known_answers(tmp_path):
    """cpp/tests/tinymodel.cpp:129-196: value, score, 361 policy and ownership numbers of the embedded net."""
    r = subprocess.run([KATAGO_ORACLE, "runtinynntests", str(tmp_path), "1.0"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    assert "Tiny net sanity check complete" in r.stdout + r.stderr


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_golden_vectors(name, oracle):
    factory, n, sizes, seed = CASES[name]
    golden = np.load(os.path.join(ROOT, "tests", "golden", f"{name}.npz"))
    om = oracle.OracleModel(mf.to_blob(factory()))
    sp, gl = mf.random_positions(n, seed=seed, board_sizes=sizes)
    out = om.forward(sp, gl)
    for k in golden.files:
        # same code, same seeds: differences can only come from compiler/FMA choices
        assert np.abs(out[k] - golden[k]).max() <= 2e-5 * max(1.0, np.abs(golden[k]).max()), k


def test_oracle_masking_and_batch_independence(oracle):
    """A row's result must not depend on its neighbours in the batch or on the board size of other rows."""
    om = oracle.OracleModel(mf.to_blob(mf.make_b18c384nbt(num_blocks=2)))
    sp, gl = mf.random_positions(3, seed=11, board_sizes=[13, 19, 9])
    full = om.forward(sp, gl)
    for i in range(3):
        one = om.forward(sp[i : i + 1], gl[i : i + 1])
        for k in full:
            assert np.abs(one[k][0] - full[k][i]).max() <= 1e-5 * max(1.0, np.abs(full[k]).max())
    # off-board policy/ownership positions of the 9x9 board carry no information from the board
    own = full["ownership"][2].reshape(19, 19)
    assert np.all(own[9:, :] == own[9, 9]) or np.allclose(own[9:, :], 0.0, atol=1e-6)


def test_oracle_rejects_malformed_blobs(oracle):
    blob = mf.to_blob(mf.make_b6c96())
    with pytest.raises(RuntimeError):
        oracle.OracleModel(blob[: len(blob) // 2])
    with pytest.raises(RuntimeError):
        oracle.OracleModel(b"\x00" * 64)

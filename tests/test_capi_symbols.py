"""The C-ABI library loads on a machine without a GPU and exports every symbol include/katab200.h declares;
host-only entry points behave; compute entry points fail loudly instead of falling back to the CPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from katago_b200 import capi
from katago_b200 import modelfile as mf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "katab200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = capi.lib()
    declared = _declared_symbols()
    assert len(declared) >= 20
    missing = [s for s in declared if not hasattr(L, s)]
    assert missing == []
    assert sorted(capi.EXPORTED_SYMBOLS) == declared


def test_model_parsing_is_host_only_and_validates():
    m = capi.Model(mf.to_blob(mf.make_b18c384nbt(num_blocks=2)))
    assert (m.version, m.in_c, m.in_global_c, m.policy_c, m.value_c, m.score_c, m.trunk_c, m.num_blocks) == (15, 22, 19, 2, 3, 6, 384, 2)
    blob = mf.to_blob(mf.make_b6c96())
    with pytest.raises(capi.KBError):
        capi.Model(blob[:1000])
    with pytest.raises(capi.KBError):
        capi.Model(b"")
    # corrupt a channel count: the policy head no longer chains with the trunk
    bad = bytearray(blob)
    words = np.frombuffer(bytes(bad), "<u4").copy()
    words[5 + 1] = 23  # MODEL record: ints start at word 5 (tag, nInts, then version, inC, ...)
    with pytest.raises(capi.KBError):
        capi.Model(words.tobytes())


def _has_gpu():
    try:
        return capi.device_count() > 0
    except capi.KBError:
        return False


@pytest.mark.skipif(_has_gpu(), reason="checks the behaviour on a machine WITHOUT a GPU")
def test_compute_fails_loudly_without_gpu():
    m = capi.Model(mf.to_blob(mf.make_b6c96()))
    with pytest.raises(capi.KBError):
        capi.Handle(m, 4, precision=capi.PRECISION_FP32)
    with pytest.raises(capi.KBError):
        g = mf._Gen(1)
        capi.eval_layer(mf.layer_blob(g.conv(3, 4, 4)), np.zeros((1, 5, 5, 4), np.float32), None, 4)

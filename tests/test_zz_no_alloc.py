"""kb_conv_noalloc: the convolution entry point for callers that are not allowed to allocate device memory
(plug-ins inside another application's memory pool, latency-critical loops that must stay clear of
cudaMalloc's locks and implicit synchronisation).  Its working memory is an array built into the library.

The file name sorts last on purpose: if this addition fails, a run that stops at the first failure has already
executed every other test.  The check: through the C ABI, on device buffers owned by the test, the result must
equal that of the allocating entry point kb_eval_layer and that of the CPU oracle -- on calls in a row with different
shapes, since the built-in array keeps whatever the previous call wrote -- and a call must leave the amount of free
device memory exactly as it found it.
"""
import numpy as np
import pytest

from katago_b200 import capi
from katago_b200 import modelfile as mf

pytestmark = pytest.mark.gpu


def _run_pair(torch, conv, x, oracle, check_free_memory=False):
    n, ylen, xlen, ic = x.shape
    oc, k = conv["outC"], conv["kY"]
    ref = capi.eval_layer(mf.layer_blob(conv), x, None, oc, precision=capi.PRECISION_FP32)  # existing, allocating path
    ref_cpu = oracle.eval_layer(mf.layer_blob(conv), x, None, oc)                            # CPU oracle
    d_in = torch.from_numpy(x).cuda()
    d_w = torch.from_numpy(np.ascontiguousarray(conv["w"], np.float32)).cuda()  # [oc][ic][y][x]
    d_out = torch.full((n, ylen, xlen, oc), float("nan"), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    capi.conv_noalloc(d_in.data_ptr(), d_w.data_ptr(), d_out.data_ptr(), n, xlen, ylen, ic, oc, k, k, 0)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    if check_free_memory:
        # the property the entry point exists for (checked on calls after the first, whose set-up may load the kernels)
        assert free_after == free_before, (free_before, free_after)
    got = d_out.cpu().numpy()
    assert np.all(np.isfinite(got))
    assert np.abs(got - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())
    assert np.abs(got - ref_cpu).max() <= 1e-4 * max(1.0, np.abs(ref_cpu).max())


def test_conv_noalloc_matches_allocating_entry_point_twice(oracle):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    g = mf._Gen(4242)
    rng = np.random.default_rng(17)
    # first call: 3x3, 9 boards of 19x19 (3600 padded rows, close to the 4096-row limit), 22 -> 64 channels
    _run_pair(torch, g.conv(3, 22, 64), rng.standard_normal((9, 19, 19, 22)).astype(np.float32), oracle)
    # second call right after, smaller and differently shaped: stale scratch contents must not leak into it
    _run_pair(torch, g.conv(5, 7, 5), rng.standard_normal((2, 9, 13, 7)).astype(np.float32), oracle, check_free_memory=True)
    _run_pair(torch, g.conv(1, 64, 48), rng.standard_normal((3, 19, 19, 64)).astype(np.float32), oracle, check_free_memory=True)
    _run_pair(torch, g.conv(3, 22, 64), rng.standard_normal((9, 19, 19, 22)).astype(np.float32), oracle, check_free_memory=True)


def test_conv_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    buf = torch.zeros(1024, device="cuda")
    p = buf.data_ptr()
    with pytest.raises(capi.KBError, match="exceed the built-in scratch"):
        capi.conv_noalloc(p, p, p, 11, 19, 19, 8, 8, 3, 3)  # 11 boards -> 4400 rows > 4096
    with pytest.raises(capi.KBError, match="channels"):
        capi.conv_noalloc(p, p, p, 1, 19, 19, 65, 8, 3, 3)
    with pytest.raises(capi.KBError, match="kernel size"):
        capi.conv_noalloc(p, p, p, 1, 19, 19, 8, 8, 7, 7)
    with pytest.raises(capi.KBError, match="NULL"):
        capi.conv_noalloc(0, p, p, 1, 19, 19, 8, 8, 3, 3)

"""Shared test helpers: board symmetries in numpy and the parity metrics of the reference's
testgpuerror harness (cpp/tests/testnnevalcanary.cpp:249-307), computed after the same
post-processing NNEvaluator applies (cpp/neuralnet/nneval.cpp:945-1240)."""
import numpy as np


def apply_sym(a, sym, reverse):
    """a [H,W,C]; scatter form of SymmetryHelpers (cpp/neuralnet/nninputs.cpp:529-575)."""
    H, W = a.shape[0], a.shape[1]
    transpose = (sym & 4) != 0 and H == W
    fx, fy = (sym & 2) != 0, (sym & 1) != 0
    if transpose and not reverse:
        fx, fy = fy, fx
    hh, ww = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
    if not transpose:
        h2 = np.where(fy, H - 1 - hh, hh)
        w2 = np.where(fx, W - 1 - ww, ww)
    else:
        h2 = np.where(fy, H - 1 - ww, ww)
        w2 = np.where(fx, W - 1 - hh, hh)
    out = np.empty_like(a)
    out[h2, w2] = a[hh, ww]
    return out


def symmetrise_inputs(spatial, syms):
    return np.stack([apply_sym(spatial[i], int(syms[i]), False) for i in range(spatial.shape[0])])


def unsymmetrise_outputs(out, syms, nn_len=19):
    """Maps network-frame policy/ownership back to the caller's frame (inverse symmetry)."""
    n = out["policy"].shape[0]
    res = dict(out)
    res["policy"] = np.stack([apply_sym(out["policy"][i].reshape(nn_len, nn_len, -1), int(syms[i]), True).reshape(nn_len * nn_len, -1) for i in range(n)])
    res["ownership"] = np.stack([apply_sym(out["ownership"][i].reshape(nn_len, nn_len, 1), int(syms[i]), True).reshape(nn_len * nn_len) for i in range(n)])
    return res


def _softmax(x, axis=-1):
    x = x - x.max(axis=axis, keepdims=True)
    e = np.exp(x)
    return e / e.sum(axis=axis, keepdims=True)


def parity_metrics(got, ref, mask, score_mult=20.0):
    """Per-position error metrics.  mask [n,S] = on-board points (legal-move stand-in).
    Returns dict of arrays [n]: winrate (fraction), score (points), lead (points), policy_kl, policy_max (prob), ownership."""
    n = mask.shape[0]
    res = {}
    vg, vr = _softmax(got["value"].astype(np.float64)), _softmax(ref["value"].astype(np.float64))
    res["winrate"] = np.abs(0.5 * (vg[:, 0] - vg[:, 1]) - 0.5 * (vr[:, 0] - vr[:, 1])) + np.abs(vg[:, 2] - vr[:, 2])
    res["score"] = np.abs(got["scoreValue"][:, 0].astype(np.float64) - ref["scoreValue"][:, 0]) * score_mult
    if got["scoreValue"].shape[1] > 2:
        res["lead"] = np.abs(got["scoreValue"][:, 2].astype(np.float64) - ref["scoreValue"][:, 2]) * score_mult
    kl, pmax = np.zeros(n), np.zeros(n)
    for i in range(n):
        legal = mask[i] > 0.5
        lg = np.concatenate([got["policy"][i, legal, 0], got["policyPass"][i, :1]]).astype(np.float64)
        lr = np.concatenate([ref["policy"][i, legal, 0], ref["policyPass"][i, :1]]).astype(np.float64)
        pg, pr = _softmax(lg), _softmax(lr)
        kl[i] = float(np.sum(pr * (np.log(pr + 1e-30) - np.log(pg + 1e-30))))
        pmax[i] = float(np.abs(pg - pr).max())
    res["policy_kl"], res["policy_max"] = kl, pmax
    if "ownership" in got and "ownership" in ref:
        og, orf = np.tanh(got["ownership"].astype(np.float64)), np.tanh(ref["ownership"].astype(np.float64))
        res["ownership"] = (np.abs(og - orf) * (mask > 0.5)).max(axis=1)
    return res


def round_storage(a, dtype):
    """fp32 array rounded to the nearest value of `dtype` ("fp16" or "bf16", ties to even), returned as fp32."""
    a = np.ascontiguousarray(a, np.float32)
    if dtype == "fp16":
        return a.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        u = a.view(np.uint32).astype(np.uint64)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        return u.view(np.float32).reshape(a.shape)
    raise ValueError(dtype)


def device_weights(tree, dtype):
    """The model as the CUDA path holds it in reduced precision: the weights of every convolution that runs on the matrix
    units rounded to `dtype`; the last 1x1 convolutions of the heads (policy p2, ownership), all norms, per-board
    matmuls and biases stay fp32 on the device."""
    import copy
    t = copy.deepcopy(tree)

    def walk(x, key=None):
        if isinstance(x, dict):
            if "kY" in x and isinstance(x.get("w"), np.ndarray) and key not in ("p2Conv", "ownConv"):
                x["w"] = round_storage(x["w"], dtype)
            for k, v in x.items():
                walk(v, k)
        elif isinstance(x, list):
            for v in x:
                walk(v)
    walk(t)
    return t

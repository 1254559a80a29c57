"""Generates the committed golden vectors: outputs of the CPU oracle (oracle/kata_oracle.cpp, pinned to the
reference by oracle/_ref/katago_oracle runnnlayertests / runtinynntests) on seeded synthetic networks and
positions.  Only the outputs are stored; networks and inputs are regenerated from their seeds.

    python tests/golden/make_golden.py            # the small whole-net cases
    python tests/golden/make_golden.py full       # the full-depth reduced-precision cases (several minutes)

Full-depth cases (FULL_CASES) store, per net: `ref` = the fp32 oracle; and per storage type T in {fp16, bf16}:
`floorw_T` = the fp32 oracle run on convolution weights rounded to T (what ANY backend that keeps its weights in T
computes at best), `floorwa_T` = the same with every convolution input rounded to T as well (both operands of the
matrix units in T, everything else exact), `emu_T` = the oracle emulating the storage scheme of the CUDA path
(weights, convolution inputs and residual streams in T, fp32 arithmetic; oracle/kata_oracle.h
ko_set_storage_emulation).  Stored per set: policy channel 0, pass logit, value, score values.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from katago_b200 import modelfile as mf  # noqa: E402
from oracle import pyoracle as po  # noqa: E402

CASES = {
    # name: (model factory, n, board sizes, position seed)
    "b6c96": (lambda: mf.make_b6c96(seed=1000), 8, [19, 19, 13, 9, 19, 13, 9, 19], 2000),
    "b18c384nbt_3blocks": (lambda: mf.make_b18c384nbt(seed=1001, num_blocks=3), 6, [19, 13, 9, 19, 19, 13], 2001),
    "b28c512nbt_3blocks": (lambda: mf.make_b28c512nbt(seed=1002, num_blocks=3), 4, [19, 9, 13, 19], 2002),
    "transformer_rope_2layers": (lambda: mf.make_transformer(seed=1003, layers=2), 4, [19, 13, 9, 19], 2003),
    "transformer_relbias_2layers": (lambda: mf.make_transformer_relbias(seed=1004, layers=2), 4, [19, 9, 13, 19], 2004),
}


FULL_CASES = {
    # name: (model factory, n, board sizes, position seed, symmetry multiplier)
    "b18c384nbt_full": (lambda: mf.make_b18c384nbt(), 64, [9, 13, 19, 19] * 16, 2004, 3),
    "b28c512nbt_full": (lambda: mf.make_b28c512nbt(), 32, [9, 13, 19, 19] * 8, 2004, 5),
}
KEEP = ("policy", "policyPass", "value", "scoreValue")


def full_case_inputs(name):
    factory, n, sizes, seed, mult = FULL_CASES[name]
    sp, gl = mf.random_positions(n, seed=seed, board_sizes=sizes)
    syms = (np.arange(n) * mult % 8).astype(np.int32)
    return factory(), sp, gl, syms


def main_full():
    from tests.helpers import device_weights, symmetrise_inputs, unsymmetrise_outputs
    L = po.lib()
    for name in FULL_CASES:
        tree, sp, gl, syms = full_case_inputs(name)
        sym_in = symmetrise_inputs(sp, syms)

        def run(t, storage, flags):
            L.ko_set_storage_emulation(storage, flags)
            try:
                out = unsymmetrise_outputs(po.OracleModel(mf.to_blob(t)).forward(sym_in, gl), syms)
            finally:
                L.ko_set_storage_emulation(0, 0)
            out["policy"] = out["policy"][:, :, :1]
            out["policyPass"] = out["policyPass"][:, :1]
            return {k: out[k].astype(np.float32) for k in KEEP}
        sets = {"ref": run(tree, 0, 0)}
        for code, dt in ((1, "fp16"), (2, "bf16")):
            dev = device_weights(tree, dt)
            sets["floorw_" + dt] = run(dev, 0, 0)
            sets["floorwa_" + dt] = run(dev, code, 1)
            sets["emu_" + dt] = run(dev, code, 3)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **{f"{s}.{k}": v for s, d in sets.items() for k, v in d.items()})
        print(name, sorted(sets), os.path.getsize(path), "bytes")


def load_full(name):
    """{set name: {output name: array}} of a full-depth fixture."""
    z = np.load(os.path.join(HERE, f"{name}.npz"))
    out = {}
    for key in z.files:
        s, k = key.split(".")
        out.setdefault(s, {})[k] = z[key]
    return out


def main():
    for name, (factory, n, sizes, seed) in CASES.items():
        model = factory()
        om = po.OracleModel(mf.to_blob(model))
        sp, gl = mf.random_positions(n, seed=seed, board_sizes=sizes)
        out = om.forward(sp, gl)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **{k: v.astype(np.float32) for k, v in out.items()})
        print(name, {k: v.shape for k, v in out.items()}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "full":
        main_full()
    else:
        main()

"""Generates the committed golden vectors: outputs of the CPU oracle (oracle/kata_oracle.cpp, pinned to the
reference by oracle/_ref/katago_oracle runnnlayertests / runtinynntests) on seeded synthetic networks and
positions.  Only the outputs are stored; networks and inputs are regenerated from their seeds.

    python tests/golden/make_golden.py
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
    main()

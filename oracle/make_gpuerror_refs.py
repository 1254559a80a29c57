"""Writes the reference-value files for the reference's cross-backend harness `testgpuerror`
(cpp/command/gputest.cpp, cpp/tests/testnnevalcanary.cpp:517-761).  TEST INFRASTRUCTURE ONLY.

For each case it runs oracle/_ref/katago_oracle (the reference's program linked with the CPU oracle, built like the
reference builds its Eigen backend) with `-reference-file`, exactly as cpp/rungpuerrortest.sh does for the Eigen
build.  Models are either generated from seeds (katago_b200.modelfile) or the trained test nets that ship with the
reference (copied next to the reference files so that they travel to the GPU box).  Everything goes to
oracle/_ref/gpuerror/, which is not committed.

    python oracle/make_gpuerror_refs.py [--reference <directory of the reference checkout>]
"""
import argparse
import json
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)

OUT = os.path.join(HERE, "_ref", "gpuerror")
CFG = """logFile = /dev/null
logToStderr = false
numSearchThreads = 8
nnMaxBatchSize = 16
nnCacheSizePowerOfTwo = 10
nnMutexPoolSizePowerOfTwo = 10
numNNServerThreadsPerModel = 1
"""

# name, model ("gen:<factory>" or file under cpp/tests/models), board size dataset, config overrides
CASES = [
    ("b6c96_random_19", "gen:b6c96", "19", "requireMaxBoardSize=False"),
    ("b18x4_random_19", "gen:b18x4", "19", "requireMaxBoardSize=True, maxBatchSize=16"),
    ("b18x4_random_rect", "gen:b18x4", "rectangle", "requireMaxBoardSize=False, maxBatchSize=7"),
    ("g170_b6c96_13", "g170-b6c96-s175395328-d26788732.bin.gz", "13", "requireMaxBoardSize=False"),
    ("g170e_b10c128_19", "g170e-b10c128-s1141046784-d204142634.bin.gz", "19", "requireMaxBoardSize=True, maxBatchSize=19"),
    ("b7c96h3tfrs_13", "b7c96h3tfrs-test5-cnorm.bin.gz", "13", "requireMaxBoardSize=False, maxBatchSize=5"),
    ("b4c256h4nbttflrs_rect", "b4c256h4nbttflrs-fson-silu-rsnh.bin.gz", "rectangle", "requireMaxBoardSize=False, maxBatchSize=6"),
    ("b7c96h6kv3_9", "b7c96h6kv3qk32v16tflrs-fson-bnh.bin.gz", "9", "requireMaxBoardSize=True, maxBatchSize=12"),
    # attention with a learned relative-position bias instead of RoPE: model file + extension file (<model>.kbext,
    # katago_b200/host/model_ext.h), which both backends pick up when they load the model
    ("tf2_relbias_random_19", "gen:tf2relbias", "19", "requireMaxBoardSize=False, maxBatchSize=9"),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("KATAGO_REFERENCE", "/root/reference"))
    args = ap.parse_args()
    from katago_b200 import modelfile as mf
    katago = os.path.join(HERE, "_ref", "katago_oracle")
    if not os.path.exists(katago):
        raise SystemExit("oracle/_ref/katago_oracle is missing: run `make -C oracle ref` first")
    os.makedirs(OUT, exist_ok=True)
    with open(os.path.join(OUT, "gpuerror.cfg"), "w") as f:
        f.write(CFG)
    gen = {"b6c96": lambda: mf.make_b6c96(), "b18x4": lambda: mf.make_b18c384nbt(num_blocks=4),
           "tf2relbias": lambda: mf.make_transformer_relbias(layers=2)}
    index = []
    for name, model, size, overrides in CASES:
        if model.startswith("gen:"):
            model_file = os.path.join(OUT, model[4:] + "-random.bin.gz")
            if not os.path.exists(model_file):
                mf.save_model_file(gen[model[4:]](), model_file)
        else:
            src = os.path.join(args.reference, "cpp", "tests", "models", model)
            model_file = os.path.join(OUT, model)
            if not os.path.exists(model_file):
                shutil.copyfile(src, model_file)
        ref_file = os.path.join(OUT, name + ".json")
        if not os.path.exists(ref_file):
            cmd = [katago, "testgpuerror", "-model", model_file, "-config", os.path.join(OUT, "gpuerror.cfg"), "-boardsize", size, "-quick",
                   "-reference-file", ref_file, "-override-config", overrides]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0 or not os.path.exists(ref_file):
                raise SystemExit(f"{name}: katago_oracle testgpuerror failed\n{(r.stdout + r.stderr)[-2000:]}")
        index.append(dict(name=name, model=os.path.basename(model_file), boardsize=size, overrides=overrides, reference=name + ".json"))
        print(name, os.path.getsize(ref_file) >> 10, "KiB")
    with open(os.path.join(OUT, "index.json"), "w") as f:
        json.dump(index, f, indent=1)


if __name__ == "__main__":
    main()

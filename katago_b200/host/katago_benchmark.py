"""Runs the reference program's own `benchmark` subcommand (search threads -> NNEvaluator -> getOutput) on the B200
backend with a random-weight b18c384nbt model file, and prints its nnEvals/s lines.

    python katago_b200/host/katago_benchmark.py [--binary oracle/_ref/katago_b200] [--visits 30000] [--threads 512,1024]

The binary is the reference's sources compiled with katago_b200/host/b200backend.cpp as the backend (oracle/Makefile,
target ref_b200).  This number goes through MCTS, the NN cache and the batching queue, so it is a secondary figure next
to bench.py's device-timed and host-buffer figures.
"""
import argparse
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from katago_b200 import modelfile as mf  # noqa: E402

CFG = """logFile = /dev/null
logToStderr = false
logAllGTPCommunication = false
logSearchInfo = false
rules = tromp-taylor
numSearchThreads = 256
nnMaxBatchSize = 256
nnCacheSizePowerOfTwo = 20
nnMutexPoolSizePowerOfTwo = 14
numNNServerThreadsPerModel = 2
cudaUseFP16 = true
maxVisits = {visits}
"""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--binary", default=os.path.join(ROOT, "oracle", "_ref", "katago_b200"))
    ap.add_argument("--visits", type=int, default=30000)
    ap.add_argument("--threads", default="512,1024")
    ap.add_argument("--positions", type=int, default=4)
    args = ap.parse_args()
    if not os.path.exists(args.binary):
        sys.exit(f"{args.binary} not found: build it with `make -C oracle ref_b200` where the reference sources are available")
    with tempfile.TemporaryDirectory() as d:
        model = os.path.join(d, "b18c384nbt-random.bin.gz")
        cfg = os.path.join(d, "benchmark.cfg")
        mf.save_model_file(mf.make_b18c384nbt(), model)
        with open(cfg, "w") as f:
            f.write(CFG.format(visits=args.visits))
        env = dict(os.environ)
        env["LD_LIBRARY_PATH"] = os.path.join(ROOT, "katago_b200") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
        cmd = [args.binary, "benchmark", "-model", model, "-config", cfg, "-v", str(args.visits), "-t", args.threads, "-n", str(args.positions)]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=1200)
        for line in (r.stdout + r.stderr).replace("\r", "\n").splitlines():
            if "nnEvals/s" in line or "finishing" in line or "rror" in line:
                print(line.strip())
        sys.exit(r.returncode)


if __name__ == "__main__":
    main()

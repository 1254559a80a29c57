"""Multi-process plumbing of bench.py on CPU (gloo, world_size 2): the control plane is torch.distributed with the
gloo backend (barrier + max over ranks); there is no data-path collective because GPUs run independent replicas."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(extra, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "bench.py")] + extra
    env = dict(os.environ, OMP_NUM_THREADS="1")  # what torchrun itself exports to its workers
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)


def test_reference_arm_under_torchrun_prints_one_line_from_rank0():
    r = _torchrun(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"], 29631)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["unit"] == "evals/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["e2e"]["h2d_bytes_per_step"] == 0
    # the CPU arm uses every core it may run on, also under torchrun (which starts its workers with one OpenMP thread)
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))


def test_max_over_ranks_and_barrier_with_gloo(tmp_path):
    code = (
        "import os, sys; sys.path.insert(0, %r)\n"
        "import bench\n"
        "rank, world, local, pg = bench._dist()\n"
        "bench._barrier_sync(pg)\n"
        "m = bench._max_over_ranks(pg, float(rank + 1))\n"
        "assert world == 2 and m == 2.0, (world, m)\n"
        "pg.barrier(); pg.destroy_process_group()\n"
        "print('rank', rank, 'ok')\n" % ROOT)
    path = str(tmp_path / "rank_test.py")
    with open(path, "w") as f:
        f.write(code)
    if True:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
               "--master-port", "29633", path]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
        assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
        assert r.stdout.count("ok") == 2

"""Helpers that run a worker script as N ranks under torchrun and collect its JSON result."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_workers(script: str, world: int, args=(), timeout: int = 600, env=None, expect_rc: int = 0):
    """Launch tests/workers/<script> on `world` ranks. Rank 0 prints one line `RESULT {json}`;
    returns the decoded object. Raises with the output tail when a rank fails."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "workers", script), *map(str, args)]
    full_env = dict(os.environ)
    full_env.setdefault("OMP_NUM_THREADS", "2")
    full_env["PYTHONPATH"] = ROOT + os.pathsep + full_env.get("PYTHONPATH", "")
    if env:
        full_env.update(env)
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=full_env, cwd=ROOT)
    out = proc.stdout + "\n" + proc.stderr
    log_dir = os.environ.get("TDIST_TEST_LOG_DIR")
    if log_dir:
        os.makedirs(log_dir, exist_ok=True)
        with open(os.path.join(log_dir, f"{os.path.splitext(script)[0]}_w{world}.log"), "w") as f:
            f.write(out)
    if proc.returncode != expect_rc:
        raise AssertionError(f"{script} exited {proc.returncode} (expected {expect_rc}):\n{out[-6000:]}")
    result = None
    for line in proc.stdout.splitlines():
        if line.startswith("RESULT "):
            result = json.loads(line[len("RESULT "):])
    return result, out

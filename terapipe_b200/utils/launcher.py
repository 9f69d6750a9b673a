"""Local process launcher: one process per GPU (or per CPU rank) on this machine.

Replaces the reference's ``mpirun --map-by ppr:N:node python script.py ... --use-mpi``
(mpirun_terapipe.sh:27-39).  Children get both torchrun-style (RANK, LOCAL_RANK, WORLD_SIZE,
MASTER_ADDR, MASTER_PORT) and OpenMPI-style (OMPI_COMM_WORLD_*) environment variables, so
drivers started with ``--use-mpi`` find their ranks.  If any child exits non-zero or the
optional time limit runs out, every child of THIS launcher is terminated by PID (never by
name pattern) and the launcher returns a non-zero status.

    python -m terapipe_b200.utils.launcher --nproc 8 [--timeout 500] script.py args...
"""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time
from typing import List, Optional


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(cmd: List[str], nproc: int, timeout: Optional[float] = None, port: Optional[int] = None,
           env_extra: Optional[dict] = None, poll_s: float = 0.2) -> int:
    port = port or _free_port()
    procs = []
    for rank in range(nproc):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(nproc),
                    "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                    "OMPI_COMM_WORLD_SIZE": str(nproc), "OMPI_COMM_WORLD_RANK": str(rank),
                    "OMPI_COMM_WORLD_LOCAL_RANK": str(rank)})
        env.update(env_extra or {})
        procs.append(subprocess.Popen(cmd, env=env, start_new_session=True))
    deadline = time.time() + timeout if timeout else None
    status = 0
    try:
        while True:
            codes = [p.poll() for p in procs]
            if any(c not in (None, 0) for c in codes):
                status = next(c for c in codes if c not in (None, 0))
                break
            if all(c == 0 for c in codes):
                break
            if deadline and time.time() > deadline:
                status = 124
                break
            time.sleep(poll_s)
    finally:
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        t_end = time.time() + 5
        for p in procs:
            try:
                p.wait(timeout=max(0.1, t_end - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
    return status


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--timeout", type=float, default=None)
    ap.add_argument("--port", type=int, default=None)
    ap.add_argument("script")
    ap.add_argument("args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    return launch([sys.executable, a.script, *a.args], a.nproc, a.timeout, a.port)


if __name__ == "__main__":
    sys.exit(main())

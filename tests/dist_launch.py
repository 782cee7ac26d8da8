r"""Launches N worker processes (one per rank) of a distributed test and collects exit codes.

The reference's tests spawn ranks with ``subprocess.Popen`` and OpenMPI-style environment
variables (``tests/test_ddp.py:30-69``); here the children get the torchrun variables and the
rendezvous address is always 127.0.0.1.
"""
import os
import socket
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(script, case, world_size, timeout=300, extra_env=None, stop_on_failure=True,
              args=None):
    r"""Returns the list of exit codes; children are killed (by pid) when `timeout` expires, and
    — unless `stop_on_failure` is off — a few seconds after the first rank has failed.
    `script` is relative to this directory (or absolute); `args` replaces `[case]` as the
    script's command line."""
    port = free_port()
    procs = []
    for rank in range(world_size):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world_size),
                    "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
        if extra_env:
            env.update(extra_env)
        cmd = [sys.executable, os.path.join(HERE, script)] + (list(args) if args is not None else [case])
        procs.append(subprocess.Popen(cmd, env=env))
    # Poll all ranks: when one fails, the others would wait for it in their next collective
    # until `timeout`, so they are stopped (by pid) right away and reported as -9.
    deadline = time.monotonic() + timeout
    codes = [None] * world_size
    while any(c is None for c in codes):
        for i, p in enumerate(procs):
            if codes[i] is None:
                rc = p.poll()
                if rc is not None:
                    codes[i] = rc
        failed = stop_on_failure and any(c not in (None, 0) for c in codes)
        if failed or time.monotonic() > deadline:
            grace = time.monotonic() + (3.0 if failed else 0.0)
            while time.monotonic() < grace and any(p.poll() is None for p in procs):
                time.sleep(0.1)
            for i, p in enumerate(procs):
                if codes[i] is None:
                    rc = p.poll()
                    if rc is None:
                        p.kill()
                        p.wait()
                        rc = -9
                    codes[i] = rc
            break
        time.sleep(0.05)
    return codes

r"""Launches N worker processes (one per rank) of a distributed test and collects exit codes.

The reference's tests spawn ranks with ``subprocess.Popen`` and OpenMPI-style environment
variables (``tests/test_ddp.py:30-69``); here the children get the torchrun variables and the
rendezvous address is always 127.0.0.1.
"""
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(script, case, world_size, timeout=300, extra_env=None):
    r"""Returns the list of exit codes; children are killed (by pid) when `timeout` expires."""
    port = free_port()
    procs = []
    for rank in range(world_size):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world_size),
                    "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
        if extra_env:
            env.update(extra_env)
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, script), case], env=env))
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=timeout))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    return codes

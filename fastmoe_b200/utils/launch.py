r"""
Environment mapping for cluster launchers.

The reference ships ``tests/test.sh``, which translates SLURM / OpenMPI variables into
``RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT`` and pins one GPU per local rank.
``setup_env()`` does the same from Python (call it before ``init_process_group``); GPUs are not
hidden from the process — the peer-to-peer path needs to see its peers — the local rank is
returned instead so that the caller can ``torch.cuda.set_device`` it.
"""
import os


def setup_env(default_port=29500):
    env = os.environ
    if "RANK" not in env:
        if "OMPI_COMM_WORLD_RANK" in env:
            env["RANK"] = env["OMPI_COMM_WORLD_RANK"]
            env["WORLD_SIZE"] = env["OMPI_COMM_WORLD_SIZE"]
            env.setdefault("LOCAL_RANK", env.get("OMPI_COMM_WORLD_LOCAL_RANK", "0"))
        elif "SLURM_PROCID" in env:
            env["RANK"] = env["SLURM_PROCID"]
            env["WORLD_SIZE"] = env.get("SLURM_NPROCS", env.get("SLURM_NTASKS", "1"))
            env.setdefault("LOCAL_RANK", env.get("SLURM_LOCALID", "0"))
        else:
            env["RANK"], env["WORLD_SIZE"] = "0", "1"
    env.setdefault("LOCAL_RANK", "0")
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env.setdefault("MASTER_PORT", str(default_port))
    return int(env["RANK"]), int(env["WORLD_SIZE"]), int(env["LOCAL_RANK"])

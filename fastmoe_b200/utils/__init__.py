r"""Helpers: pytree mapping, process-group lookup (``fmoe/utils.py``), timers and logging."""
from ..parallel.comm import get_rank_0_in_comm, get_torch_default_comm  # noqa: F401

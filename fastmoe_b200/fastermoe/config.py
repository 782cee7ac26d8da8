r"""Environment helpers under their reference names (``fmoe/fastermoe/config.py:4-13``)."""
from ..config import float_from_env, switch_from_env  # noqa: F401

r"""FasterMoE features: the smart (pipelined) schedule and shadow experts.

Parity: ``fmoe/fastermoe/`` (``config.py``, ``expert_utils.py``, ``schedule.py``,
``shadow_policy.py``) and the native scheduler ``cuda/fastermoe/smart_schedule.{h,cpp}``.
"""

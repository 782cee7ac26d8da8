r"""
The interface every routing policy implements.

A gate maps token features ``[B, d_model]`` to ``(expert ids [B, k], scores [B, k])`` over
``tot_expert = num_expert * world_size`` experts (``num_expert`` per rank) and may leave one
scalar auxiliary loss behind for the training loop to pick up.  Parity:
``fmoe/gates/base_gate.py:7-29`` (same constructor, ``set_loss`` / ``get_loss(clear)`` /
``has_loss`` protocol, ``loss`` attribute).
"""
import torch.nn as nn


class BaseGate(nn.Module):
    r"""Holds the expert geometry and the auxiliary loss of the latest forward.

    The loss slot is single-entry: a forward overwrites what the previous one left, and
    ``get_loss()`` empties it unless called with ``clear=False`` (used by code that only wants
    to look, e.g. logging).
    """

    def __init__(self, num_expert, world_size):
        super().__init__()
        self.num_expert, self.world_size = num_expert, world_size
        self.tot_expert = num_expert * world_size
        self._aux_loss = None

    # ``gate.loss`` stays readable and writable like a plain attribute.
    @property
    def loss(self):
        return self._aux_loss

    @loss.setter
    def loss(self, value):
        self._aux_loss = value

    @property
    def has_loss(self):
        return self._aux_loss is not None

    def set_loss(self, loss):
        self._aux_loss = loss

    def get_loss(self, clear=True):
        value = self._aux_loss
        if clear:
            self._aux_loss = None
        return value

    def forward(self, x):
        raise NotImplementedError("%s does not implement a routing policy" % type(self).__name__)

    def extra_repr(self):
        return "num_expert=%d, world_size=%d" % (self.num_expert, self.world_size)

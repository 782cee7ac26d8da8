r"""Common interface of all gates (parity: ``fmoe/gates/base_gate.py:7-29``)."""
import torch.nn as nn


class BaseGate(nn.Module):
    r"""Stores the expert geometry and the most recent balance loss."""

    def __init__(self, num_expert, world_size):
        super().__init__()
        self.world_size = world_size
        self.num_expert = num_expert
        self.tot_expert = world_size * num_expert
        self.loss = None

    def forward(self, x):
        raise NotImplementedError("BaseGate is an interface; use a concrete gate")

    def set_loss(self, loss):
        self.loss = loss

    def get_loss(self, clear=True):
        loss = self.loss
        if clear:
            self.loss = None
        return loss

    @property
    def has_loss(self):
        return self.loss is not None

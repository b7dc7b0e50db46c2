"""ReLU and JumpReLU nonlinearities (reference: crosslayer_transcoder/model/jumprelu.py:17-73).

In the training step both run fused into the encoder contraction's epilogue
(forward) and into the feature-gradient contraction's epilogue (backward); the
autograd function below is the eager definition for direct calls.
"""
from __future__ import annotations

import torch
from torch import nn

from .serializable_module import SerializableModule


class ReLU(SerializableModule):
    def forward(self, input, layer=None):
        return torch.relu(input)


class _JumpReLUEager(torch.autograd.Function):
    """f = x [x > theta, x > 0];  dx = g [x >= 0];
    dtheta = -(theta / bw) rect((x - theta) / bw) g with rect = 1 on (-1/2, 1/2]."""

    @staticmethod
    def forward(ctx, x, theta, bandwidth):
        ctx.save_for_backward(x, theta)
        ctx.bandwidth = bandwidth
        return x * ((x > theta) & (x > 0))

    @staticmethod
    def backward(ctx, g):
        x, theta = ctx.saved_tensors
        bw = ctx.bandwidth
        u = (x - theta) / bw
        rect = ((u > -0.5) & ~(u > 0.5)).to(g.dtype)
        return g.masked_fill(x < 0, 0), -(theta / bw) * rect * g, None


class JumpReLU(SerializableModule):
    def __init__(self, theta=0.0, bandwidth=1.0, n_layers=12, d_features=768 * 8):
        super().__init__()
        self.theta = nn.Parameter(torch.full((1, n_layers, d_features), float(theta)))
        self.register_buffer("bandwidth", torch.tensor(float(bandwidth)))
        self._init_theta, self.n_layers, self.d_features = theta, n_layers, d_features

    def forward(self, input):
        return _JumpReLUEager.apply(input, self.theta, self.bandwidth)

    def _init_args(self):
        return {"theta": self._init_theta, "bandwidth": self.bandwidth.item(), "n_layers": self.n_layers,
                "d_features": self.d_features}

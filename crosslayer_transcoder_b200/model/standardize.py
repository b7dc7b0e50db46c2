"""Activation standardizers (reference: crosslayer_transcoder/model/standardize.py:12-117).

The training step applies them inside the CUDA input-preparation and loss kernels;
the ``forward`` / ``standardize`` methods here are the eager definitions used for
inference-time calls and for folding.
"""
from __future__ import annotations

import torch

from .serializable_module import SerializableModule


class Standardizer(SerializableModule):
    """Identity standardizer (reference standardize.py:12-27)."""

    def __init__(self, **kwargs):
        super().__init__()

    def initialize_from_batch(self, batch):
        pass

    def forward(self, batch, layer="all"):
        return batch

    def standardize(self, batch, layer="all"):
        return batch


class _Dimensionwise(Standardizer):
    _config_fields = ("n_layers", "activation_dim")
    _io_index = 0

    def __init__(self, n_layers, activation_dim):
        super().__init__()
        self.n_layers, self.activation_dim = n_layers, activation_dim
        self.register_buffer("mean", torch.empty(n_layers, activation_dim))
        self.register_buffer("std", torch.empty(n_layers, activation_dim))
        self.is_initialized = False

    @torch.no_grad()
    def initialize_from_batch(self, batch):
        """Per (layer, dimension) mean and unbiased std over the batch, std floored at 1e-8
        (reference standardize.py:39-47, 80-86).  ``batch`` is ``[B, 2, L, D]``."""
        side = batch[:, self._io_index]
        self.mean.data = side.mean(dim=0)
        self.std.data = side.std(dim=0).clamp_(min=1e-8)
        self.is_initialized = True

    def _sel(self, layer):
        if layer == "all":
            return self.mean, self.std
        return self.mean[layer], self.std[layer]


class DimensionwiseInputStandardizer(_Dimensionwise):
    _io_index = 0

    def forward(self, batch, layer="all"):
        if not self.is_initialized:
            raise ValueError("Standardizer not initialized")
        mu, sd = self._sel(layer)
        return (batch - mu) / sd


class DimensionwiseOutputStandardizer(_Dimensionwise):
    _io_index = 1

    def forward(self, batch, layer="all"):
        """De-standardise a normalised reconstruction (reference standardize.py:88-98)."""
        if not self.is_initialized:
            raise ValueError("Standardizer not initialized")
        mu, sd = self._sel(layer)
        return batch * sd + mu

    def standardize(self, mlp_out, layer="all"):
        mu, sd = self._sel(layer)
        return (mlp_out - mu) / sd

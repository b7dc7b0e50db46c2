"""TopK feature selections (reference: crosslayer_transcoder/model/topk.py:11-133).

The training step selects with the CUDA selection kernels and never materialises the
dense ``[B, L, F]`` result; the methods here are the eager definitions for direct
calls (inference, the auxiliary module handed to the TopK training module).
"""
from __future__ import annotations

import torch

from .serializable_module import SerializableModule


def _keep_top(flat: torch.Tensor, n: int):
    """Zero everything but the n largest entries along the last axis; kept values are relu'd."""
    out = torch.zeros_like(flat)
    if n == 0:
        return out, None
    vals, idx = torch.topk(flat, n, dim=-1, sorted=False)
    vals = torch.relu(vals)
    out.scatter_(-1, idx, vals)
    return out, vals


class TopK(SerializableModule):
    _config_fields = ("k", "e", "n_layers")

    def __init__(self, k: int, e=None, n_layers=None, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.k, self.e, self.n_layers = k, e, n_layers

    def forward(self, features, layer="all"):
        if layer == "all":
            return self._training_forward(features)
        return self._inference_forward(features, layer)


class PerLayerTopK(TopK):
    """k largest per (token, layer) (reference topk.py:48-63)."""

    def _training_forward(self, features):
        assert self.k <= features.shape[-1]
        return _keep_top(features, self.k)[0]

    @torch.no_grad()
    def _inference_forward(self, features, layer):
        return self._training_forward(features)


class BatchTopK(TopK):
    """k B L largest of the whole batch, all layers together, with an EMA of the smallest
    kept value as the inference threshold (reference topk.py:66-96)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("threshold", torch.zeros(1))

    def _training_forward(self, features):
        B, L, F = features.shape
        assert self.k <= F
        out, vals = _keep_top(features.flatten(), self.k * B * L)
        if vals is not None:
            self.threshold = (1 - self.e) * self.threshold + self.e * vals.min().detach()
        return out.reshape(B, L, F)

    @torch.no_grad()
    def _inference_forward(self, features, layer):
        thr = max(0, self.threshold.item())
        return torch.where(features > thr, features, torch.zeros_like(features))


class PerLayerBatchTopK(TopK):
    """k B largest per layer over the batch, one EMA threshold per layer (reference topk.py:99-133)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("threshold", torch.zeros(self.n_layers))

    def _training_forward(self, features):
        B, L, F = features.shape
        assert self.k <= F
        per_layer = features.transpose(0, 1).reshape(L, B * F)
        out, vals = _keep_top(per_layer, self.k * B)
        if vals is not None:
            self.threshold = (1 - self.e) * self.threshold + self.e * vals.detach().min(dim=-1).values
        return out.reshape(L, B, F).transpose(0, 1).contiguous()

    @torch.no_grad()
    def _inference_forward(self, features, layer):
        thr = max(0, self.threshold[layer].item())
        return torch.where(features > thr, features, torch.zeros_like(features))

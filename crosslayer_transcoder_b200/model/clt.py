"""Encoder, decoders and the transcoder container with the reference's constructor
arguments, parameter names and shapes (crosslayer_transcoder/model/clt.py:115-467):

    encoder.W [L, D, F]   encoder.b [L, F]
    decoder.W_t [(t+1), F, D] for t = 0..L-1 (crosslayer)   or   decoder.W [L, F, D] (per-layer)
    decoder.b [L, D]

The training step does not call these ``forward`` methods: it runs the fused CUDA
path of ``crosslayer_transcoder_b200.engine`` on the same parameters.  The per-layer
``forward_layer`` calls run on the same kernels when the stack belongs to a training
module and the input is on the GPU; otherwise, and for folding and export, the eager
definitions below apply.
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Union

import torch
import yaml
from torch import nn

from .serializable_module import SerializableModule
from .standardize import Standardizer


class _Layered(SerializableModule):
    _config_fields = ("d_acts", "d_features", "n_layers")

    def __init__(self, d_acts: int, d_features: int, n_layers: int):
        super().__init__()
        self.d_acts, self.d_features, self.n_layers = d_acts, d_features, n_layers
        self._is_folded = False

    def _engine(self):
        """The fused-step engine of the training module that owns this layer stack (set by
        ``CrossLayerTranscoderModule``), or None: with it the per-layer forwards run on the CUDA kernels."""
        return self.__dict__.get("_kernel_engine")

    def __getstate__(self):
        state = dict(self.__dict__)
        state.pop("_kernel_engine", None)      # device buffers and events of the engine are not part of the module
        return state


class Encoder(_Layered):
    def __init__(self, d_acts: int, d_features: int, n_layers: int):
        super().__init__(d_acts, d_features, n_layers)
        self.bias = True
        self.W = nn.Parameter(torch.empty(n_layers, d_acts, d_features))
        self.b = nn.Parameter(torch.empty(n_layers, d_features))
        self.reset_parameters()

    def reset_parameters(self):
        bound = self.d_features ** -0.5          # reference clt.py:129-130
        with torch.no_grad():
            self.W.uniform_(-bound, bound)
            self.b.zero_()

    @torch.no_grad()
    def forward_layer(self, acts_norm, layer: int):
        eng = self._engine()
        if eng is not None and acts_norm.is_cuda:
            return eng.encode_layer(acts_norm, layer)
        return acts_norm @ self.W[layer] + self.b[layer]

    def forward(self, acts_norm, layer="all"):
        if layer != "all":
            return self.forward_layer(acts_norm, layer)
        pre = torch.einsum("bld,ldf->blf", acts_norm, self.W).contiguous()
        return pre + self.b.to(acts_norm.dtype)

    def fold(self, input_standardizer: Standardizer):
        """Absorb (x - mean) / std into the weights: W /= std, b -= mean @ W (reference clt.py:169-187)."""
        if not self._is_folded:
            self.W.data = self.W / input_standardizer.std.unsqueeze(-1)
            self.b.data = self.b - torch.einsum("ld,ldf->lf", input_standardizer.mean, self.W)
            self._is_folded = True
        return self


class Decoder(_Layered):
    """Per-layer decoder: layer l's features write only to layer l's output."""

    crosslayer = False

    def __init__(self, d_acts: int, d_features: int, n_layers: int):
        super().__init__(d_acts, d_features, n_layers)
        self.W = nn.Parameter(torch.empty(n_layers, d_features, d_acts))
        self.b = nn.Parameter(torch.empty(n_layers, d_acts))
        self.reset_parameters()

    def reset_parameters(self):
        bound = (self.d_acts * self.n_layers) ** -0.5   # reference clt.py:212-214
        with torch.no_grad():
            self.W.uniform_(-bound, bound)
            self.b.zero_()

    def blocks(self):
        return [self.W]

    @torch.no_grad()
    def forward_layer(self, features, layer: int):
        eng = self._engine()
        if eng is not None and features.is_cuda:
            return eng.decode_layer(features, layer)
        if features.ndim == 4:
            features = features[:, :, layer, :]
        return features @ self.W[layer] + self.b[layer]

    def forward(self, features, layer="all"):
        if layer != "all":
            return self.forward_layer(features, layer)
        return torch.einsum("blf,lfd->bld", features, self.W) + self.b

    def fold(self, output_standardizer: Standardizer):
        if not self._is_folded:
            self.W.data = self.W * output_standardizer.std.unsqueeze(1)
            self.b.data = self.b * output_standardizer.std + output_standardizer.mean
            self._is_folded = True
        return self


class CrosslayerDecoder(_Layered):
    """Features of source layer s write to every target layer t >= s through ``W_t[s]``."""

    crosslayer = True

    def __init__(self, d_acts: int, d_features: int, n_layers: int):
        super().__init__(d_acts, d_features, n_layers)
        for t in range(n_layers):
            self.register_parameter(f"W_{t}", nn.Parameter(torch.empty(t + 1, d_features, d_acts)))
        self.register_parameter("b", nn.Parameter(torch.empty(n_layers, d_acts)))
        self.reset_parameters()

    def reset_parameters(self):
        bound = (self.d_acts * self.n_layers) ** -0.5   # reference clt.py:294-298
        with torch.no_grad():
            for w in self.blocks():
                w.uniform_(-bound, bound)
            self.b.zero_()

    def blocks(self):
        return [self.get_parameter(f"W_{t}") for t in range(self.n_layers)]

    @torch.no_grad()
    def forward_layer(self, features, layer: int):
        eng = self._engine()
        if eng is not None and features.is_cuda:
            return eng.decode_layer(features, layer)
        return torch.einsum("bqsf,sfd->bqd", features, self.get_parameter(f"W_{layer}")) + self.b[layer]

    def forward(self, features, layer="all"):
        if layer != "all":
            return self.forward_layer(features, layer)
        cols = [torch.einsum("bsf,sfd->bd", features[:, : t + 1], w).to(features.dtype)
                for t, w in enumerate(self.blocks())]
        return torch.stack(cols, dim=1) + self.b.to(features.dtype)

    def fold(self, output_standardizer: Standardizer):
        if not self._is_folded:
            self.b.data = self.b * output_standardizer.std + output_standardizer.mean
            for t, w in enumerate(self.blocks()):
                w.data = w * output_standardizer.std[t]
            self._is_folded = True
        return self


class CrossLayerTranscoder(SerializableModule):
    def __init__(self, nonlinearity: SerializableModule, encoder: Encoder,
                 decoder: Union[Decoder, CrosslayerDecoder],
                 input_standardizer: Optional[Standardizer] = None,
                 output_standardizer: Optional[Standardizer] = None):
        super().__init__()
        self.encoder, self.decoder, self.nonlinearity = encoder, decoder, nonlinearity
        self.input_standardizer, self.output_standardizer = input_standardizer, output_standardizer
        self._is_folded = False
        self.reset_parameters()

    def reset_parameters(self):
        self.encoder.reset_parameters()
        self.decoder.reset_parameters()

    def initialize_standardizers(self, batch):
        self.input_standardizer.initialize_from_batch(batch)
        self.output_standardizer.initialize_from_batch(batch)

    def forward(self, acts):
        """(pre_actvs [B,L,F], features [B,L,F], recons_norm [B,L,D], recons [B,L,D])
        (reference clt.py:403-425)."""
        if self.input_standardizer is not None:
            acts = self.input_standardizer(acts)
        pre_actvs = self.encoder(acts)
        features = self.nonlinearity(pre_actvs)
        recons_norm = self.decoder(features)
        recons = self.output_standardizer(recons_norm) if self.output_standardizer is not None else recons_norm
        return pre_actvs, features, recons_norm, recons

    def _init_args(self):
        sub = lambda m: None if m is None else m.to_config()
        return {"nonlinearity": self.nonlinearity.to_config(), "encoder": self.encoder.to_config(),
                "decoder": self.decoder.to_config(), "input_standardizer": sub(self.input_standardizer),
                "output_standardizer": sub(self.output_standardizer)}

    def fold(self):
        if self._is_folded:
            return
        if self.input_standardizer is not None:
            self.encoder.fold(self.input_standardizer)
        if self.output_standardizer is not None:
            self.decoder.fold(self.output_standardizer)
        self._is_folded = True
        self.input_standardizer = self.output_standardizer = None

    def save_pretrained(self, directory: Path, fold_standardizers: bool = True, reference_class_paths: bool = False):
        from safetensors.torch import save_file

        directory = Path(directory)
        directory.mkdir(parents=True, exist_ok=True)
        if fold_standardizers:
            self.fold()
        cfg = self.config_for_export(reference_class_paths)
        cfg["is_folded"] = self._is_folded
        (directory / "config.yaml").write_text(yaml.dump({"model": cfg}))
        save_file({k: v.contiguous() for k, v in self.state_dict().items()}, directory / "checkpoint.safetensors")

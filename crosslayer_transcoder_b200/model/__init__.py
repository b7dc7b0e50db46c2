"""Module surface of the crosslayer transcoder (same class names as the reference's
``crosslayer_transcoder.model`` package)."""
from .clt import CrossLayerTranscoder, CrosslayerDecoder, Decoder, Encoder
from .clt_lightning import (CrossLayerTranscoderModule, JumpReLUCrossLayerTranscoderModule,
                            TopKCrossLayerTranscoderModule)
from .jumprelu import JumpReLU, ReLU
from .standardize import DimensionwiseInputStandardizer, DimensionwiseOutputStandardizer, Standardizer
from .topk import BatchTopK, PerLayerBatchTopK, PerLayerTopK

__all__ = [
    "CrossLayerTranscoder", "CrosslayerDecoder", "Decoder", "Encoder", "CrossLayerTranscoderModule",
    "JumpReLUCrossLayerTranscoderModule", "TopKCrossLayerTranscoderModule", "JumpReLU", "ReLU",
    "DimensionwiseInputStandardizer", "DimensionwiseOutputStandardizer", "Standardizer", "BatchTopK",
    "PerLayerBatchTopK", "PerLayerTopK",
]

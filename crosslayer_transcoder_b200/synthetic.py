"""Seeded synthetic activations and weights with the shapes and value
distributions of the benchmark configurations.

They stand in for the GPT-2 / OpenWebText MLP activations the reference trains
on (config/default.yaml:114-118 of the reference), which cannot be downloaded
where the benchmark runs.  By default everything is drawn on the CPU from one
``torch.Generator`` so that the same tensors reach the CUDA path and the CPU
checker; the benchmark draws its (much larger) batch on the device instead.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass(frozen=True)
class WorkloadSpec:
    name: str
    n_layers: int
    d_acts: int
    d_features: int
    batch: int
    kind: str                 # jumprelu | topk | batchtopk
    crosslayer: bool
    bf16: bool
    rank_u: int = 64          # width of the shared latent u
    n_outlier: int = 4
    outlier_scale: float = 20.0
    theta: float = 0.03
    bandwidth: float = 1.0
    lambda_sparsity: float = 0.0
    c_sparsity: float = 1.0
    use_tanh: bool = True
    pre_actv_loss: float = 0.0
    k: int = 0
    k_aux: int = 0
    aux_loss_scale: float = 0.0
    tokens_till_dead: int = 1_000_000
    dead_fraction: float = 0.0
    e: float = 0.01
    lr: float = 1e-4


WORKLOADS: Dict[str, WorkloadSpec] = {
    # configs[0]: tiny crosslayer transcoder, fp32, JumpReLU + tanh sparsity
    "c1_tiny_clt_fp32": WorkloadSpec("c1_tiny_clt_fp32", 12, 768, 1024, 512, "jumprelu", True, False,
                                     lambda_sparsity=4e-4),
    # configs[1]: per-layer transcoder, bf16, JumpReLU + pre-activation loss
    "c2_plt_bf16": WorkloadSpec("c2_plt_bf16", 12, 768, 24576, 4000, "jumprelu", False, True,
                                pre_actv_loss=3e-6),
    # configs[2]: crosslayer transcoder, bf16, TopK k=32 with the dead-feature auxiliary loss
    "c3_clt_topk_bf16": WorkloadSpec("c3_clt_topk_bf16", 12, 768, 32768, 4000, "topk", True, True,
                                     k=32, k_aux=512, aux_loss_scale=1 / 32, tokens_till_dead=100_000,
                                     dead_fraction=0.10),
    # configs[3]: crosslayer transcoder, bf16, BatchTopK (64 active per token on average)
    "c4_clt_batchtopk_bf16": WorkloadSpec("c4_clt_batchtopk_bf16", 16, 2048, 16384, 8192, "batchtopk", True, True,
                                          rank_u=128, n_outlier=8, outlier_scale=30.0, k=4),
    # configs[4]: crosslayer transcoder, bf16, JumpReLU, dense decoder (needs 8 GPUs)
    "c5_clt_jumprelu_bf16": WorkloadSpec("c5_clt_jumprelu_bf16", 26, 2304, 16384, 4096, "jumprelu", True, True,
                                         rank_u=128, n_outlier=8, outlier_scale=30.0,
                                         lambda_sparsity=4e-4, pre_actv_loss=3e-6),
}


def scaled(spec: WorkloadSpec, **over) -> WorkloadSpec:
    """Copy of ``spec`` with some fields replaced (reduced shapes for tests)."""
    d = dict(spec.__dict__)
    d.update(over)
    return WorkloadSpec(**d)


def make_batch(spec: WorkloadSpec, seed: int = 0, dtype=torch.float32, device="cpu") -> torch.Tensor:
    """``[B, 2, L, D]`` batch: ``[:,0]`` residual-stream input, ``[:,1]`` MLP output.

    x_l = (0.5 u B_l + 0.87 eps_l) * s,  u ~ N(0, I_r) shared over layers,
    B_l ~ N(0, 1/r), eps_l ~ N(0, I), s = per-dimension lognormal(0, 0.5) with a
    few outlier dimensions scaled up; y_l = x_l M_l + 0.1 N(0, I), M_l ~ N(0, 1/D).

    ``device`` selects where the draws and products happen: the CPU generator gives the tensors
    the tests and golden vectors use; a CUDA device gives the same distribution (other values)
    quickly for the large benchmark shapes.
    """
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    B, L, D, r = spec.batch, spec.n_layers, spec.d_acts, spec.rank_u
    kw = dict(generator=g, device=dev)
    u = torch.randn(B, r, **kw)
    s = torch.exp(0.5 * torch.randn(D, **kw))
    out_idx = torch.randperm(D, **kw)[: spec.n_outlier]
    s[out_idx] *= spec.outlier_scale
    batch = torch.empty(B, 2, L, D, dtype=dtype, device=dev)
    for l in range(L):
        Bl = torch.randn(r, D, **kw) / math.sqrt(r)
        eps = torch.randn(B, D, **kw)
        x = (0.5 * (u @ Bl) + 0.87 * eps) * s
        M = torch.randn(D, D, **kw) / math.sqrt(D)
        y = x @ M + 0.1 * torch.randn(B, D, **kw)
        batch[:, 0, l] = x.to(dtype)
        batch[:, 1, l] = y.to(dtype)
    return batch


def make_weights(spec: WorkloadSpec, seed: int = 1, f_lo: int = 0, f_hi: Optional[int] = None) -> Dict[str, object]:
    """Weights of the benchmark configurations:
    W_enc ~ U(+-1/sqrt(D)), b_enc = 0, W_dec ~ U(+-1/sqrt(L F)) for the crosslayer
    decoder and U(+-1/sqrt(F)) for the per-layer one, b_dec = 0, theta constant.

    ``f_lo:f_hi`` returns only that slice of the feature axis (one rank's shard);
    each layer / decoder block draws from its own derived seed, so a shard holds
    exactly the values the unsharded tensors have at those positions.
    """
    L, D, F = spec.n_layers, spec.d_acts, spec.d_features
    f_hi = F if f_hi is None else f_hi
    Fl = f_hi - f_lo

    def uni(shape, bound, sub):
        g = torch.Generator().manual_seed(seed * 1_000_003 + sub)
        return (torch.rand(shape, generator=g) * 2 - 1) * bound

    W_enc = torch.empty(L, D, Fl)
    for l in range(L):
        W_enc[l] = uni((D, F), 1 / math.sqrt(D), l)[:, f_lo:f_hi]
    out: Dict[str, object] = {"W_enc": W_enc, "b_enc": torch.zeros(L, Fl), "b_dec": torch.zeros(L, D)}
    if spec.crosslayer:
        bound = 1 / math.sqrt(L * F)
        Ws: List[torch.Tensor] = []
        for t in range(L):
            Wt = torch.empty(t + 1, Fl, D)
            for s_ in range(t + 1):
                Wt[s_] = uni((F, D), bound, 10_000 + t * (t + 1) // 2 + s_)[f_lo:f_hi]
            Ws.append(Wt)
        out["W_dec"] = Ws
    else:
        Wd = torch.empty(L, Fl, D)
        for l in range(L):
            Wd[l] = uni((F, D), 1 / math.sqrt(F), 10_000 + l)[f_lo:f_hi]
        out["W_dec"] = Wd
    if spec.kind == "jumprelu":
        out["theta"] = torch.full((1, L, Fl), spec.theta)
    return out


def make_last_active(spec: WorkloadSpec, seed: int = 2, f_lo: int = 0, f_hi: Optional[int] = None) -> torch.Tensor:
    """Seeded ``last_active`` counters [L, F] (int64) with ``dead_fraction`` of the
    features already past ``tokens_till_dead`` so that the auxiliary loss has
    dead features to work on."""
    L, F = spec.n_layers, spec.d_features
    f_hi = F if f_hi is None else f_hi
    g = torch.Generator().manual_seed(seed)
    dead = torch.rand(L, F, generator=g) < spec.dead_fraction
    la = torch.where(dead, torch.full((L, F), 2 * spec.tokens_till_dead), torch.zeros(L, F, dtype=torch.long))
    return la[:, f_lo:f_hi].to(torch.long).contiguous()

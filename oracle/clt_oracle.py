"""CPU oracle for the crosslayer-transcoder training step.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain CPU PyTorch, the arithmetic of the reference
project's training step so that the CUDA path can be checked against it on
machines where the reference itself is not installed.  It is a checker: only
the test-suite, the smoke entry and the CPU-baseline leg of the benchmark may
import it.  Nothing in the shipped package imports it.

Parity pin: every function here is compared against the unmodified reference
modules (imported with ``oracle/ref_import.py`` where the reference tree is
present) by ``tests/test_oracle_vs_reference.py``, and against the committed
vectors under ``tests/golden/`` (made from the reference by
``tests/golden/make_golden.py``) everywhere else.

Each function cites the reference file:line it follows
(paths are relative to the reference project root).
"""
from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #
def _autocast(bf16):
    """bf16 runs restate the reference's ``precision: bf16-mixed`` trainer flag
    (config/default.yaml:13) with CPU autocast; ``"fp16"`` restates its default ``16-mixed``; fp32 runs
    use no autocast."""
    if bf16 == "fp16":
        return torch.autocast("cpu", dtype=torch.float16)
    if bf16:
        return torch.autocast("cpu", dtype=torch.bfloat16)
    return contextlib.nullcontext()


def pair_index(t: int, s: int) -> int:
    """Position of decoder block (source s -> target t) in the flat [P, F, D]
    buffer: blocks are ordered by target, then source, exactly as the
    reference's parameters ``W_0 .. W_{L-1}`` are laid out one after another
    (crosslayer_transcoder/model/clt.py:285-288)."""
    return t * (t + 1) // 2 + s


# --------------------------------------------------------------------------- #
# a1  standardizers  (crosslayer_transcoder/model/standardize.py:39-59, 80-108)
# --------------------------------------------------------------------------- #
def standardizer_stats(batch: Tensor) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """mean / unbiased std over the batch axis of ``batch[:,0]`` (input side)
    and ``batch[:,1]`` (output side); std clamped at 1e-8
    (standardize.py:43-46, 83-85)."""
    x, y = batch[:, 0], batch[:, 1]
    mu_i, sd_i = x.mean(dim=0), x.std(dim=0).clamp_(min=1e-8)
    mu_o, sd_o = y.mean(dim=0), y.std(dim=0).clamp_(min=1e-8)
    return mu_i, sd_i, mu_o, sd_o


# --------------------------------------------------------------------------- #
# a3  JumpReLU  (crosslayer_transcoder/model/jumprelu.py:9-48)
# --------------------------------------------------------------------------- #
class _JumpReLU(torch.autograd.Function):
    """forward  f = x * [x > theta and x > 0]             (jumprelu.py:36-37)
    backward dx = g * [x >= 0]                            (jumprelu.py:43-44)
             dtheta = -(theta/bw) * rect((x-theta)/bw) * g (jumprelu.py:46)
    with rect(u) = 1 on -0.5 < u <= 0.5 ... precisely
    step(u+0.5) - step(u-0.5), step(v) = [v > 0]          (jumprelu.py:9-14)."""

    @staticmethod
    def forward(ctx, x, theta, bandwidth):
        ctx.save_for_backward(x, theta)
        ctx.bw = float(bandwidth)
        return x * ((x > theta) & (x > 0.0))

    @staticmethod
    def backward(ctx, g):
        x, theta = ctx.saved_tensors
        bw = ctx.bw
        dx = torch.where(x < 0, torch.zeros_like(g), g)
        u = (x - theta) / bw
        rect = ((u + 0.5) > 0).to(g.dtype) - ((u - 0.5) > 0).to(g.dtype)
        dtheta = -(theta / bw) * rect * g
        return dx, dtheta, None


def jumprelu(x: Tensor, theta: Tensor, bandwidth: float) -> Tensor:
    return _JumpReLU.apply(x, theta, bandwidth)


# --------------------------------------------------------------------------- #
# a4 / a5  TopK selections  (crosslayer_transcoder/model/topk.py:53-63, 76-96)
# --------------------------------------------------------------------------- #
def per_layer_topk(pre: Tensor, k: int) -> Tensor:
    """Per (token, layer): keep the k largest of the F values, relu them,
    everything else 0 (topk.py:56-61).  k > F is an AssertionError (topk.py:56)."""
    assert k <= pre.shape[-1]
    out = torch.zeros_like(pre)
    if k == 0:
        return out
    vals, idx = torch.topk(pre, k, dim=-1, sorted=False)
    out.scatter_(dim=-1, index=idx, src=torch.relu(vals))
    return out


def batch_topk(pre: Tensor, k: int, threshold: Tensor, e: float) -> Tuple[Tensor, Tensor]:
    """One global top-(k*B*L) over the flattened [B*L*F] values, relu, scatter;
    the running threshold moves to (1-e)*thr + e*min(kept) (topk.py:80-95).
    Returns (features, new_threshold)."""
    B, L, F = pre.shape
    assert k <= F
    n = k * B * L
    flat = pre.flatten()
    out = torch.zeros_like(flat)
    if n == 0:
        return out.reshape(B, L, F), threshold
    vals, idx = torch.topk(flat, n, dim=-1, sorted=False)
    vals = torch.relu(vals)
    out.scatter_(dim=-1, index=idx, src=vals)
    new_thr = (1 - e) * threshold + e * vals.min().detach()
    return out.reshape(B, L, F), new_thr


def per_layer_batch_topk(pre: Tensor, k: int, threshold: Tensor, e: float) -> Tuple[Tensor, Tensor]:
    """Per layer, the k*B largest of that layer's [B*F] values, relu, scatter; one running threshold
    per layer (topk.py:109-133).  Returns (features, new_threshold [L])."""
    B, L, F = pre.shape
    assert k <= F
    n = k * B
    flat = pre.permute(1, 0, 2).reshape(L, B * F)
    out = torch.zeros_like(flat)
    if n == 0:
        return out.reshape(L, B, F).permute(1, 0, 2).contiguous(), threshold
    vals, idx = torch.topk(flat, n, dim=-1, sorted=False)
    vals = torch.relu(vals)
    out.scatter_(dim=-1, index=idx, src=vals)
    new_thr = (1 - e) * threshold + e * vals.detach().min(dim=-1).values
    return out.reshape(L, B, F).permute(1, 0, 2).contiguous(), new_thr


# --------------------------------------------------------------------------- #
# parameters / hyper-parameters containers
# --------------------------------------------------------------------------- #
@dataclass
class Params:
    """Plain tensors with the reference's shapes.
    W_enc [L,D,F], b_enc [L,F]            (clt.py:121-125)
    W_dec: list of L tensors [(t+1),F,D]  (clt.py:285-288)  -- crosslayer, or a
           single tensor [L,F,D]          (clt.py:204-206)  -- per-layer
    b_dec [L,D]                           (clt.py:207, 290)
    theta [1,L,F] or None                 (jumprelu.py:55)"""

    W_enc: Tensor
    b_enc: Tensor
    W_dec: object
    b_dec: Tensor
    theta: Optional[Tensor] = None

    @property
    def crosslayer(self) -> bool:
        return isinstance(self.W_dec, (list, tuple))

    def tensors(self) -> List[Tensor]:
        out = [self.W_enc, self.b_enc]
        out += list(self.W_dec) if self.crosslayer else [self.W_dec]
        out.append(self.b_dec)
        if self.theta is not None:
            out.append(self.theta)
        return out

    def clone(self, requires_grad: bool = True) -> "Params":
        c = lambda t: t.detach().clone().requires_grad_(requires_grad)
        return Params(
            c(self.W_enc), c(self.b_enc),
            [c(w) for w in self.W_dec] if self.crosslayer else c(self.W_dec),
            c(self.b_dec), None if self.theta is None else c(self.theta))


@dataclass
class Hyper:
    kind: str = "jumprelu"          # jumprelu | relu | topk | batchtopk | perlayer_batchtopk
    bf16: object = False            # False: fp32, True: bf16 autocast, "fp16": fp16 autocast
    # JumpReLU module (clt_lightning.py:396-409)
    bandwidth: float = 1.0
    lambda_sparsity: float = 0.0    # already multiplied by global_step/max_steps (clt_lightning.py:411-418)
    c_sparsity: float = 1.0
    use_tanh: bool = True
    pre_actv_loss: float = 0.0
    # TopK module (clt_lightning.py:499-517)
    k: int = 0
    k_aux: int = 0
    aux_loss_scale: float = 0.0
    tokens_till_dead: int = 1_000_000
    # BatchTopK
    e: float = 0.01


# --------------------------------------------------------------------------- #
# a2  encoder, a6/a7 decoders
# --------------------------------------------------------------------------- #
def encoder_fwd(xn: Tensor, P: Params, bf16: bool) -> Tensor:
    """pre[b,l,:] = xn[b,l,:] @ W_enc[l] + b_enc[l] (clt.py:157-165).  Under
    bf16 autocast the contraction output is bf16 and the bias add promotes it
    back to the activations' dtype (fp32)."""
    with _autocast(bf16):
        pre = torch.einsum("bld,ldf->blf", xn, P.W_enc).contiguous()
        pre = pre + P.b_enc.to(xn.dtype)
    return pre


def decoder_fwd(feat: Tensor, P: Params, bf16: bool) -> Tensor:
    """Crosslayer: recons[b,t,:] = sum_{s<=t} feat[b,s,:] @ W_t[s] + b[t]
    (clt.py:334-343); each target's contraction is written into a buffer of the
    features' dtype.  Per-layer: recons[b,l,:] = feat[b,l,:] @ W[l] + b[l]
    (clt.py:241-248)."""
    with _autocast(bf16):
        if P.crosslayer:
            L = len(P.W_dec)
            cols = []
            for t in range(L):
                r = torch.einsum("bsf,sfd->bd", feat[:, : t + 1], P.W_dec[t])
                cols.append(r.to(feat.dtype))
            recons = torch.stack(cols, dim=1)
            recons = recons + P.b_dec.to(feat.dtype)
        else:
            recons = torch.einsum("blf,lfd->bld", feat, P.W_dec) + P.b_dec
    return recons


def decoder_norms(P: Params) -> Tensor:
    """[1,L,F] norm of everything feature (s,f) writes: sqrt(sum_{t>=s} |W_t[s,f,:]|^2)
    for the crosslayer decoder (clt_lightning.py:438-445), |W[l,f,:]| for the
    per-layer one (clt_lightning.py:447-448).  Gradients flow through it."""
    if P.crosslayer:
        L = len(P.W_dec)
        F = P.W_dec[0].shape[1]
        acc = torch.zeros(1, L, F, dtype=P.W_dec[0].dtype)
        for t in range(L):
            pad = torch.zeros(L - t - 1, F, dtype=acc.dtype)
            acc = acc + torch.cat([(P.W_dec[t] ** 2).sum(dim=-1), pad], dim=0).unsqueeze(0)
        return acc.sqrt()
    return torch.sqrt((P.W_dec ** 2).sum(dim=-1))


# --------------------------------------------------------------------------- #
# a10  dead-feature bookkeeping (clt_lightning.py:282-288)
# --------------------------------------------------------------------------- #
def update_dead_features(last_active: Tensor, feat: Tensor, tokens_till_dead: int) -> Tuple[Tensor, Tensor]:
    la = last_active.clone()
    la[feat.detach().sum(dim=0) > 0.0] = 0
    la += feat.shape[0]
    return la, la > tokens_till_dead


# --------------------------------------------------------------------------- #
# a9 / a11 / a12  training steps
# --------------------------------------------------------------------------- #
@dataclass
class StepOut:
    loss: Tensor
    terms: Dict[str, Tensor] = field(default_factory=dict)
    pre: Optional[Tensor] = None
    feat: Optional[Tensor] = None
    recons_norm: Optional[Tensor] = None
    last_active: Optional[Tensor] = None
    threshold: Optional[Tensor] = None
    aux_feat: Optional[Tensor] = None


def training_step(P: Params, batch: Tensor, stats, H: Hyper,
                  last_active: Optional[Tensor] = None,
                  threshold: Optional[Tensor] = None) -> StepOut:
    """One forward of the training step up to the scalar loss.

    base module   loss = mean((recons_norm - standardize(y))^2)           (clt_lightning.py:298-304)
    JumpReLU      + lambda * mean_b sum_{l,f} tanh(feat*dec_norm*c)       (clt_lightning.py:450-461)
                  + coef * mean_{b,l} sum_f relu(-pre)                    (clt_lightning.py:465-468)
    TopK          + aux_scale * mean(nan_to_num((decoder(topk_aux(where(dead, pre, -inf)))
                                  - (standardize(y) - recons_norm))^2))   (clt_lightning.py:541-553)
    """
    mu_i, sd_i, mu_o, sd_o = stats
    x, y = batch[:, 0], batch[:, 1]
    xn = (x - mu_i) / sd_i                      # standardize.py:57
    yn = (y - mu_o) / sd_o                      # standardize.py:106
    out = StepOut(loss=torch.zeros(()))
    with _autocast(H.bf16):
        pre = encoder_fwd(xn, P, H.bf16)
        if H.kind == "jumprelu":
            feat = jumprelu(pre, P.theta, H.bandwidth)
        elif H.kind == "relu":
            feat = torch.relu(pre)              # jumprelu.py:21-22
        elif H.kind == "topk":
            feat = per_layer_topk(pre, H.k)
        elif H.kind == "batchtopk":
            feat, out.threshold = batch_topk(pre, H.k, threshold, H.e)
        elif H.kind == "perlayer_batchtopk":
            feat, out.threshold = per_layer_batch_topk(pre, H.k, threshold, H.e)
        else:
            raise ValueError(H.kind)
        recons_norm = decoder_fwd(feat, P, H.bf16)
        mse = ((recons_norm - yn) ** 2).mean()
        loss = mse
        out.terms["mse"] = mse.detach()
        dead = None
        if last_active is not None:
            out.last_active, dead = update_dead_features(last_active, feat, H.tokens_till_dead)
        if H.kind == "jumprelu":
            n = decoder_norms(P)
            w = feat * n * H.c_sparsity
            if H.use_tanh:
                w = torch.tanh(w)
            sparsity = H.lambda_sparsity * w.sum(dim=[1, 2]).mean()
            pal = torch.relu(-pre).sum(dim=-1).mean() * H.pre_actv_loss
            loss = mse + sparsity + pal
            out.terms["sparsity"] = sparsity.detach()
            out.terms["pre_actv"] = pal.detach()
        if H.kind == "topk" and H.k_aux > 0 and dead is not None:
            dead_b = dead.repeat(feat.shape[0], 1, 1)
            dead_pre = torch.where(dead_b, pre, -torch.inf)
            aux_feat = per_layer_topk(dead_pre, H.k_aux)
            aux_recons = decoder_fwd(aux_feat, P, H.bf16)
            err = yn - recons_norm
            aux = torch.nan_to_num((aux_recons - err) ** 2, 0.0)
            loss = mse + H.aux_loss_scale * aux.mean()
            out.terms["aux"] = aux.mean().detach()
            out.aux_feat = aux_feat.detach()
    out.loss = loss
    out.pre, out.feat, out.recons_norm = pre.detach(), feat.detach(), recons_norm.detach()
    return out


def step_with_grads(P: Params, batch: Tensor, stats, H: Hyper, **kw) -> Tuple[StepOut, List[Tensor]]:
    """training_step + autograd backward; returns gradients in ``P.tensors()`` order
    (a zero tensor where a parameter received none)."""
    Pg = P.clone(requires_grad=True)
    out = training_step(Pg, batch, stats, H, **kw)
    out.loss.backward()
    grads = [t.grad if t.grad is not None else torch.zeros_like(t) for t in Pg.tensors()]
    out.loss = out.loss.detach()
    return out, grads


# --------------------------------------------------------------------------- #
# a13  Adam  (clt_lightning.py:339-345: torch.optim.Adam, eps 1e-8, no weight decay)
# --------------------------------------------------------------------------- #
def adam_step(p: Tensor, g: Tensor, m: Tensor, v: Tensor, step: int, lr: float,
              beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
              weight_decay: float = 0.0, decoupled: bool = False) -> Tuple[Tensor, Tensor, Tensor]:
    """Textbook Adam as torch.optim.Adam computes it (step counts from 1):
    m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ;
    p -= lr/(1-b1^t) * m / (sqrt(v)/sqrt(1-b2^t) + eps).
    ``decoupled`` selects the AdamW form p *= 1 - lr*wd (clt_lightning.py:346-352)."""
    if weight_decay != 0.0:
        if decoupled:
            p = p * (1 - lr * weight_decay)
        else:
            g = g + weight_decay * p
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = v.sqrt() / math.sqrt(bc2) + eps
    p = p - (lr / bc1) * (m / denom)
    return p, m, v

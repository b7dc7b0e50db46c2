"""Training modules with the reference's constructor arguments, buffers and logged
scalar names (crosslayer_transcoder/model/clt_lightning.py:29-567).  ``training_step``
hands the batch to the fused CUDA step of ``crosslayer_transcoder_b200.engine`` and
returns its scalar loss; ``loss.backward()`` then runs the fused backward kernels and
``configure_optimizers()`` returns the fused Adam.  Logging-only parts of the reference
(the W&B metric dump every ``log_metrics_every`` steps, the replacement-model
validation) are not part of the training step and are left to the caller.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..engine import FusedAdam, StepEngine
from .clt import CrossLayerTranscoder
from .jumprelu import JumpReLU, ReLU
from .topk import BatchTopK, PerLayerBatchTopK, PerLayerTopK

try:  # Lightning is optional: with it the classes are real LightningModules
    import lightning as L

    _Base = L.LightningModule
except Exception:  # pragma: no cover - depends on the environment

    class _Trainer:
        max_steps = 1
        num_devices = 1

    class _Base(torch.nn.Module):
        """Stand-in with the few LightningModule members the step uses."""

        def __init__(self, *args, **kwargs):
            super().__init__()
            self.trainer = _Trainer()
            self.global_step = 0
            self.logged = {}

        def log(self, name, value, *args, **kwargs):
            self.logged[name] = value

        def save_hyperparameters(self, *args, **kwargs):
            pass


class CrossLayerTranscoderModule(_Base):
    def __init__(self, model: CrossLayerTranscoder, replacement_model=None, dead_features=None,
                 learning_rate: float = 1e-3, compile: bool = False, warmup_steps: int = 0, lr_decay_step: int = 0,
                 lr_decay_factor: float = 1.0, compute_dead_features: bool = False,
                 compute_dead_features_every: int = 100, tokens_till_dead: int = 1_000_000, optimizer: str = "adam",
                 beta1: Optional[float] = None, beta2: Optional[float] = None, log_metrics_every: int = 50,
                 *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.save_hyperparameters(ignore=["model", "replacement_model", "dead_features"])
        self.model, self.replacement_model, self.dead_features = model, replacement_model, dead_features
        self.learning_rate, self.compile, self.tokens_till_dead = learning_rate, compile, tokens_till_dead
        self.warmup_steps, self.lr_decay_step, self.lr_decay_factor = warmup_steps, lr_decay_step, lr_decay_factor
        self.compute_dead_features = compute_dead_features
        self.compute_dead_features_every = compute_dead_features_every
        self.optimizer, self.beta1, self.beta2 = optimizer, beta1, beta2
        self.log_metrics_every = log_metrics_every
        assert model.encoder.n_layers == model.decoder.n_layers, \
            "Encoder and decoder must have the same number of layers"
        self.register_buffer("last_active",
                             torch.zeros(model.encoder.n_layers, model.encoder.d_features, dtype=torch.long))
        #: "auto" follows torch.autocast (bf16-mixed -> tensor cores); "bf16" / "fp32" force a path
        self.precision = "auto"
        #: fuse the (Jump)ReLU into the contraction epilogues: "auto" (by d_acts), True or False
        self.fuse_activation = "auto"
        #: TopK / BatchTopK steps: apply Adam to the decoder inside the sparse backward (see
        #: StepEngine._fused_optimizer).  Off by default because the decoder blocks then have no ``.grad``.
        self.fuse_optimizer = False
        self._engine = StepEngine(self)
        # per-layer forwards of the encoder / decoder (validation-time calls) run on the engine's kernels
        model.encoder.__dict__["_kernel_engine"] = self._engine
        model.decoder.__dict__["_kernel_engine"] = self._engine

    # ---- nonlinearity -> step kind -----------------------------------------------------
    def _kind(self) -> str:
        nl = self.model.nonlinearity
        if isinstance(nl, JumpReLU):
            return "jumprelu"
        if isinstance(nl, (ReLU, torch.nn.ReLU)):
            return "relu"
        if isinstance(nl, PerLayerTopK):
            return "topk"
        if isinstance(nl, BatchTopK):
            return "batchtopk"
        if isinstance(nl, PerLayerBatchTopK):
            return "perlayer_batchtopk"
        raise NotImplementedError(f"nonlinearity {type(nl).__name__} has no fused training step")

    def _hyper(self) -> dict:
        return {"kind": self._kind()}

    def forward(self, acts_norm):
        """``(pre_actvs, features, recons_norm, recons)`` (reference clt_lightning.py:121-129).  On CUDA
        tensors with gradients disabled (validation, metrics) the two contractions run on this library's
        kernels (``StepEngine.infer``); otherwise this is the model's differentiable PyTorch forward."""
        if acts_norm.is_cuda and not torch.is_grad_enabled():
            return self._engine.infer(acts_norm)
        return self.model(acts_norm)

    def configure_model(self):
        """Feature-axis sharding of an unsharded module (reference clt_lightning.py:100-119, which applies
        its DTensor plan when ``trainer.num_devices > 1``): with more than one device and an initialised
        process group, every rank keeps its contiguous slice of the feature axis of the encoder, the
        nonlinearity's thresholds, the decoder blocks and ``last_active`` (``parallel.shard_module``) and
        joins the group (``parallel.attach``).  A module that was built from a shard and attached by hand
        is left as it is.  ``compile`` is accepted and ignored: the step is already a fixed sequence of
        kernels."""
        import torch.distributed as dist

        from .. import parallel

        if getattr(self, "tp_world", 1) > 1:
            return
        n_dev = int(getattr(self.trainer, "num_devices", 1) or 1)
        if n_dev > 1 and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            parallel.shard_module(self, dist.get_rank(), dist.get_world_size())
            parallel.attach(self)

    def _run_step(self, batch, batch_idx):
        if batch_idx == 0:
            self.model.initialize_standardizers(batch)
        loss = self._engine.forward(batch, self._hyper())
        terms = self._engine.last_terms
        periodic = bool(self.log_metrics_every) and batch_idx % self.log_metrics_every == 0
        if getattr(self, "tp_world", 1) == 1 or periodic:
            # every step as the reference does (clt_lightning.py:287); feature shards need a collective
            # for the mean over all shards and log it with the periodic metrics only
            self.log("metrics/dead_features", self._engine.dead_fraction())
        self.log("training/loss", loss.detach())
        if periodic:
            self.log_training_metrics(batch_idx)
        return loss, terms

    def log_training_metrics(self, batch_idx=0):
        """The scalar part of the reference's ``log_training_metrics`` (clt_lightning.py:131-199), computed
        on the device by ``StepEngine.training_metrics`` from the buffers of the step that just ran — no
        ``features.cpu()``.  Histograms, tables and the W&B-specific plots are left to the caller."""
        if not hasattr(self, "tokens_seen"):
            self.tokens_seen = 0
        B = int(self._engine._last_ctx["B"])
        self.tokens_seen += B * self.log_metrics_every
        self.log("training/tokens_seen", self.tokens_seen)
        for name, value in self._engine.training_metrics().items():
            self.log(name, value)

    def training_step(self, batch, batch_idx):
        loss, _ = self._run_step(batch, batch_idx)
        return loss

    def validation_step(self, batch, batch_idx):
        pass

    def on_train_epoch_end(self):
        """A blocking look at the device status word (``training_step`` itself only polls it)."""
        self._engine.check_status("at the end of the epoch")

    def configure_optimizers(self):
        b1 = 0.9 if self.beta1 is None else self.beta1
        b2 = 0.999 if self.beta2 is None else self.beta2
        self.beta1, self.beta2 = b1, b2
        if self.optimizer not in ("adam", "adamw"):
            raise ValueError(f"Optimizer {self.optimizer} not supported")
        decoupled = self.optimizer == "adamw"
        opt = FusedAdam(self.parameters(), self._engine, lr=self.learning_rate, betas=(b1, b2),
                        weight_decay=1e-2 if decoupled else 0.0, decoupled=decoupled)
        if self.warmup_steps > 0:
            sched = torch.optim.lr_scheduler.LinearLR(opt, start_factor=1e-7, end_factor=1.0,
                                                      total_iters=self.warmup_steps)
            return {"optimizer": opt, "lr_scheduler": {"scheduler": sched, "interval": "step", "frequency": 1,
                                                       "name": "warmup"}}
        if self.lr_decay_step > 0:
            sched = torch.optim.lr_scheduler.MultiStepLR(opt, milestones=[self.lr_decay_step],
                                                         gamma=self.lr_decay_factor)
            return {"optimizer": opt, "lr_scheduler": {"scheduler": sched, "interval": "step", "frequency": 1,
                                                       "name": "step_decay"}}
        return opt


class JumpReLUCrossLayerTranscoderModule(CrossLayerTranscoderModule):
    def __init__(self, lambda_sparsity: float = 0.0002, c_sparsity: float = 0.1, use_tanh: bool = True,
                 pre_actv_loss: float = 0.0, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._lambda, self.c, self.use_tanh, self.pre_actv_loss = lambda_sparsity, c_sparsity, use_tanh, pre_actv_loss

    def current_sparsity_penalty(self):
        """Linear ramp lambda * global_step / max_steps (reference clt_lightning.py:411-418)."""
        cur = self._lambda * (self.global_step / self.trainer.max_steps)
        self.log("training/sparsity_penalty", cur)
        return cur

    def _hyper(self) -> dict:
        return {"kind": self._kind(), "lambda_sparsity": self.current_sparsity_penalty(), "c_sparsity": self.c,
                "use_tanh": self.use_tanh, "pre_actv_loss": self.pre_actv_loss, "with_penalties": True}

    def training_step(self, batch, batch_idx):
        loss, terms = self._run_step(batch, batch_idx)
        self.log("training/sparsity_loss", terms[1])
        self.log("training/pre_actv_loss", terms[2])
        return loss


class TopKCrossLayerTranscoderModule(CrossLayerTranscoderModule):
    def __init__(self, topk_aux: torch.nn.Module, tokens_till_dead: int = 100_000, aux_loss_scale: float = 1 / 32,
                 *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.tokens_till_dead, self.topk_aux, self.aux_loss_scale = tokens_till_dead, topk_aux, aux_loss_scale

    def _hyper(self) -> dict:
        return {"kind": self._kind(), "k_aux": int(self.topk_aux.k), "aux_loss_scale": float(self.aux_loss_scale)}

    def training_step(self, batch, batch_idx):
        loss, terms = self._run_step(batch, batch_idx)
        # the reference logs the unscaled mean (clt_lightning.py:554); the step's summand carries the scale
        scale = float(self.aux_loss_scale)
        self.log("training/aux_loss", terms[3] / scale if scale != 0.0 else terms[3])
        return loss

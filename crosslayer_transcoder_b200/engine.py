"""Fused training step of the crosslayer transcoder on B200.

``StepEngine`` runs the reference's ``training_step`` arithmetic
(crosslayer_transcoder/model/clt_lightning.py:290-312, 420-475, 519-567) as a
sequence of calls into ``libclt_b200.so``: forward kernels inside
``StepEngine.forward``, backward kernels inside the autograd node it returns, so
that the caller's ``loss.backward()`` / ``optimizer.step()`` work unchanged.

All parameters of the module live in one flat fp32 buffer (the ``nn.Parameter``s
are views into it), with a flat gradient buffer and, in bf16 mode, a flat bf16 copy
that the tensor-core kernels read and the fused Adam step refreshes.  PyTorch is used
for allocation, streams and autograd plumbing only; there is no eager fallback.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import _lib
from ._lib import DTYPE_CODE, CltError, lib, stream_ptr

_ALIGN = 64  # elements; keeps every segment 256-byte aligned in fp32 and 128-byte aligned in bf16


def _round_up(n: int, a: int = _ALIGN) -> int:
    return (n + a - 1) // a * a


class FlatParams:
    """One flat fp32 buffer holding every parameter of a module, plus matching flat
    buffers for gradients, Adam moments and the bf16 operand copy."""

    def __init__(self, module: torch.nn.Module, device: torch.device, want_bf16: bool):
        self.params: List[torch.nn.Parameter] = [p for p in module.parameters()]
        if not self.params:
            raise CltError("module has no parameters")
        for p in self.params:
            if p.dtype != torch.float32:
                raise CltError(f"parameters must be fp32 master weights (got {p.dtype})")
        self.offsets: Dict[int, int] = {}
        off = 0
        for p in self.params:
            self.offsets[id(p)] = off
            off += _round_up(p.numel())
        self.numel = off
        self.device = device
        self.flat = torch.zeros(off, dtype=torch.float32, device=device)
        self.grad = torch.zeros(off, dtype=torch.float32, device=device)
        self.shadow: Optional[torch.Tensor] = None
        self.exp_avg: Optional[torch.Tensor] = None
        self.exp_avg_sq: Optional[torch.Tensor] = None
        with torch.no_grad():
            for p in self.params:
                view = self.view_of(p, self.flat)
                view.copy_(p.data)
                p.data = view
        self._shadow_version = None
        if want_bf16:
            self.ensure_shadow()

    def view_of(self, p: torch.nn.Parameter, buf: torch.Tensor) -> torch.Tensor:
        o = self.offsets[id(p)]
        return buf[o:o + p.numel()].view(p.shape)

    def is_packed(self) -> bool:
        base = self.flat.data_ptr()
        return all(p.data_ptr() == base + 4 * self.offsets[id(p)] for p in self.params)

    def _version(self):
        return tuple(p._version for p in self.params)

    def ensure_shadow(self):
        """(Re)build the bf16 copy when parameters were changed by anything but the fused Adam step."""
        v = self._version()
        if self.shadow is None:
            self.shadow = torch.empty(self.numel, dtype=torch.bfloat16, device=self.device)
            self._shadow_version = None
        if self._shadow_version != v:
            lib().call("clt_cast_bf16", self.flat, self.shadow, self.numel, stream_ptr())
            self._shadow_version = v

    def ensure_moments(self):
        if self.exp_avg is None:
            self.exp_avg = torch.zeros_like(self.flat)
            self.exp_avg_sq = torch.zeros_like(self.flat)


class _Workspace:
    """Per-batch-size activation buffers, reused between steps."""

    def __init__(self):
        self.key = None
        self.buf: Dict[str, torch.Tensor] = {}

    def get(self, name, shape, dtype, device, zero=False):
        t = self.buf.get(name)
        if t is None or t.shape != torch.Size(shape) or t.dtype != dtype or t.device != device:
            t = (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=device)
            self.buf[name] = t
        return t


class StepEngine:
    def __init__(self, module):
        self.module = module                      # a CrossLayerTranscoderModule
        self.flat: Optional[FlatParams] = None
        self.ws = _Workspace()
        self.status: Optional[torch.Tensor] = None
        self.fired: Optional[torch.Tensor] = None
        self.launches = 0                         # kernels launched by this engine (for reporting)
        self.last_terms: Optional[torch.Tensor] = None
        self.profile: Optional[dict] = None
        # the device status word is copied to pinned host memory after every backward and looked at,
        # without waiting, when the next steps begin
        self.optimizer = None                     # the FusedAdam of configure_optimizers (for fuse_optimizer)
        #: feature shards, fused exchange: called right before the last collective of a step (the all-reduce
        #: of the decoder-bias gradient); parallel.ShardedBatchUploader orders its peer copies through it
        self.before_last_collective = None
        self.after_backward = None          # called when the last kernel of a backward pass has been enqueued
        self.decoder_updated = False              # set by a backward that stepped the decoder itself
        self._status_host: Optional[torch.Tensor] = None
        self._status_evt = [None, None]
        self._status_pending = [False, False]
        self._status_slot = 0

    # ------------------------------------------------------------------ setup
    def _call(self, name, *args, tag: str = ""):
        """One C-ABI call = one kernel launch on the current stream.  With ``self.profile`` set to a
        dict, CUDA events around the call collect per-entry-point device time (``tag`` keeps apart two uses
        of one entry point with different shapes)."""
        if self.profile is None:
            lib().call(name, *args)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            lib().call(name, *args)
            e1.record()
            self.profile.setdefault(name + tag, []).append((e0, e1))
        self.launches += 1

    def profile_summary(self) -> Dict[str, dict]:
        """{entry point: {"launches", "ms_total", "ms_avg"}} from the collected events (synchronises)."""
        torch.cuda.synchronize()
        out = {}
        for name, evs in (self.profile or {}).items():
            ms = [a.elapsed_time(b) for a, b in evs]
            out[name] = {"launches": len(ms), "ms_total": sum(ms), "ms_avg": sum(ms) / max(1, len(ms))}
        return out

    def _precision(self, batch) -> bool:
        """True for the bf16 tensor-core path.  ``module.precision`` forces it ("bf16" / "fp32");
        "auto" follows the autocast state the trainer set up (bf16-mixed and 16-mixed -> bf16 operands)."""
        mode = getattr(self.module, "precision", "auto")
        if mode == "bf16":
            return True
        if mode == "fp32":
            return False
        if torch.is_autocast_enabled("cuda"):
            dt = torch.get_autocast_dtype("cuda")
            if dt in (torch.bfloat16, torch.float16):
                # fp16 autocast (the reference's default "16-mixed", config/default.yaml:13) also runs on the
                # bf16 tensor-core path: the operands are rounded to bf16 (fp32 exponent range, so nothing can
                # overflow under a GradScaler's loss scale), which stays inside the bf16 parity bar against
                # the reference's fp16 run; the scale itself reaches the kernels as the loss gradient.
                return True
            raise NotImplementedError(f"autocast dtype {dt} is not supported by the fused step")
        return False

    def prepare(self, device: torch.device, bf16: bool):
        lib().check_device()
        if self.flat is None or self.flat.device != device or not self.flat.is_packed():
            old = self.flat
            self.flat = FlatParams(self.module, device, bf16)
            if old is not None and old.exp_avg is not None and old.numel == self.flat.numel and old.device == device:
                self.flat.exp_avg, self.flat.exp_avg_sq = old.exp_avg, old.exp_avg_sq
        if bf16:
            self.flat.ensure_shadow()
        if self.status is None or self.status.device != device:
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
        enc = self.module.model.encoder
        if self.fired is None or self.fired.device != device:
            # one bit per feature, set by the kernels that see the features of a step
            self.fired = torch.zeros(enc.n_layers, (enc.d_features + 31) // 32, dtype=torch.int32, device=device)

    def check_status(self, where=""):
        """Blocking check: synchronises with the device, raises ``CltError`` if any kernel since the last
        check gave up on a bounded wait, met an out-of-range index or overflowed a list."""
        if self.status is not None:
            self._status_pending = [False, False]
            _lib.check_status(self.status, where)

    def post_status(self):
        """Enqueue a copy of the status word to pinned host memory (no synchronisation).  Called at the
        end of every backward; ``poll_status`` reads the copies that have arrived."""
        if self.status is None:
            return
        if self._status_host is None:
            self._status_host = torch.zeros(2, dtype=torch.int32).pin_memory()
            self._status_evt = [torch.cuda.Event(), torch.cuda.Event()]
        slot = self._status_slot
        self._status_slot ^= 1
        self._status_host[slot:slot + 1].copy_(self.status, non_blocking=True)
        self._status_evt[slot].record()
        self._status_pending[slot] = True

    def poll_status(self, where="(reported by an earlier step)"):
        """Non-blocking check on the training path: looks at the status copies whose transfer has
        finished (normally the one of the step before last) and raises ``CltError`` on a failure code, so
        that a run never trains on for long with partial results.  The word is sticky on the device
        until it is reported."""
        for slot in (0, 1):
            if self._status_pending[slot] and self._status_evt[slot].query():
                self._status_pending[slot] = False
                code = int(self._status_host[slot])
                if code != 0:
                    self._status_pending = [False, False]
                    self.status.zero_()
                    raise CltError(f"device status {code:#x} {where}: "
                                   f"{_lib.STATUS_NAMES.get(code, 'unknown code')}")

    # ------------------------------------------------------------------ helpers
    def _operand(self, p: torch.nn.Parameter, bf16: bool) -> torch.Tensor:
        """The tensor a contraction reads for parameter ``p``: its bf16 copy or the fp32 master."""
        return self.flat.view_of(p, self.flat.shadow) if bf16 else p.data

    def _dec_flat(self, bf16: bool):
        """(operand buffer [P,F,D], fp32 master [P,F,D], gradient [P,F,D]) of the decoder blocks;
        they are adjacent in the flat buffer in block order."""
        dec = self.module.model.decoder
        blocks = dec.blocks()
        F, D = dec.d_features, dec.d_acts
        o0 = self.flat.offsets[id(blocks[0])]
        n = 0
        for w in blocks:
            if self.flat.offsets[id(w)] != o0 + n:
                raise CltError("decoder blocks are not adjacent in the flat parameter buffer")
            n += _round_up(w.numel())
            if w.numel() % _ALIGN:
                raise CltError("decoder block size must be a multiple of 64 elements")
        P = n // (F * D)
        sl = slice(o0, o0 + n)
        op = (self.flat.shadow if bf16 else self.flat.flat)[sl].view(P, F, D)
        return op, self.flat.flat[sl].view(P, F, D), self.flat.grad[sl].view(P, F, D)

    def _stats(self):
        m = self.module.model
        ins, outs = m.input_standardizer, m.output_standardizer
        if ins is None or outs is None:
            raise CltError("the fused step needs both standardizers")
        if not (ins.is_initialized and outs.is_initialized):
            raise ValueError("Standardizer not initialized")
        f = lambda t: t.detach().float().contiguous()
        return f(ins.mean), f(ins.std), f(outs.mean), f(outs.std)

    def _fuse_activation(self, D: int, F: int, bf16: bool) -> bool:
        """Fuse the (Jump)ReLU into the contraction epilogues?  ``module.fuse_activation`` forces it
        (True / False); "auto" fuses when the contraction is long enough to hide the epilogue behind
        the tensor-core main loop of a tile (d_acts >= 1536), and always on the fp32 CUDA-core path."""
        mode = getattr(self.module, "fuse_activation", "auto")
        if F % 8 != 0:
            return True
        if mode == "auto":
            return (not bf16) or D >= 1536
        return bool(mode)

    def _dead_count(self, dev) -> torch.Tensor:
        """One device int that ``clt_dead_update`` fills with the number of dead features of this rank."""
        t = getattr(self, "_dead_cnt", None)
        if t is None or t.device != dev:
            t = self._dead_cnt = torch.zeros(1, dtype=torch.int32, device=dev)
        return t

    def dead_fraction(self) -> torch.Tensor:
        """``idxs_dead.float().mean()`` of the last step (reference clt_lightning.py:286-287) as a device
        scalar; on feature shards the mean over all shards."""
        enc = self.module.model.encoder
        cnt = self._dead_cnt.to(torch.float32)
        world = getattr(self.module, "tp_world", 1)
        if world > 1:
            from .parallel import all_reduce_sum

            all_reduce_sum(cnt, self.module.tp_group)
        return (cnt / float(enc.n_layers * enc.d_features * world)).reshape(())

    @torch.no_grad()
    def training_metrics(self) -> Dict[str, torch.Tensor]:
        """The scalar metrics of the reference's ``log_training_metrics`` (clt_lightning.py:131-199) for the
        step that just ran, as device scalars under the reference's names: fraction of variance unexplained
        (overall and per layer), MSE (overall, per layer, rescaled), the standard deviation of the
        normalised reconstruction and L0 (overall and per layer).  Two kernels reduce buffers the step
        already holds (``clt_recon_stats``, ``clt_count_active``); nothing is copied to the host.  On feature
        shards every rank gets the figures of the whole model."""
        c = getattr(self, "_last_ctx", None)
        if c is None:
            raise CltError("training_metrics() needs a training step to have run")
        B, L, D, F = c["B"], c["L"], c["D"], c["F"]
        dev = c["batch"].device
        s = stream_ptr()
        _, _, mu_o, sd_o = c["stats"]
        world = getattr(self.module, "tp_world", 1)
        group = getattr(self.module, "tp_group", None)
        rows, b_lo, n = c["recon_rows"]
        st = torch.zeros(L, D, 6, dtype=torch.float32, device=dev)
        if n > 0:
            self._call("clt_recon_stats", rows, c["batch"], c["in_code"], mu_o, sd_o, st, b_lo, n, L, D, s)
        cnt = torch.zeros(L, dtype=torch.int64, device=dev)
        src, code, npl = c["l0_src"]
        self._call("clt_count_active", src, code, npl, L, cnt, s)
        if world > 1:
            from .parallel import all_reduce_sum

            if c.get("px") is not None:
                all_reduce_sum(st, group)           # every rank reduced its own tokens
            all_reduce_sum(cnt, group)              # every rank counted its own features
        yn, yn2, err, err_raw, r, r2 = st.unbind(-1)
        ss_tot = yn2 - yn * yn / B
        fvu = err / ss_tot
        n_el = float(B) * L * D
        out = {"metrics/fraction_of_variance_unexplained": fvu.mean(),
               "metrics/train_mse": err.sum() / n_el,
               "metrics/train_mse_rescaled": err_raw.sum() / n_el,
               "metrics/recons_standardized_std": ((r2.sum() - r.sum() ** 2 / n_el) / (n_el - 1)).clamp_min(0).sqrt(),
               "metrics/L0_avg_per_layer": cnt.sum().float() / (float(B) * L)}
        fvu_l, mse_l, l0_l = fvu.mean(dim=-1), err.sum(dim=-1) / (float(B) * D), cnt.float() / float(B)
        for l in range(L):
            out[f"layers/fraction_of_variance_unexplained/layer_{l}"] = fvu_l[l]
            out[f"layers/train_mse/layer_{l}"] = mse_l[l]
            out[f"layers/L0/layer_{l}"] = l0_l[l]
        return out

    def _bandwidth(self, nl) -> float:
        """JumpReLU bandwidth as a host number, read from the device buffer once."""
        if getattr(self, "_bw_cache", None) is None:
            self._bw_cache = float(nl.bandwidth)
        return self._bw_cache

    # ------------------------------------------------------------------ fused exchange over peer memory
    def _peer_exchange(self, B: int, L: int, D: int, T, dev):
        """Buffers of the exchange that is fused into the kernels (feature shards on one node), created
        once per shape, collectively over the group.  The token axis is split over the ranks: this rank
        owns rows ``[b_lo, b_lo + b_cnt)``.  ``slots`` [2, R, rows_per_rank, L, D] fp32 receives every rank's
        partial (auxiliary) reconstruction rows for the owned tokens, one slot per source rank (the
        decoder kernels store into them); ``recon_own`` / ``aux_own`` are their sums (``_sum_slots``);
        ``drecon`` / ``daux`` [L, B, D] receive every owner's gradient rows (the loss backward writes
        them into all ranks' copies)."""
        mod = self.module
        # bf16 steps exchange the partial rows as bf16 (half the NVLink bytes; the owner sums them in fp32);
        # module.tp_bf16_partials = False keeps fp32 slots
        slot_bf16 = T == torch.bfloat16 and bool(getattr(mod, "tp_bf16_partials", True)) and D % 8 == 0
        key = (B, L, D, T, dev, slot_bf16)
        px = getattr(self, "_px", None)
        if px is not None and px["key"] == key:
            return px
        from .parallel import PeerBuffer

        world, rank, group = mod.tp_world, mod.tp_rank, mod.tp_group
        rpr = (B + world - 1) // world
        b_lo = min(B, rank * rpr)
        b_cnt = max(0, min(B, b_lo + rpr) - b_lo)
        # [0] main, [1] auxiliary reconstruction; one slot per source rank
        slots = PeerBuffer((2, world, rpr, L, D), torch.bfloat16 if slot_bf16 else torch.float32, dev, group)
        own = torch.empty(2, rpr, L, D, dtype=torch.float32, device=dev)
        drecon = PeerBuffer((L, B, D), T, dev, group)
        daux = PeerBuffer((L, B, D), T, dev, group)
        self._px = dict(key=key, rpr=rpr, b_lo=b_lo, b_cnt=b_cnt, slots=slots, recon_own=own[0], aux_own=own[1],
                        recon_bases=slots.bases, slot_bf16=int(slot_bf16),
                        aux_bases=slots.bases + world * rpr * L * D * (2 if slot_bf16 else 4),
                        drecon=drecon, daux=daux, token=torch.zeros(1, dtype=torch.float32, device=dev))
        return self._px

    def has_fused_exchange(self) -> bool:
        """Does this module's step run the exchange fused into the kernels (token rows owned by ranks)?"""
        mod = self.module
        return bool(getattr(mod, "tp_fused", False)) and getattr(mod, "tp_world", 1) > 1 and \
            mod._kind() in ("jumprelu", "relu", "topk", "batchtopk", "perlayer_batchtopk") and \
            mod.model.encoder.d_acts % 8 == 0

    def _sum_slots(self, px, which: int):
        """Add the per-source slots of the owned rows (0: main, 1: auxiliary reconstruction)."""
        n = px["recon_own"].numel()
        self._call("clt_sum_slots", px["slots"].local[which], px["recon_own"] if which == 0 else px["aux_own"],
                   self.module.tp_world, n, px["slot_bf16"], stream_ptr())

    def _gather_form(self, k: int, world: int, D: int) -> int:
        """``_warp_rows`` unless ``module.decoder_gather_warp`` (True / False) forces a form."""
        forced = getattr(self.module, "decoder_gather_warp", None)
        return int(bool(forced)) if forced is not None else self._warp_rows(k, world, D)

    @staticmethod
    def _warp_rows(k: int, world: int, D: int) -> int:
        """Which form of the token-major decoder gather: 1 = one warp per (token, target layer), 0 = one CTA
        of four warps that split the row's entries.  The warp form keeps four times as many tokens in flight, so
        the tokens that gather from one decoder block at about the same time share more of its rows in L2
        (12-layer, 32768-feature workload, k = 32: 1.99 ms against 2.34 ms); the CTA form is for long entry
        lists and for rows too wide for one warp's registers."""
        return int(k <= 8 * world or (k <= 64 and D <= 1024))

    def _rank_barrier(self, px):
        """Order the ranks on the compute stream: a one-element all-reduce.  After it, every kernel that
        any rank enqueued before its own call has finished, so rows pushed into this rank's buffers
        have landed."""
        from .parallel import all_reduce_sum

        all_reduce_sum(px["token"], self.module.tp_group)

    # ------------------------------------------------------------------ forward
    def forward(self, batch: torch.Tensor, hyper: dict) -> torch.Tensor:
        """Run the forward half of the step on ``batch`` ``[B, 2, L, D]`` and return the scalar
        loss, connected to the parameters through an autograd node that runs the backward half."""
        if not batch.is_cuda:
            raise CltError("the fused training step runs on CUDA tensors only (no CPU fallback)")
        if batch.dtype not in DTYPE_CODE:
            raise CltError(f"unsupported batch dtype {batch.dtype}")
        batch = batch.contiguous()
        bf16 = self._precision(batch)
        self.prepare(batch.device, bf16)
        self.poll_status()
        kind = hyper["kind"]
        if kind in ("jumprelu", "relu"):
            ctx = self._forward_dense(batch, hyper, bf16)
        elif kind == "topk":
            ctx = self._forward_topk(batch, hyper, bf16)
        elif kind in ("batchtopk", "perlayer_batchtopk"):
            ctx = self._forward_batchtopk(batch, hyper, bf16)
        else:
            raise NotImplementedError(f"nonlinearity kind {kind!r}")
        self.last_terms = ctx["out"][1:5]          # mse, sparsity, pre-activation, auxiliary summands
        self._last_ctx = ctx
        params = self.flat.params
        return _StepFunction.apply(self, ctx, *params)

    def _forward_dense(self, batch, h, bf16):
        mod = self.module
        model = mod.model
        enc, dec, nl = model.encoder, model.decoder, model.nonlinearity
        B, L, D, F = batch.shape[0], enc.n_layers, enc.d_acts, enc.d_features
        dev = batch.device
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        crosslayer = 1 if dec.crosslayer else 0
        mu_i, sd_i, mu_o, sd_o = self._stats()
        ws = self.ws
        xn = ws.get("xn", (L, B, D), T, dev)
        z = ws.get("z", (L, B, F), T, dev)
        feat = ws.get("feat", (L, B, F), T, dev)
        # reconstruction buffer with an 8-float tail: [0:2] encoder-side loss sums (summed over
        # feature shards together with the partial reconstructions), [2:4] reconstruction-loss sums
        rbuf = ws.get("recon", (B * L * D + 8,), torch.float32, dev)
        recon, acc = rbuf[: B * L * D].view(B, L, D), rbuf[B * L * D:]
        out = torch.empty(5, dtype=torch.float32, device=dev)       # loss + 4 terms
        acc.zero_()
        world, group = getattr(mod, "tp_world", 1), getattr(mod, "tp_group", None)
        first_rank = getattr(mod, "tp_rank", 0) == 0
        in_code = DTYPE_CODE[batch.dtype]
        self._call("clt_prep_input", batch, in_code, mu_i, sd_i, xn, int(bf16), B, L, D, s)
        theta = nl.theta.data if h["kind"] == "jumprelu" else None
        lam = float(h.get("lambda_sparsity", 0.0))
        norm = None
        W_op, W_master, _ = self._dec_flat(bf16)
        if lam != 0.0:
            norm = ws.get("dec_norm", (L, F), torch.float32, dev)
            self._call("clt_dec_norms", W_master, norm, L, F, D, crosslayer, s)
        c_sp, use_tanh = float(h.get("c_sparsity", 1.0)), int(h.get("use_tanh", True))
        want_pre = int(float(h.get("pre_actv_loss", 0.0)) != 0.0)
        fused = self._fuse_activation(D, F, bf16)
        if fused:
            self._call("clt_encoder_fwd_act", xn, self._operand(enc.W, bf16), enc.b.data, theta, norm, z, feat,
                       self.fired, acc[0:2], c_sp, use_tanh, want_pre, B, L, D, F, int(bf16), self.status, s)
        else:
            self._call("clt_encoder_fwd_store", xn, self._operand(enc.W, bf16), z, B, L, D, F, int(bf16), self.status, s)
            self._call("clt_act_fwd", z, enc.b.data, theta, norm, feat, self.fired, acc[0:2], c_sp, use_tanh, want_pre,
                       B, L, F, int(bf16), s)
        px = None
        if world > 1 and getattr(mod, "tp_fused", False) and D % 8 == 0:
            # exchange fused into the kernels (see _peer_exchange): the contraction's epilogue adds each tile
            # to the owning rank's buffer, the loss runs on the owned rows
            from .parallel import all_reduce_sum

            px = self._peer_exchange(B, L, D, T, dev)
            self._call("clt_decoder_dense_fwd_push", feat, W_op, dec.b.data if first_rank else None,
                       px["recon_bases"], px["rpr"], world, mod.tp_rank, px["slot_bf16"], B, L, D, F, crosslayer,
                       int(bf16), self.status, s)
            self._rank_barrier(px)                      # every rank's tiles have landed in the owners' slots
            self._sum_slots(px, 0)
            b_lo, b_cnt = px["b_lo"], px["b_cnt"]
            if b_cnt > 0:
                self._call("clt_loss_fwd", px["recon_own"], None, batch[b_lo:b_lo + b_cnt], in_code, mu_o, sd_o,
                           acc[2:4], b_cnt, L, D, s)
            all_reduce_sum(acc[0:4], group)             # encoder-side sums of all shards, loss sums of all owners
        else:
            self._call("clt_decoder_dense_fwd", feat, W_op, dec.b.data if first_rank else None, recon, B, L, D, F,
                       crosslayer, int(bf16), self.status, s)
            if world > 1:
                from .parallel import all_reduce_sum

                all_reduce_sum(rbuf[: B * L * D + 2], group)      # partial reconstructions + encoder-side sums
            self._call("clt_loss_fwd", recon, None, batch, in_code, mu_o, sd_o, acc[2:4], B, L, D, s)
        pal = float(h.get("pre_actv_loss", 0.0))
        self._call("clt_finalize_loss", acc[2:4], acc[0:2], out[0:1], out[1:5], 1.0 / (B * L * D), lam / B,
                   pal / (B * L), 0.0, s)
        self._call("clt_dead_update", mod.last_active, self.fired, None, B, int(mod.tokens_till_dead), L, F,
                   self._dead_count(dev), None, s)
        return dict(kind=h["kind"], bf16=bf16, batch=batch, B=B, L=L, D=D, F=F, crosslayer=crosslayer, lam=lam,
                    pal=pal, c=float(h.get("c_sparsity", 1.0)), use_tanh=int(h.get("use_tanh", True)),
                    bandwidth=self._bandwidth(nl) if h["kind"] == "jumprelu" else 1.0, out=out,
                    stats=(mu_i, sd_i, mu_o, sd_o), norm=norm, in_code=in_code, fused=fused, px=px,
                    recon_rows=(px["recon_own"], px["b_lo"], px["b_cnt"]) if px is not None else (recon, 0, B),
                    l0_src=(feat, 2 if bf16 else 0, B * F))

    # ------------------------------------------------------------------ inference forward
    @torch.no_grad()
    def infer(self, acts: torch.Tensor):
        """``(pre_actvs [B,L,F], features [B,L,F], recons_norm [B,L,D], recons [B,L,D])`` of
        ``CrossLayerTranscoder.forward`` (reference crosslayer_transcoder/model/clt.py:403-425) on this
        library's kernels from end to end: standardise + cast (``clt_prep_acts``), encoder contraction
        (``clt_encoder_fwd_store``), the nonlinearity — (Jump)ReLU by ``clt_act_fwd``, PerLayerTopK by
        ``clt_select_topk``, BatchTopK / PerLayerBatchTopK by the histogram select, each exactly what the
        module's ``forward(..., layer="all")`` computes, running-threshold update included — the dense or
        sparse decoder, and the output de-standardisation (``clt_destandardize``).  The token-major fp32
        tensors of the return value are written by ``clt_export_blf`` / ``clt_scatter_features``.  No
        autograd graph is built.  On feature shards the partial reconstructions are summed over the ranks;
        the returned features are the rank's slice, and nonlinearities that rank across the whole feature
        axis (TopK, BatchTopK) are refused there."""
        if not acts.is_cuda:
            raise CltError("the kernel forward runs on CUDA tensors only (no CPU fallback)")
        if acts.dim() != 3:
            raise CltError(f"expected acts [batch, n_layers, d_acts], got {tuple(acts.shape)}")
        if acts.dtype not in DTYPE_CODE:
            raise CltError(f"unsupported activation dtype {acts.dtype}")
        mod, model = self.module, self.module.model
        enc, dec, nl = model.encoder, model.decoder, model.nonlinearity
        B, L, D, F = acts.shape[0], enc.n_layers, enc.d_acts, enc.d_features
        if acts.shape[1] != L or acts.shape[2] != D:
            raise CltError(f"acts {tuple(acts.shape)} do not match n_layers={L}, d_acts={D}")
        acts = acts.contiguous()
        bf16 = self._precision(acts)
        dev = acts.device
        self.prepare(dev, bf16)
        kind = mod._kind()
        world, group = getattr(mod, "tp_world", 1), getattr(mod, "tp_group", None)
        if world > 1 and kind not in ("jumprelu", "relu"):
            raise NotImplementedError("the kernel forward on feature shards supports element-wise nonlinearities only")
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        f32 = lambda t: t.detach().float().contiguous()
        ins, outs = model.input_standardizer, model.output_standardizer
        if ins is not None and not ins.is_initialized:
            raise ValueError("Standardizer not initialized")
        xn = torch.empty(L, B, D, dtype=T, device=dev)
        self._call("clt_prep_acts", acts, DTYPE_CODE[acts.dtype], f32(ins.mean) if ins is not None else None,
                   f32(ins.std) if ins is not None else None, xn, int(bf16), B, L, D, s)
        z = torch.empty(L, B, F, dtype=T, device=dev)
        self._call("clt_encoder_fwd_store", xn, self._operand(enc.W, bf16), z, B, L, D, F, int(bf16), self.status, s)
        pre_actvs = torch.empty(B, L, F, dtype=torch.float32, device=dev)
        self._call("clt_export_blf", z, enc.b.data, pre_actvs, B, L, F, int(bf16), s)
        features = torch.empty(B, L, F, dtype=torch.float32, device=dev)
        recon = torch.empty(B, L, D, dtype=torch.float32, device=dev)
        W_op, _, _ = self._dec_flat(bf16)
        crosslayer = 1 if dec.crosslayer else 0
        bias = dec.b.data if getattr(mod, "tp_rank", 0) == 0 else None
        if kind in ("jumprelu", "relu"):
            feat = torch.empty(L, B, F, dtype=T, device=dev)
            scratch = torch.zeros(2, dtype=torch.float32, device=dev)
            theta = nl.theta.data if kind == "jumprelu" else None
            self._call("clt_act_fwd", z, enc.b.data, theta, None, feat, None, scratch, 1.0, 0, 0, B, L, F, int(bf16), s)
            self._call("clt_export_blf", feat, None, features, B, L, F, int(bf16), s)
            self._call("clt_decoder_dense_fwd", feat, W_op, bias, recon, B, L, D, F, crosslayer, int(bf16),
                       self.status, s)
            if world > 1:
                from .parallel import all_reduce_sum

                all_reduce_sum(recon, group)
        elif kind == "topk":
            k = int(nl.k)
            assert k <= F                                   # reference topk.py:56
            if k == 0:
                features.zero_()
                recon.copy_(dec.b.data.float().unsqueeze(0).expand(B, L, D))
            else:
                idx = torch.empty(L, B, k, dtype=torch.int32, device=dev)
                val = torch.empty(L, B, k, dtype=torch.float32, device=dev)
                self._call("clt_select_topk", z, enc.b.data, idx, val, None, B, L, F, k, int(bf16), s)
                self._call("clt_scatter_features", idx, val, None, features, B, L, F, k, B * k, self.status, s)
                self._call("clt_sparse_decoder_fwd", idx, val, None, None, B * k, W_op, bias, recon, B, L, D, F, k,
                           crosslayer, 0, int(bf16), self.status, s)
        else:
            k = int(nl.k)
            assert k <= F                                   # reference topk.py:80, 113
            if nl.e is None and k > 0:
                raise TypeError("BatchTopK needs its EMA rate `e` (reference topk.py:95)")
            idx, val, etok, row_start, row_cnt, npl = self._batchtopk_select(z, kind, k, B, L, F, bf16, dev, fired=None)
            self._call("clt_scatter_features", idx, val, etok, features, B, L, F, 1, npl, self.status, s)
            self._call("clt_sparse_decoder_fwd", idx, val, row_start, row_cnt, npl, W_op, bias, recon, B, L, D, F, 1,
                       crosslayer, 0, int(bf16), self.status, s)
        if outs is not None:
            if not outs.is_initialized:
                raise ValueError("Standardizer not initialized")
            recons = torch.empty_like(recon)
            self._call("clt_destandardize", recon, f32(outs.mean), f32(outs.std), recons, B, L, D, s)
        else:
            recons = recon
        return pre_actvs, features, recon, recons

    @torch.no_grad()
    def encode_layer(self, acts_norm: torch.Tensor, layer: int) -> torch.Tensor:
        """``Encoder.forward_layer`` (reference clt.py:134-145): ``acts_norm [..., D] @ W[layer] + b[layer]``
        on the contraction kernel, fp32 ``[..., F]`` out."""
        enc = self.module.model.encoder
        lead, D, F = acts_norm.shape[:-1], enc.d_acts, enc.d_features
        x = acts_norm.reshape(-1, D).contiguous()
        if x.dtype not in DTYPE_CODE:
            x = x.float()
        B = x.shape[0]
        bf16 = self._precision(x)
        dev = x.device
        self.prepare(dev, bf16)
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        xn = torch.empty(1, B, D, dtype=T, device=dev)
        self._call("clt_prep_acts", x, DTYPE_CODE[x.dtype], None, None, xn, int(bf16), B, 1, D, s)
        z = torch.empty(1, B, F, dtype=T, device=dev)
        self._call("clt_encoder_fwd_store", xn, self._operand(enc.W, bf16)[layer:layer + 1], z, B, 1, D, F, int(bf16),
                   self.status, s)
        out = torch.empty(B, 1, F, dtype=torch.float32, device=dev)
        self._call("clt_export_blf", z, enc.b.data[layer:layer + 1] if enc.bias else None, out, B, 1, F, int(bf16), s)
        return out.reshape(*lead, F)

    @torch.no_grad()
    def decode_layer(self, features: torch.Tensor, layer: int) -> torch.Tensor:
        """``Decoder.forward_layer`` / ``CrosslayerDecoder.forward_layer`` (reference clt.py:216-231, 304-317):
        the reconstruction of target ``layer`` from ``features [..., F]`` (per-layer decoder; a 4-D input
        ``[batch, seq, L, F]`` is cut to its ``layer``) or ``[..., layer + 1, F]`` (crosslayer decoder: the
        features of the source layers 0..layer), as one contraction over the concatenated source axis."""
        dec = self.module.model.decoder
        D, F = dec.d_acts, dec.d_features
        if dec.crosslayer:
            n_src = layer + 1
            if features.shape[-2] != n_src or features.shape[-1] != F:
                raise CltError(f"expected features [..., {n_src}, {F}], got {tuple(features.shape)}")
            lead = features.shape[:-2]
            w = dec.get_parameter(f"W_{layer}")
        else:
            if features.ndim == 4:
                features = features[:, :, layer, :]
            n_src, lead = 1, features.shape[:-1]
            w = dec.W
        K = n_src * F
        x = features.reshape(-1, K).float().contiguous()
        B = x.shape[0]
        bf16 = self._precision(x)
        dev = x.device
        self.prepare(dev, bf16)
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        feat = torch.empty(1, B, K, dtype=T, device=dev)
        self._call("clt_import_blf", x, feat, B, 1, K, int(bf16), s)
        w_op = self._operand(w, bf16)
        w_op = w_op.reshape(1, K, D) if dec.crosslayer else w_op[layer:layer + 1]
        recon = torch.empty(B, 1, D, dtype=torch.float32, device=dev)
        self._call("clt_decoder_dense_fwd", feat, w_op, dec.b.data[layer:layer + 1], recon, B, 1, D, K, 0, int(bf16),
                   self.status, s)
        return recon.reshape(*lead, D)

    # ------------------------------------------------------------------ backward
    def backward(self, ctx: dict, gscale: torch.Tensor):
        if ctx["kind"] in ("jumprelu", "relu"):
            self._backward_dense(ctx, gscale)
        elif ctx["kind"] in ("topk", "batchtopk"):
            self._backward_topk(ctx, gscale)
        else:
            raise NotImplementedError(ctx["kind"])
        if self.after_backward is not None:
            self.after_backward()
        self.post_status()

    def _zero_small_grads(self):
        """Gradients accumulated with atomics start from zero; contraction outputs are overwritten."""
        model = self.module.model
        small = [model.encoder.b, model.decoder.b]
        if hasattr(model.nonlinearity, "theta"):
            small.append(model.nonlinearity.theta)
        for p in small:
            self.flat.view_of(p, self.flat.grad).zero_()

    def _backward_dense(self, c, gscale):
        model = self.module.model
        enc, dec, nl = model.encoder, model.decoder, model.nonlinearity
        B, L, D, F, bf16 = c["B"], c["L"], c["D"], c["F"], c["bf16"]
        dev = c["batch"].device
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        ws = self.ws
        xn, z, feat = ws.buf["xn"], ws.buf["z"], ws.buf["feat"]
        recon = ws.buf["recon"][: B * L * D].view(B, L, D)
        drecon = ws.get("drecon", (L, B, D), T, dev)
        dpre = ws.get("dpre", (L, B, F), T, dev)
        _, _, mu_o, sd_o = c["stats"]
        g = self.flat.grad
        gview = lambda p: self.flat.view_of(p, g)
        self._zero_small_grads()
        gs = gscale.detach().to(torch.float32).reshape(1).contiguous()
        px = c.get("px")
        if px is not None:
            from .parallel import all_reduce_sum

            drecon = px["drecon"].local
            if px["b_cnt"] > 0:
                self._call("clt_loss_bwd_push", px["recon_own"], None, c["batch"], c["in_code"], mu_o, sd_o, gs, 0.0,
                           px["drecon"].bases, None, self.module.tp_world, int(bf16), gview(dec.b), B, px["b_lo"],
                           px["b_cnt"], L, D, s)
            if self.before_last_collective is not None:
                self.before_last_collective()
            all_reduce_sum(gview(dec.b), self.module.tp_group)   # partial bias gradients; orders the ranks
        else:
            self._call("clt_loss_bwd", recon, None, c["batch"], c["in_code"], mu_o, sd_o, gs, 0.0, drecon, None,
                       int(bf16), gview(dec.b), B, L, D, s)
        W_op, W_master, dW_dec = self._dec_flat(bf16)
        theta = nl.theta.data if c["kind"] == "jumprelu" else None
        dtheta = gview(nl.theta) if c["kind"] == "jumprelu" else None
        norm = c["norm"]
        dnorm = None
        if norm is not None:
            dnorm = ws.get("dnorm", (L, F), torch.float32, dev)
            dnorm.zero_()
        if c["fused"]:
            self._call("clt_decoder_dense_bwd_dfeat", drecon, W_op, z, enc.b.data, theta, norm, dpre, dtheta,
                       gview(enc.b), dnorm, c["bandwidth"], c["lam"] / B, c["c"], c["pal"] / (B * L), c["use_tanh"], gs,
                       B, L, D, F, c["crosslayer"], int(bf16), self.status, s)
        else:
            self._call("clt_decoder_dense_bwd_dfeat_raw", drecon, W_op, dpre, B, L, D, F, c["crosslayer"], int(bf16),
                       self.status, s)
            self._call("clt_act_bwd", dpre, z, enc.b.data, theta, norm, dpre, dtheta, gview(enc.b), dnorm,
                       c["bandwidth"], c["lam"] / B, c["c"], c["pal"] / (B * L), c["use_tanh"], gs, B, L, F, int(bf16), s)
        rowcoef = None
        if norm is not None:
            rowcoef = ws.get("rowcoef", (L, F), torch.float32, dev)
            self._call("clt_norm_coef", dnorm, norm, rowcoef, L * F, s)
        self._call("clt_decoder_dense_bwd_dw", feat, drecon, dW_dec, rowcoef, W_master if rowcoef is not None else None,
                   B, L, D, F, c["crosslayer"], int(bf16), self.status, s)
        self._call("clt_encoder_dense_bwd_dw", xn, dpre, gview(enc.W), B, L, D, F, int(bf16), self.status, s)



    # ------------------------------------------------------------------ TopK path
    def _forward_topk(self, batch, h, bf16):
        """PerLayerTopK step (reference clt_lightning.py:519-567): encoder contraction, exact per-row
        selection, sparse decoder gather; the auxiliary dead-feature loss runs as dense contractions
        over the compacted dead features."""
        mod = self.module
        model = mod.model
        enc, dec, nl = model.encoder, model.decoder, model.nonlinearity
        B, L, D, F = batch.shape[0], enc.n_layers, enc.d_acts, enc.d_features
        k = int(nl.k)
        assert k <= F                                   # reference topk.py:56
        k_aux = int(h.get("k_aux", 0))
        assert k_aux <= F
        dev = batch.device
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        crosslayer = 1 if dec.crosslayer else 0
        mu_i, sd_i, mu_o, sd_o = self._stats()
        ws = self.ws
        xn = ws.get("xn", (L, B, D), T, dev)
        z = ws.get("z", (L, B, F), T, dev)
        # [reconstruction | auxiliary reconstruction | 8-float tail of loss sums]: the first two are
        # partial sums over this rank's features and are reduced together across feature shards
        n_rec = B * L * D
        rbuf = ws.get("recon2", (2 * n_rec + 8,), torch.float32, dev)
        recon, aux_recon_buf, acc = rbuf[:n_rec].view(B, L, D), rbuf[n_rec:2 * n_rec].view(B, L, D), rbuf[2 * n_rec:]
        out = torch.empty(5, dtype=torch.float32, device=dev)
        acc.zero_()
        world, group = getattr(mod, "tp_world", 1), getattr(mod, "tp_group", None)
        bias = dec.b.data if getattr(mod, "tp_rank", 0) == 0 else None      # added once, not per shard
        in_code = DTYPE_CODE[batch.dtype]
        W_op, _, _ = self._dec_flat(bf16)
        # exchange fused into the kernels: the main decoder adds its rows into the owning rank's buffer,
        # the loss runs on the owned rows only (see _peer_exchange)
        px = None
        if world > 1 and getattr(mod, "tp_fused", False) and k > 0 and D % 8 == 0:
            px = self._peer_exchange(B, L, D, T, dev)
        self._call("clt_prep_input", batch, in_code, mu_i, sd_i, xn, int(bf16), B, L, D, s)
        self._call("clt_encoder_fwd_store", xn, self._operand(enc.W, bf16), z, B, L, D, F, int(bf16), self.status, s)
        kk = max(k, 1)
        idx = ws.get("idx", (L, B, kk), torch.int32, dev)
        val = ws.get("val", (L, B, kk), torch.float32, dev)
        if k > 0:
            self._call("clt_select_topk", z, enc.b.data, idx, val, self.fired if world == 1 else None, B, L, F, k,
                       int(bf16), s)
            if world > 1:
                # every shard offers its k best values per row; the k-th largest of all of them is the
                # row's threshold, and each shard keeps its candidates at or above it
                from .parallel import all_gather

                val_all = ws.get("val_all", (world, L, B, kk), torch.float32, dev)
                all_gather(val_all, val, group)
                thr = ws.get("thr_main", (L, B), torch.float32, dev)
                self._call("clt_topk_threshold", val_all, thr, L * B, world, k, s)
                self._call("clt_topk_apply_threshold", idx, val, thr, self.fired, B, L, F, k, s)
        else:
            idx.zero_()
            val.zero_()
        dead = ws.get("dead", (L, F), torch.uint8, dev)
        soon = ws.get("soon_dead", (L,), torch.int32, dev)
        self._call("clt_dead_update", mod.last_active, self.fired, dead, B, int(mod.tokens_till_dead), L, F,
                   self._dead_count(dev), soon, s)
        aux = None
        aux_recon = None
        aux_scale = float(h.get("aux_loss_scale", 0.0))
        pending = []                                    # collectives in flight (feature shards only)
        h_gather = None
        main_early, h_cnt = False, None

        def main_decoder():
            if px is not None:
                self._call("clt_sparse_decoder_fwd_push", idx, val, None, None, B * kk, W_op, bias,
                           px["recon_bases"], px["rpr"], world, mod.tp_rank, px["slot_bf16"], B, L, D, F, kk,
                           crosslayer, self._gather_form(kk, world, D), int(bf16), self.status, s)
                return
            self._call("clt_sparse_decoder_fwd", idx, val, None, None, B * kk, W_op, bias, recon, B, L, D, F, kk,
                       crosslayer, self._gather_form(kk, world, D), int(bf16), self.status, s)
            if world > 1:
                from .parallel import all_reduce_sum

                pending.append(all_reduce_sum(rbuf[:n_rec], group, async_op=True))

        if k_aux > 0:
            dead_list = ws.get("dead_list", (L, F), torch.int32, dev)
            n_dead = ws.get("n_dead", (L,), torch.int32, dev)
            self._call("clt_dead_compact", dead, dead_list, n_dead, L, F, s)
            nd_pad = self._aux_width(n_dead)
            self.last_nd_pad = nd_pad
            # The dead features' pre-activations come from a small contraction of their own over the compact
            # encoder columns (nd_pad of F columns: a tenth of the main one) instead of a second and third sweep
            # of z, whose dead columns are spread over four fifths of its 32-byte sectors.
            az, ab, alist, aF = z, enc.b.data, dead_list, F
            if getattr(mod, "aux_compact_encoder", True) and nd_pad < F:
                w_ec = ws.get("w_enc_c", (L, D, nd_pad), T, dev)
                ab = ws.get("b_enc_c", (L, nd_pad), torch.float32, dev)
                self._call("clt_gather_enc_cols", self._operand(enc.W, bf16), enc.b.data, dead_list, n_dead, w_ec, ab,
                           L, D, F, nd_pad, int(bf16), s)
                az = ws.get("z_c", (L, B, nd_pad), T, dev)
                self._call("clt_encoder_fwd_store", xn, w_ec, az, B, L, D, nd_pad, int(bf16), self.status, s,
                           tag="[dead]")
                alist, aF = self._iota(L, nd_pad, dev), nd_pad
            exchange = False
            if world > 1:
                # a row whose positive dead values, summed over the shards, do not exceed k_aux keeps all
                # of them: the candidate exchange is needed only if some row has more
                from .parallel import all_gather, all_reduce_sum

                cnt = ws.get("aux_cnt", (L, B), torch.int32, dev)
                self._call("clt_aux_count", az, ab, alist, n_dead, cnt, B, L, aF, int(bf16), s)
                if px is not None:
                    # the sum of the counts travels while the main decoder's gather and push run
                    h_cnt = all_reduce_sum(cnt, group, async_op=True)
                    main_early = True
                else:
                    all_reduce_sum(cnt, group)
            else:
                cnt = None
        if main_early:
            main_decoder()
            h_cnt.wait()
        if k_aux > 0:
            exchange = self._aux_exchange(soon, cnt, k_aux)
            a_aux = ws.get("a_aux", (L, B, nd_pad), T, dev)
            if exchange:
                # offer this shard's k_aux best dead values per row; the gather runs while the main
                # decoder works
                cand = ws.get("aux_cand", (L, B, k_aux), torch.float32, dev)
                self._call("clt_select_aux", az, ab, alist, n_dead, None, cand, None, 1, B, L, aF, k_aux,
                           nd_pad, int(bf16), None, self.status, s)
                cand_all = ws.get("aux_cand_all", (world, L, B, k_aux), torch.float32, dev)
                h_gather = all_gather(cand_all, cand, group, async_op=True)
        if px is None:
            main_decoder()          # its all-reduce runs while the auxiliary path computes
        if k_aux > 0:
            if not exchange:
                self._call("clt_select_aux", az, ab, alist, n_dead, a_aux, None, None, 0, B, L, aF, k_aux,
                           nd_pad, int(bf16), cnt, self.status, s)
            else:
                h_gather.wait()
                thr_aux = ws.get("thr_aux", (L, B), torch.float32, dev)
                self._call("clt_topk_threshold", cand_all, thr_aux, L * B, world, k_aux, s)
                self._call("clt_select_aux", az, ab, alist, n_dead, a_aux, None, thr_aux, 2, B, L, aF, k_aux,
                           nd_pad, int(bf16), None, self.status, s)
            P = W_op.shape[0]
            w_c = ws.get("w_c", (P, nd_pad, D), T, dev)
            self._call("clt_gather_rows", W_op, dead_list, n_dead, w_c, L, F, D, nd_pad, crosslayer, int(bf16), s)
            aux_recon = aux_recon_buf
            if px is not None:
                # the contraction's epilogue adds each tile to the owning ranks' buffers
                self._call("clt_decoder_dense_fwd_push", a_aux, w_c, bias, px["aux_bases"], px["rpr"], world,
                           mod.tp_rank, px["slot_bf16"], B, L, D, nd_pad, crosslayer, int(bf16), self.status, s)
            else:
                self._call("clt_decoder_dense_fwd", a_aux, w_c, bias, aux_recon, B, L, D, nd_pad, crosslayer,
                           int(bf16), self.status, s)
            aux = dict(dead_list=dead_list, n_dead=n_dead, nd_pad=nd_pad, a_aux=a_aux, w_c=w_c)
            if world > 1 and px is None:
                pending.append(all_reduce_sum(rbuf[n_rec:2 * n_rec], group, async_op=True))
        if px is not None:
            from .parallel import all_reduce_sum

            if not main_early:
                main_decoder()
            self._rank_barrier(px)                      # every rank's rows have landed in the owners' slots
            for h_ in pending:
                h_.wait()
            self._sum_slots(px, 0)
            if aux is not None:
                self._sum_slots(px, 1)
            b_lo, b_cnt = px["b_lo"], px["b_cnt"]
            if b_cnt > 0:
                self._call("clt_loss_fwd", px["recon_own"], px["aux_own"] if aux is not None else None,
                           batch[b_lo:b_lo + b_cnt], in_code, mu_o, sd_o, acc[2:4], b_cnt, L, D, s)
            all_reduce_sum(acc[2:4], group)             # loss sums of all owners
        else:
            for h_ in pending:
                h_.wait()
            self._call("clt_loss_fwd", recon, aux_recon, batch, in_code, mu_o, sd_o, acc[2:4], B, L, D, s)
        self._call("clt_finalize_loss", acc[2:4], None, out[0:1], out[1:5], 1.0 / (B * L * D), 0.0, 0.0,
                   aux_scale if aux is not None else 0.0, s)
        return dict(kind="topk", bf16=bf16, batch=batch, B=B, L=L, D=D, F=F, k=kk, crosslayer=crosslayer, out=out,
                    stats=(mu_i, sd_i, mu_o, sd_o), in_code=in_code, aux=aux, aux_scale=aux_scale, idx=idx, val=val,
                    px=px,
                    recon_rows=(px["recon_own"], px["b_lo"], px["b_cnt"]) if px is not None else (recon, 0, B),
                    l0_src=(val, 0, B * kk))

    # ------------------------------------------------------------------ BatchTopK path
    def _forward_batchtopk(self, batch, h, bf16):
        """BatchTopK step (reference topk.py:76-96 inside clt_lightning.py:290-312): one threshold for
        the whole batch from a three-level histogram select, survivors collected into per-layer entry
        lists, then the same sparse decoder and loss as the per-layer TopK path."""
        mod = self.module
        model = mod.model
        enc, dec, nl = model.encoder, model.decoder, model.nonlinearity
        B, L, D, F = batch.shape[0], enc.n_layers, enc.d_acts, enc.d_features
        k = int(nl.k)
        assert k <= F                                   # reference topk.py:80
        if nl.e is None and k > 0:
            raise TypeError("BatchTopK needs its EMA rate `e` for training (reference topk.py:95)")
        dev = batch.device
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        crosslayer = 1 if dec.crosslayer else 0
        mu_i, sd_i, mu_o, sd_o = self._stats()
        ws = self.ws
        world, group = getattr(mod, "tp_world", 1), getattr(mod, "tp_group", None)
        rank = getattr(mod, "tp_rank", 0)
        bias = dec.b.data if rank == 0 else None
        xn = ws.get("xn", (L, B, D), T, dev)
        z = ws.get("z", (L, B, F), T, dev)
        n_rec = B * L * D
        rbuf = ws.get("recon2", (2 * n_rec + 8,), torch.float32, dev)
        recon, acc = rbuf[:n_rec].view(B, L, D), rbuf[2 * n_rec:]
        out = torch.empty(5, dtype=torch.float32, device=dev)
        acc.zero_()
        in_code = DTYPE_CODE[batch.dtype]
        W_op, _, _ = self._dec_flat(bf16)
        self._call("clt_prep_input", batch, in_code, mu_i, sd_i, xn, int(bf16), B, L, D, s)
        self._call("clt_encoder_fwd_store", xn, self._operand(enc.W, bf16), z, B, L, D, F, int(bf16), self.status, s)
        idx, val, etok, row_start, row_cnt, npl = self._batchtopk_select(z, h["kind"], k, B, L, F, bf16, dev,
                                                                          fired=self.fired)
        self._call("clt_dead_update", mod.last_active, self.fired, None, B, int(mod.tokens_till_dead), L, F,
                   self._dead_count(dev), None, s)
        px = None
        if world > 1 and getattr(mod, "tp_fused", False) and D % 8 == 0:
            # exchange fused into the kernels: the sparse decoder stores its partial rows into the owning
            # ranks' slots, the loss runs on the owned rows (see _peer_exchange)
            from .parallel import all_reduce_sum

            px = self._peer_exchange(B, L, D, T, dev)
            self._call("clt_sparse_decoder_fwd_push", idx, val, row_start, row_cnt, npl, W_op, bias,
                       px["recon_bases"], px["rpr"], world, rank, px["slot_bf16"], B, L, D, F, 1, crosslayer,
                       self._gather_form(k, world, D), int(bf16), self.status, s)
            self._rank_barrier(px)                      # every rank's rows have landed in the owners' slots
            self._sum_slots(px, 0)
            b_lo, b_cnt = px["b_lo"], px["b_cnt"]
            if b_cnt > 0:
                self._call("clt_loss_fwd", px["recon_own"], None, batch[b_lo:b_lo + b_cnt], in_code, mu_o, sd_o,
                           acc[2:4], b_cnt, L, D, s)
            all_reduce_sum(acc[2:4], group)             # loss sums of all owners
        else:
            self._call("clt_sparse_decoder_fwd", idx, val, row_start, row_cnt, npl, W_op, bias, recon, B, L, D, F, 1,
                       crosslayer, self._gather_form(k, world, D), int(bf16), self.status, s)
            if world > 1:
                from .parallel import all_reduce_sum

                all_reduce_sum(rbuf[:n_rec], group)
            self._call("clt_loss_fwd", recon, None, batch, in_code, mu_o, sd_o, acc[2:4], B, L, D, s)
        self._call("clt_finalize_loss", acc[2:4], None, out[0:1], out[1:5], 1.0 / (B * L * D), 0.0, 0.0, 0.0, s)
        return dict(kind="batchtopk", bf16=bf16, batch=batch, B=B, L=L, D=D, F=F, k=1, crosslayer=crosslayer, out=out,
                    stats=(mu_i, sd_i, mu_o, sd_o), in_code=in_code, aux=None, aux_scale=0.0, idx=idx, val=val,
                    npl=npl, etok=etok, px=px,
                    recon_rows=(px["recon_own"], px["b_lo"], px["b_cnt"]) if px is not None else (recon, 0, B),
                    l0_src=(val, 0, npl))

    def _batchtopk_select(self, z, kind, k, B, L, F, bf16, dev, fired):
        """BatchTopK / PerLayerBatchTopK selection on the stored contraction output ``z`` (reference
        topk.py:76-96, 109-133): threshold by the three-level histogram select, survivors collected into
        per-layer entry lists, running threshold updated.  Returns (idx, val, etok, row_start, row_cnt, npl)."""
        mod = self.module
        enc, nl = mod.model.encoder, mod.model.nonlinearity
        ws, s = self.ws, stream_ptr()
        world, group = getattr(mod, "tp_world", 1), getattr(mod, "tp_group", None)
        rank = getattr(mod, "tp_rank", 0)
        h = {"kind": kind}
        # BatchTopK: one selection over the whole batch (all layers, all feature shards);
        # PerLayerBatchTopK: one per layer
        groups = L if h["kind"] == "perlayer_batchtopk" else 1
        n_keep = k * B * L // groups
        npl = max(1, min(n_keep, B * F))                # entry slots per layer (worst case: all in one layer)
        idx = ws.get("bt_idx", (L, npl), torch.int32, dev)
        val = ws.get("bt_val", (L, npl), torch.float32, dev)
        etok = ws.get("bt_tok", (L, npl), torch.int32, dev)
        row_start = ws.get("bt_row_start", (L, B), torch.int32, dev)
        row_cnt = ws.get("bt_row_cnt", (L, B), torch.int32, dev)
        if n_keep > 0:
            state = ws.get("bt_state", (groups, 8), torch.int64, dev, zero=True)
            # histograms [groups, 2048] followed by the "candidate list invalid" word, so that feature shards
            # sum the flag together with the counters
            nh = groups * 2048
            hbuf_l = ws.get("bt_hist_local", (nh + 8,), torch.int64, dev, zero=True)
            hbuf = ws.get("bt_hist", (nh + 8,), torch.int64, dev) if world > 1 else hbuf_l
            hist_l, inval_l, hist, inval = hbuf_l[:nh], hbuf_l[nh:], hbuf[:nh], hbuf[nh:]
            # steady state: one sweep of z collects everything at or above 0.9 of the last threshold, and the
            # radix levels and the collection read that list; the full sweeps below are enqueued as well and
            # return at once unless this step cannot trust its list
            use_list = bool(getattr(mod, "batchtopk_candidates", True))
            if use_list:
                cap = int(min(L * B * F, max(8 * k * B * L, 65536), 2 ** 31 - 1))
                cand_feat = ws.get("bt_cand_feat", (cap,), torch.int32, dev)
                cand_val = ws.get("bt_cand_val", (cap,), torch.float32, dev)
                cand_row = ws.get("bt_cand_row", (cap,), torch.int32, dev)
                cand_fill = ws.get("bt_cand_fill", (1,), torch.int32, dev)
                cand_start = ws.get("bt_cand_start", (L, B), torch.int32, dev)
                cand_cnt = ws.get("bt_cand_cnt", (L, B), torch.int32, dev)
                self._call("clt_batchtopk_candidates", z, enc.b.data, state, cand_feat, cand_val, cand_row, cand_fill,
                           cand_start, cand_cnt, inval_l, groups, B, L, F, cap, int(bf16), s)
            # level 0, its retry without the guessed floor (returns at once unless requested), levels 1, 2
            for level, retry in ((0, 0), (0, 1), (1, 0), (2, 0)):
                self._call("clt_batchtopk_hist", z, enc.b.data, state, hist_l, inval_l if use_list else None, level,
                           retry, groups, B, L, F, int(bf16), s)
                if use_list and not retry:
                    self._call("clt_batchtopk_hist_list", cand_val, cand_row, cand_fill, state, hist_l, inval_l, level,
                               groups, B, cap, s)
                if world > 1:
                    from .parallel import all_reduce_sum

                    hbuf.copy_(hbuf_l)
                    all_reduce_sum(hbuf, group)
                self._call("clt_batchtopk_pick", hist, hist_l if world > 1 else None, state,
                           inval if use_list else None, level, retry, groups, n_keep, s)
            quota = None
            if world > 1:
                # elements equal to the threshold are kept in rank order until the global count is reached
                from .parallel import all_gather

                ties = torch.empty(world, groups, dtype=torch.int64, device=dev)
                all_gather(ties, state[:, 5].contiguous(), group)
                before = ties[:rank].sum(dim=0)
                quota = (state[:, 3] - before).clamp(min=0).minimum(state[:, 5]).contiguous()
            fill = ws.get("bt_fill", (L,), torch.int32, dev)
            self._call("clt_batchtopk_collect", z, enc.b.data, state, quota, idx, val, etok, row_start, row_cnt, fill,
                       fired, groups, B, L, F, npl, int(bf16), self.status, s)
            if use_list:
                self._call("clt_batchtopk_filter", cand_feat, cand_val, cand_start, cand_cnt, state, quota, idx, val,
                           etok, row_start, row_cnt, fill, fired, groups, B, L, F, npl, self.status, s)
            self._call("clt_batchtopk_threshold_update", state, nl.threshold, float(nl.e), groups, s)
        else:
            val.zero_()
            row_start.zero_()
            row_cnt.zero_()
        return idx, val, etok, row_start, row_cnt, npl

    def _backward_topk(self, c, gscale):
        model = self.module.model
        enc, dec = model.encoder, model.decoder
        B, L, D, F, k, bf16 = c["B"], c["L"], c["D"], c["F"], c["k"], c["bf16"]
        cross = c["crosslayer"]
        dev = c["batch"].device
        T = torch.bfloat16 if bf16 else torch.float32
        s = stream_ptr()
        ws = self.ws
        xn = ws.buf["xn"]
        n_rec = B * L * D
        recon = ws.buf["recon2"][:n_rec].view(B, L, D)
        aux_recon = ws.buf["recon2"][n_rec:2 * n_rec].view(B, L, D)
        aux = c["aux"]
        drecon = ws.get("drecon", (L, B, D), T, dev)
        daux = ws.get("daux", (L, B, D), T, dev) if aux is not None else None
        _, _, mu_o, sd_o = c["stats"]
        g = self.flat.grad
        gview = lambda p: self.flat.view_of(p, g)
        gview(dec.b).zero_()
        gs = gscale.detach().to(torch.float32).reshape(1).contiguous()
        px = c.get("px")
        if px is not None:
            # owned rows only; the gradient rows go straight into every rank's buffers, and the all-reduce
            # of the bias gradient's partial sums also orders the ranks before those buffers are read
            from .parallel import all_reduce_sum

            b_lo, b_cnt = px["b_lo"], px["b_cnt"]
            drecon, daux = px["drecon"].local, (px["daux"].local if aux is not None else None)
            if b_cnt > 0:
                self._call("clt_loss_bwd_push", px["recon_own"], px["aux_own"] if aux is not None else None,
                           c["batch"], c["in_code"], mu_o,
                           sd_o, gs, c["aux_scale"] if aux is not None else 0.0, px["drecon"].bases,
                           px["daux"].bases if aux is not None else None, self.module.tp_world, int(bf16),
                           gview(dec.b), B, b_lo, b_cnt, L, D, s)
            if self.before_last_collective is not None:
                self.before_last_collective()
            all_reduce_sum(gview(dec.b), self.module.tp_group)
        else:
            self._call("clt_loss_bwd", recon, aux_recon if aux is not None else None, c["batch"], c["in_code"],
                       mu_o, sd_o, gs, c["aux_scale"] if aux is not None else 0.0, drecon, daux, int(bf16),
                       gview(dec.b), B, L, D, s)
        W_op, W_master, dW_dec = self._dec_flat(bf16)
        idx, val = c["idx"], c["val"]
        npl, etok = c.get("npl", B * k), c.get("etok")       # entry slots per layer, token of each entry
        col_ptr = ws.get("col_ptr", (L, F + 1), torch.int32, dev)
        cursor = ws.get("cursor", (L, F), torch.int32, dev)
        ent = ws.get("ent", (L, npl), torch.int32, dev)
        dval = ws.get("dval", (L, npl), torch.float32, dev)
        self._call("clt_csc_build", idx, val, col_ptr, cursor, ent, npl, L, F, self.status, s)
        fuse_opt = self._fused_optimizer(F)
        dW_c = dpre_c = db_c = dead_pos = None
        if aux is not None:
            # position of every dead feature in the compact operands: the feature-major kernels below add the
            # auxiliary loss's compact gradients through it
            dead_pos = ws.get("dead_pos", (L, F), torch.int32, dev)
            self._call("clt_dead_positions", aux["dead_list"], aux["n_dead"], dead_pos, L, F, aux["nd_pad"], s)
            # auxiliary path, decoder side first: its compact weight gradient is an input of the fused
            # decoder backward + optimizer kernel
            nd_pad, a_aux, w_c = aux["nd_pad"], aux["a_aux"], aux["w_c"]
            dl, n_dead = aux["dead_list"], aux["n_dead"]
            P = w_c.shape[0]
            zeros_b = ws.get("zeros_b", (L, nd_pad), torch.float32, dev, zero=True)
            dpre_c = ws.get("dpre_c", (L, B, nd_pad), T, dev)
            db_c = ws.get("db_c", (L, nd_pad), torch.float32, dev)
            db_c.zero_()
            # gradient w.r.t. the auxiliary features, ReLU-masked by the selection (a_aux > 0)
            self._call("clt_decoder_dense_bwd_dfeat", daux, w_c, a_aux, zeros_b, None, None, dpre_c, None, db_c, None,
                       1.0, 0.0, 1.0, 0.0, 0, None, B, L, D, nd_pad, cross, int(bf16), self.status, s)
            dW_c = ws.get("dW_c", (P, nd_pad, D), torch.float32, dev)
            self._call("clt_decoder_dense_bwd_dw", a_aux, daux, dW_c, None, None, B, L, D, nd_pad, cross, int(bf16),
                       self.status, s)
        if fuse_opt:
            # the decoder rows are updated as their gradients are formed: no gradient buffer, no separate
            # optimizer pass over the decoder (the optimizer's step() then covers the other parameters)
            opt = self.optimizer
            fp = self.flat
            if opt._linked_to is not fp or fp.exp_avg is None:
                opt._link_state(fp)
            grp = opt.param_groups[0]
            o0 = fp.offsets[id(dec.blocks()[0])]
            n = W_master.numel()
            m_dec, v_dec = fp.exp_avg[o0:o0 + n], fp.exp_avg_sq[o0:o0 + n]
            b1, b2 = grp["betas"]
            self._call("clt_sparse_bwd_dec_adam", col_ptr, ent, val, etok, npl, W_master, m_dec, v_dec,
                       W_op if bf16 else None, drecon, dval, dW_c if aux is not None else None, dead_pos,
                       aux["nd_pad"] if aux is not None else 0, B, L, D, F, k, cross, int(bf16), float(grp["lr"]),
                       float(b1), float(b2), float(grp["eps"]), float(grp["weight_decay"]), int(grp["decoupled"]),
                       opt._step + 1, s)
            self.decoder_updated = True
        else:
            self._call("clt_sparse_bwd_dec", col_ptr, ent, val, etok, npl, W_op, drecon, dW_dec, dval, B, L, D, F, k,
                       cross, int(bf16), s)
            if aux is not None:
                self._call("clt_scatter_rows", dW_c, aux["dead_list"], aux["n_dead"], dW_dec, L, F, D, aux["nd_pad"],
                           cross, s)
        dWe_c = None
        if aux is not None:
            nd_pad = aux["nd_pad"]
            dWe_c = ws.get("dWe_c", (L, D, nd_pad), torch.float32, dev)
            self._call("clt_encoder_dense_bwd_dw", xn, dpre_c, dWe_c, B, L, D, nd_pad, int(bf16), self.status, s)
        self._call("clt_sparse_bwd_enc", col_ptr, ent, dval, etok, npl, xn, gview(enc.W), gview(enc.b), dWe_c,
                   db_c if aux is not None else None, dead_pos, aux["nd_pad"] if aux is not None else 0, B, L, D, F,
                   k, int(bf16), s)

    def _aux_state(self):
        st = getattr(self, "_aux_hist", None)
        if st is None:
            st = self._aux_hist = dict(step=0, host=torch.zeros(2, 2, dtype=torch.int32).pin_memory(),
                                       evt=[torch.cuda.Event(), torch.cuda.Event()])
        return st

    def _aux_width(self, n_dead: torch.Tensor) -> int:
        """nd_pad, the column count of the compact dead-feature operands of the auxiliary path.  It depends on a
        device value (the largest per-layer dead count); reading it every step would drain the launch queue.  The
        first two steps do read it (one blocking host read each).  From then on every step copies its values to
        pinned memory without waiting (``_aux_exchange``) and a step uses what the step before last left there,
        which has always arrived when it is needed: ``soon_dead`` of two steps ago, the number of features that
        were dead or within two steps of the limit then.  A feature leaves that set only by firing, so it bounds
        the dead count of this step from above whatever happens in between: the operands are never too small, and
        in steady state the bound is the dead count itself."""
        st = self._aux_state()
        i = st["step"]
        if i < 2:
            nd = int(n_dead.max())                              # blocking: first two steps only
        else:
            st["evt"][i & 1].synchronize()                      # the copy made two steps ago into this slot
            nd = int(st["host"][i & 1, 0])
        return max(64, _round_up(nd, 64))

    def _aux_exchange(self, soon_dead: torch.Tensor, cnt, k_aux: int) -> bool:
        """On feature shards: does some row have more than k_aux positive dead values in total (then the shards
        must exchange candidates)?  Decided like the operand width: from the current counts in the first two
        steps, afterwards from the largest row count of two steps ago, switching on at 3/4 of k_aux; should a row
        outgrow k_aux within two steps all the same, ``clt_select_aux`` reports it through the status word.
        Every rank takes the same decision (the counts are summed over the ranks first).  Also posts this step's
        values for the step after next; call once per step, after ``_aux_width``."""
        st = self._aux_state()
        i = st["step"]
        st["step"] = i + 1
        slot = i & 1
        cmax_t = cnt.max() if cnt is not None else soon_dead.new_zeros(())
        if i < 2:
            exchange = cnt is not None and int(cmax_t) > k_aux   # blocking: first two steps only
        else:
            exchange = cnt is not None and 4 * int(st["host"][slot, 1]) > 3 * k_aux
        st["host"][slot].copy_(torch.stack([soon_dead.max(), cmax_t]).to(torch.int32), non_blocking=True)
        st["evt"][slot].record()
        return exchange

    def _iota(self, L: int, n: int, dev) -> torch.Tensor:
        """[L, n] int32 rows 0, 1, ..., n-1: the "dead list" of operands that are already compact."""
        t = getattr(self, "_iota_t", None)
        if t is None or t.shape != (L, n) or t.device != dev:
            t = self._iota_t = torch.arange(n, dtype=torch.int32, device=dev).repeat(L, 1).contiguous()
        return t

    def _fused_optimizer(self, F: int) -> bool:
        """Apply the optimizer to the decoder inside the sparse backward?  Opt-in
        (``module.fuse_optimizer = True``): the decoder blocks then never get a ``.grad`` (so no gradient
        clipping, accumulation or unscaling on them) and are already updated when ``backward()`` returns;
        ``optimizer.step()`` updates the remaining parameters.  Needs the optimizer that
        ``configure_optimizers()`` returned (one parameter group) and d_features % 8 == 0."""
        if not getattr(self.module, "fuse_optimizer", False):
            return False
        opt = getattr(self, "optimizer", None)
        if opt is None:
            raise CltError("module.fuse_optimizer needs the optimizer returned by configure_optimizers()")
        if len(opt.param_groups) != 1:
            raise CltError("module.fuse_optimizer supports a single parameter group")
        if getattr(self, "decoder_updated", False):
            raise CltError("module.fuse_optimizer: a second backward() before optimizer.step() would update the "
                           "decoder twice (gradient accumulation is not available in this mode)")
        return F % 8 == 0 and self.flat.is_packed()


class _StepFunction(torch.autograd.Function):
    """Autograd node of the fused step: forward already ran; backward launches the gradient
    kernels and hands each parameter its slice of the flat gradient buffer."""

    @staticmethod
    def forward(ctx, engine: StepEngine, step_ctx: dict, *params):
        ctx.engine, ctx.step_ctx = engine, step_ctx
        ctx.n = len(params)
        return step_ctx["out"][0].clone()

    @staticmethod
    def backward(ctx, grad_out):
        eng: StepEngine = ctx.engine
        fp = eng.flat
        # After an earlier backward a parameter's .grad usually IS its slice of the flat gradient buffer
        # (autograd keeps the tensor it was handed).  The kernels overwrite that buffer, so gradients that
        # are being accumulated (no zero_grad between two backwards, or zero_grad(set_to_none=False)) are
        # saved first and handed back as the increment: autograd then adds the old values onto the new
        # ones in place and .grad stays the flat slice.
        base = fp.grad.data_ptr()
        aliased = [p.grad is not None and p.grad.data_ptr() == base + 4 * fp.offsets[id(p)] for p in fp.params]
        saved = fp.grad.clone() if any(aliased) else None
        eng.backward(ctx.step_ctx, grad_out)
        updated = set()
        if getattr(eng, "decoder_updated", False):
            updated = {id(w) for w in eng.module.model.decoder.blocks()}
        grads = []
        for p, al in zip(fp.params, aliased):
            gv = fp.view_of(p, fp.grad)
            if id(p) in updated:
                grads.append(None)             # already stepped by the fused decoder backward
            elif al:
                grads.append(fp.view_of(p, saved))
            else:
                # a gradient held in a tensor of the caller's own is accumulated into in place:
                # hand it a copy so the flat buffer can be reused by the next step
                grads.append(gv.clone() if p.grad is not None else gv)
        return (None, None, *grads)


class FusedAdam(torch.optim.Optimizer):
    """Adam / AdamW with the update of ``torch.optim.Adam`` (reference
    clt_lightning.py:339-352), run as one kernel over the engine's flat parameter
    buffer; the same kernel refreshes the bf16 operand copy."""

    def __init__(self, params, engine: StepEngine, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 decoupled=False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=decoupled))
        self.engine = engine
        engine.optimizer = self
        self._step = 0
        self._linked_to = None      # the FlatParams whose moment buffers self.state points into

    # ---- checkpoint resume -------------------------------------------------------------------
    def load_state_dict(self, state_dict):
        """Restore moments and step count (the layout of ``torch.optim.Adam.state_dict()``: per parameter
        ``exp_avg``, ``exp_avg_sq``, ``step``).  The loaded moments are copied into the flat moment
        buffers the kernel reads — at once when the flat buffers exist, else at the first step."""
        super().load_state_dict(state_dict)
        steps = [int(st["step"]) for st in self.state.values() if "step" in st]
        self._step = max(steps) if steps else 0
        self._linked_to = None
        fp = self.engine.flat
        if fp is not None and fp.is_packed():
            self._link_state(fp)

    def _link_state(self, fp: "FlatParams"):
        """Make ``self.state[p]['exp_avg' / 'exp_avg_sq']`` views of the flat moment buffers, carrying over
        moments that live in tensors of their own (loaded from a checkpoint, or created by the
        per-parameter path)."""
        fp.ensure_moments()
        for group in self.param_groups:
            for p in group["params"]:
                if id(p) not in fp.offsets:
                    continue
                st = self.state[p]
                for key, buf in (("exp_avg", fp.exp_avg), ("exp_avg_sq", fp.exp_avg_sq)):
                    view = fp.view_of(p, buf)
                    cur = st.get(key)
                    if cur is None:
                        view.zero_()        # a new optimizer starts from zero moments, whatever an earlier one left
                    elif cur.data_ptr() != view.data_ptr():
                        view.copy_(cur.to(view.dtype))
                    st[key] = view
        self._linked_to = fp

    def _flat_ready(self, group) -> bool:
        fp = self.engine.flat
        if fp is None or not fp.is_packed() or len(group["params"]) != len(fp.params):
            return False
        base = fp.grad.data_ptr()
        for p in group["params"]:
            if id(p) not in fp.offsets or p.grad is None or p.grad.data_ptr() != base + 4 * fp.offsets[id(p)]:
                return False
        return True

    def _step_around_decoder(self, group, args):
        eng, fp = self.engine, self.engine.flat
        blocks = eng.module.model.decoder.blocks()
        skip = {id(w) for w in blocks}
        base = fp.grad.data_ptr()
        for p in group["params"]:
            if id(p) in skip:
                continue
            if p.grad is None or p.grad.data_ptr() != base + 4 * fp.offsets[id(p)]:
                raise CltError("module.fuse_optimizer: the gradients of the other parameters must be the ones the "
                               "fused backward produced (no clipping / replacing of .grad in this mode)")
        if self._linked_to is not fp or fp.exp_avg is None:
            self._link_state(fp)
        o0 = fp.offsets[id(blocks[0])]
        o1 = o0 + sum(_round_up(w.numel()) for w in blocks)
        for lo, hi in ((0, o0), (o1, fp.numel)):
            if hi > lo:
                eng._call("clt_adam_step", fp.flat[lo:hi], fp.grad[lo:hi], fp.exp_avg[lo:hi], fp.exp_avg_sq[lo:hi],
                          fp.shadow[lo:hi] if fp.shadow is not None else None, hi - lo, *args)
        for p in group["params"]:
            self.state[p]["step"] = self._step
        eng.decoder_updated = False

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step += 1
        s = stream_ptr()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            args = (float(group["lr"]), float(b1), float(b2), float(group["eps"]), float(group["weight_decay"]),
                    int(group["decoupled"]), self._step, s)
            if getattr(self.engine, "decoder_updated", False):
                # the sparse backward already stepped the decoder blocks (module.fuse_optimizer): update what
                # lies before and after them in the flat buffer
                self._step_around_decoder(group, args)
                continue
            if len(self.param_groups) == 1 and self._flat_ready(group):
                fp = self.engine.flat
                if self._linked_to is not fp or fp.exp_avg is None:
                    self._link_state(fp)
                self.engine._call("clt_adam_step", fp.flat, fp.grad, fp.exp_avg, fp.exp_avg_sq, fp.shadow, fp.numel,
                                  *args)
                for p in group["params"]:
                    self.state[p]["step"] = self._step
                continue
            # general path: one launch per parameter (still the CUDA kernel)
            fp = self.engine.flat
            for p in group["params"]:
                if p.grad is None:
                    continue
                if not p.is_cuda:
                    raise CltError("FusedAdam updates CUDA parameters only")
                st = self.state[p]
                if "exp_avg" not in st:
                    if fp is not None and id(p) in fp.offsets and fp.is_packed():
                        fp.ensure_moments()
                        st["exp_avg"], st["exp_avg_sq"] = fp.view_of(p, fp.exp_avg), fp.view_of(p, fp.exp_avg_sq)
                    else:
                        st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p)
                st["step"] = self._step
                shadow = None
                if fp is not None and fp.shadow is not None and id(p) in fp.offsets and fp.is_packed():
                    shadow = fp.view_of(p, fp.shadow)
                gr = p.grad.contiguous()
                self.engine._call("clt_adam_step", p.data, gr, st["exp_avg"], st["exp_avg_sq"], shadow, p.numel(),
                                  *args)
        return loss

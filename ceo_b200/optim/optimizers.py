"""Sharded optimizers on flat buffers: AdamW, Lion, Muon and the reference's
Lion+Muon mix, with LR schedules and gradient clipping.

Update rules follow the reference: Lion (src/optim/optimizer.zig:119-142,
kernels/cuda/optim.cu:122-145), AdamW (optim.cu:147-178, CPU ref
src/kernels/optim_kernels.zig:105-137), Muon = heavy-ball momentum, Frobenius normalise,
cubic Newton-Schulz ``Y <- 1/2 Y (3I - Y^T Y)``, ``p -= lr Y`` (optimizer.zig:253-319,
optim.cu:562-623); LionMuon sends 2-D tensors to Muon and the rest to Lion
(optimizer.zig:331-441).  Differences by design: fp32 master weights and moments (the
reference keeps bf16), one fused launch per flat range instead of one per tensor, the clip
scale stays on the device, Newton-Schulz products run on the tcgen05 GEMM.
"""
from __future__ import annotations

import math

import torch

from ..ops import _lib, reference as ref
from ..ops.matmul import gemm
from .flat import FlatParams


# ----------------------------------------------------------------------------- schedules
class LRScheduler:
    """constant | linear_warmup | cosine | linear_warmup_cosine (optimizer.zig:443-522)."""

    def __init__(self, base_lr, min_lr, warmup_steps, total_steps, kind="cosine"):
        if kind not in ("constant", "linear_warmup", "cosine", "linear_warmup_cosine"):
            raise ValueError(kind)
        self.base_lr, self.min_lr = float(base_lr), float(min_lr)
        self.warmup_steps, self.total_steps = int(warmup_steps), int(total_steps)
        self.kind = kind
        self.current_step = 0

    def _warm(self):
        if self.warmup_steps == 0 or self.current_step >= self.warmup_steps:
            return self.base_lr
        return self.base_lr * max(1, self.current_step) / self.warmup_steps

    def _cos(self, step, total):
        if total == 0:
            return self.min_lr
        prog = min(max(step / total, 0.0), 1.0)
        return self.min_lr + (self.base_lr - self.min_lr) * 0.5 * (1.0 + math.cos(math.pi * prog))

    def get_lr(self) -> float:
        if self.kind == "constant":
            return self.base_lr
        if self.kind == "linear_warmup":
            return self._warm()
        if self.kind == "cosine":
            return self._cos(self.current_step, self.total_steps)
        if self.current_step < self.warmup_steps:
            return self._warm()
        total = self.total_steps - self.warmup_steps if self.total_steps > self.warmup_steps else 1
        return self._cos(max(0, self.current_step - self.warmup_steps), total)

    def step(self):
        self.current_step += 1

    def state_dict(self):
        return {"current_step": self.current_step}

    def load_state_dict(self, d):
        self.current_step = int(d["current_step"])


class GradientClipper:
    """Clip by global norm or by value on a list of tensors (optimizer.zig:524-594)."""

    def __init__(self, max_norm: float = 0.0, clip_value: float = 0.0):
        self.max_norm, self.clip_value = max_norm, clip_value

    def clip(self, grads) -> float:
        grads = [g for g in grads if g is not None]
        if self.clip_value > 0:
            for g in grads:
                g.clamp_(-self.clip_value, self.clip_value)
        total = math.sqrt(sum(float(g.float().pow(2).sum()) for g in grads))
        if self.max_norm > 0:
            s = ref.clip_scale(total, self.max_norm)
            if s != 1.0:
                for g in grads:
                    g.mul_(s)
        return total


# ---------------------------------------------------------------------------- optimizers
class ShardedOptimizer:
    """One step = reduce-scatter grads -> global norm -> clip -> update owned slice ->
    all-gather parameters.  ``comm`` provides the collectives (None = single process)."""

    def __init__(self, flat: FlatParams, kind: str = "adamw", *, weight_decay=0.1,
                 max_grad_norm=1.0, betas=(0.9, 0.95), eps=1e-8, lion_betas=(0.95, 0.98),
                 muon_momentum=0.95, muon_iterations=5, muon_ns="cubic", comm=None):
        if kind not in ("adamw", "lion", "muon", "lion_muon"):
            raise ValueError(kind)
        self.flat, self.kind, self.comm = flat, kind, comm
        self.wd, self.max_norm = weight_decay, max_grad_norm
        self.betas, self.eps, self.lion_betas = betas, eps, lion_betas
        self.muon_momentum, self.muon_iterations, self.muon_ns = \
            muon_momentum, muon_iterations, muon_ns
        self.step_count = 0
        dev = flat.device
        self.cuda = dev.type == "cuda"
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._side_state = {}
        self._muon_state = {}
        # Tensor parallelism: the squared norm is also summed over `extra_norm_group`, and the
        # parameters every rank of that group holds in full (`replicated_names`) count once.
        self.extra_norm_group = None
        self.replicated_names: set = set()
        self.use_fused_step = True
        # set by the engine when the bucket reductions of the backward pass have already
        # reduce-scattered this step's gradients (ZeRO stage 2 / 3)
        self.grads_reduced = False
        self.uses_matrices = kind in ("muon", "lion_muon")
        if self.uses_matrices:
            self._matrix_segs = [s for s in flat.segments if len(s.shape) == 2 and s.decay]
        else:
            self._matrix_segs = []

    # -------------------------------------------------------------- gradient plumbing
    def _world(self):
        return self.flat.world

    def fused_step_available(self) -> bool:
        """True when one peer-memory kernel does the whole step (``FusedComm.zero_step``)."""
        f = self.flat
        return (self.use_fused_step and self.kind in ("adamw", "lion") and self._world() > 1
                and getattr(self.comm, "fused", False) and f.grads_symm is not None
                and f.param_dtype == torch.bfloat16 and f.grads.dtype == torch.float32)

    def _reduce_grads(self):
        """Returns the fp32 gradient tensor the update reads, aligned with the owned slice."""
        f = self.flat
        if self._world() == 1:
            return f.grads
        if self.uses_matrices:
            self.comm.all_reduce(f.grads)
            return f.grads[f.lo:f.hi]
        return self.comm.reduce_scatter(f.grads, f.lo, f.hi)

    def _side_grads(self):
        out = []
        for _, p in self.flat.side:
            if p.grad is not None and p.requires_grad:
                if self._world() > 1:
                    self.comm.all_reduce(p.grad)
                out.append(p.grad)
        return out

    def _global_norm(self, gshard, side, gscale):
        """Leaves the clip scale in ``self._scale`` (device) and the norm in ``self._norm``."""
        if self.cuda:
            L = _lib.lib()
            sc = _lib.scratch(gshard.device, L.ceo_sumsq_blocks(gshard.numel()), "sumsq")
            _lib.check(L.ceo_sumsq(gshard.data_ptr(), int(gshard.dtype == torch.float32),
                                   gshard.numel(), self._sumsq.data_ptr(), 0, sc.data_ptr(),
                                   _lib.stream()), "ceo_sumsq")
            if self._world() > 1:
                self.comm.all_reduce(self._sumsq)
            for g in side:
                self._sumsq += g.float().pow(2).sum()
            if self.extra_norm_group is not None:
                import torch.distributed as dist
                tpw = dist.get_world_size(self.extra_norm_group)
                f = self.flat
                rep = torch.zeros_like(self._sumsq)
                for seg in f.segments:
                    if seg.name in self.replicated_names:
                        a = max(seg.offset, f.lo) - f.lo
                        b = min(seg.offset + seg.numel, f.hi) - f.lo
                        if b > a:
                            rep += gshard[a:b].float().pow(2).sum()
                if self._world() > 1:
                    self.comm.all_reduce(rep)
                for g in side:
                    rep += g.float().pow(2).sum()
                self._sumsq -= rep * (1.0 - 1.0 / tpw)
                dist.all_reduce(self._sumsq, group=self.extra_norm_group)
            self._sumsq *= gscale * gscale
            _lib.check(L.ceo_clip_scale(self._sumsq.data_ptr(), float(self.max_norm),
                                        self._scale.data_ptr(), self._norm.data_ptr(),
                                        _lib.stream()), "ceo_clip_scale")
        else:
            ss = gshard.float().pow(2).sum()
            if self._world() > 1:
                self.comm.all_reduce(ss)
            for g in side:
                ss = ss + g.float().pow(2).sum()
            nrm = float(ss.sqrt()) * gscale
            self._norm.fill_(nrm)
            self._scale.fill_(ref.clip_scale(nrm, self.max_norm))

    # ------------------------------------------------------------------ update rules
    def _adamw_range(self, g, a, b, decay, lr, gscale):
        f = self.flat
        m, v = f.buffer("exp_avg"), f.buffer("exp_avg_sq")
        wd = self.wd if decay else 0.0
        shadow = f.params[f.lo + a:f.lo + b]
        if self.cuda:
            sh = shadow.data_ptr() if f.param_dtype == torch.bfloat16 else None
            _lib.check(_lib.lib().ceo_adamw_step(
                f.master[a:b].data_ptr(), m[a:b].data_ptr(), v[a:b].data_ptr(), g[a:b].data_ptr(),
                int(g.dtype == torch.float32), sh, b - a, float(lr), self.betas[0], self.betas[1],
                self.eps, wd, self.step_count, self._scale.data_ptr(), float(gscale), 0,
                _lib.stream()), "ceo_adamw_step")
            if sh is None:
                shadow.copy_(f.master[a:b])
        else:
            gg = g[a:b].float() * (gscale * float(self._scale))
            ref.adamw_step(f.master[a:b], m[a:b], v[a:b], gg, lr, self.betas[0], self.betas[1],
                           self.eps, wd, self.step_count)
            shadow.copy_(f.master[a:b])

    def _lion_range(self, g, a, b, decay, lr, gscale):
        f = self.flat
        m = f.buffer("momentum")
        wd = self.wd if decay else 0.0
        shadow = f.params[f.lo + a:f.lo + b]
        if self.cuda:
            sh = shadow.data_ptr() if f.param_dtype == torch.bfloat16 else None
            _lib.check(_lib.lib().ceo_lion_step(
                f.master[a:b].data_ptr(), m[a:b].data_ptr(), g[a:b].data_ptr(),
                int(g.dtype == torch.float32), sh, b - a, float(lr), self.lion_betas[0],
                self.lion_betas[1], wd, self._scale.data_ptr(), float(gscale), 0, _lib.stream()),
                "ceo_lion_step")
            if sh is None:
                shadow.copy_(f.master[a:b])
        else:
            gg = g[a:b].float() * (gscale * float(self._scale))
            ref.lion_step(f.master[a:b], m[a:b], gg, lr, self.lion_betas[0], self.lion_betas[1], wd)
            shadow.copy_(f.master[a:b])

    def _newton_schulz(self, y):
        """y: (n, m) bf16, Frobenius-normalised.  Returns the orthogonalised matrix (bf16)."""
        n, m = y.shape
        small_left = n <= m
        L = _lib.lib()
        for _ in range(self.muon_iterations):
            a = gemm(y, y) if small_left else gemm(y, y, a_mn=True, b_mn=True)
            k = a.shape[0]
            if self.muon_ns == "cubic":
                _lib.check(L.ceo_ns_poly(a.data_ptr(), None, k, 1.5, -0.5, 0.0, _lib.stream()),
                           "ceo_ns_poly")
            else:
                a2 = gemm(a, a)
                _lib.check(L.ceo_ns_poly(a.data_ptr(), a2.data_ptr(), k, 3.4445, -4.7750, 2.0315,
                                         _lib.stream()), "ceo_ns_poly")
            y = gemm(a, y, b_mn=True) if small_left else gemm(y, a)
        return y

    def _muon_matrix(self, seg, g_full, lr, gscale):
        """Muon on one whole matrix (this rank owns it).  g_full: the full fp32 grad buffer."""
        f = self.flat
        st = self._muon_state.get(seg.name)
        p = f.params[seg.offset:seg.offset + seg.numel]
        if st is None:
            st = {"momentum": torch.zeros(seg.numel, dtype=torch.float32, device=f.device),
                  "master": p.float().clone()}
            self._muon_state[seg.name] = st
        g = g_full[seg.offset:seg.offset + seg.numel]
        if self.cuda and f.param_dtype == torch.bfloat16:
            L = _lib.lib()
            sc = _lib.scratch(f.device, L.ceo_sumsq_blocks(seg.numel), "sumsq")
            ss = torch.empty(1, dtype=torch.float32, device=f.device)
            _lib.check(L.ceo_muon_momentum(st["momentum"].data_ptr(), g.data_ptr(),
                                           int(g.dtype == torch.float32), seg.numel,
                                           self.muon_momentum, self._scale.data_ptr(),
                                           float(gscale), 0, ss.data_ptr(), sc.data_ptr(),
                                           _lib.stream()), "ceo_muon_momentum")
            y = torch.empty(seg.shape, dtype=torch.bfloat16, device=f.device)
            _lib.check(L.ceo_muon_normalize(st["momentum"].data_ptr(), ss.data_ptr(), y.data_ptr(),
                                            seg.numel, 1e-7, _lib.stream()), "ceo_muon_normalize")
            y = self._newton_schulz(y)
            _lib.check(L.ceo_muon_apply(st["master"].data_ptr(), y.data_ptr(), p.data_ptr(),
                                        seg.numel, float(lr), 0.0, 1.0, self._scale.data_ptr(),
                                        _lib.stream()), "ceo_muon_apply")
        else:
            st["momentum"].mul_(self.muon_momentum).add_(g.float() * (gscale * float(self._scale)))
            mm = st["momentum"].view(seg.shape)
            y = ref.newton_schulz_cubic(mm, self.muon_iterations) if self.muon_ns == "cubic" \
                else ref.newton_schulz_quintic(mm, self.muon_iterations)
            st["master"].sub_(lr * y.reshape(-1))
            p.copy_(st["master"])

    def _side_update(self, side, lr, gscale):
        """The few parameters outside the flat buffers (fp32 scalars).  The clip scale stays a
        device tensor (no host read); a scale of exactly zero marks a skipped step, which
        leaves parameter and moments as they were."""
        if not side:
            return
        sc = self._scale.reshape(()) if self.cuda else self._scale.reshape(()).clone()
        skip = sc == 0
        live = [(n, p) for n, p in self.flat.side if p.grad is not None and p.requires_grad]
        for (name, p), g in zip(live, side):
            st = self._side_state.setdefault(name, {"m": torch.zeros_like(p, dtype=torch.float32),
                                                    "v": torch.zeros_like(p, dtype=torch.float32)})
            gg = torch.where(skip, torch.zeros_like(g, dtype=torch.float32), g.float() * gscale * sc)
            pf, m, v = p.data.float(), st["m"].clone(), st["v"].clone()
            if self.kind == "adamw":
                ref.adamw_step(pf, m, v, gg, lr, self.betas[0], self.betas[1], self.eps, 0.0,
                               self.step_count)
            else:
                ref.lion_step(pf, m, gg, lr, self.lion_betas[0], self.lion_betas[1], 0.0)
            p.data.copy_(torch.where(skip, p.data.float(), pf))
            st["m"].copy_(torch.where(skip, st["m"], m))
            st["v"].copy_(torch.where(skip, st["v"], v))

    # -------------------------------------------------------------------------- step
    def step(self, lr: float, grad_scale: float = 1.0) -> torch.Tensor:
        """Applies one update from the accumulated ``main_grad`` buffers (scaled by
        ``grad_scale``, e.g. 1/accumulation steps) and zeroes them.  Returns the global
        gradient norm as a device scalar (no host synchronisation)."""
        f = self.flat
        self.step_count += 1
        if self.fused_step_available():
            # one kernel: reduce-scatter (unless the bucket reductions of the backward pass
            # already did it) + clip + AdamW / Lion + all-gather + zero-grad over NVLink
            side = self._side_grads()
            adam = self.kind == "adamw"
            norm = self.comm.zero_step(
                f, f.buffer("exp_avg" if adam else "momentum"),
                f.buffer("exp_avg_sq") if adam else None, lr=lr,
                betas=self.betas if adam else self.lion_betas, eps=self.eps,
                weight_decay=self.wd, step=self.step_count, grad_scale=grad_scale,
                max_norm=self.max_norm, kind=self.kind, do_reduce=not self.grads_reduced,
                clip_out=self._scale)
            self.grads_reduced = False
            self._side_update(side, lr, grad_scale)
            for _, p in f.side:
                p.grad = None
            return norm
        if f.layout != "contiguous":
            raise RuntimeError("the segment ownership layout needs the fused optimizer step "
                               "(peer-memory communicator, AdamW or Lion, bf16 parameters)")
        g = self._reduce_grads()
        side = self._side_grads()
        self._global_norm(g, side, grad_scale)
        if not self.cuda and float(self._scale) == 0.0:
            # non-finite gradient norm: skip the step (the CUDA kernels test the device scale)
            f.zero_grads()
            return self._norm
        if self.uses_matrices:
            # Tensors that are not Muon matrices take Lion (the reference's Muon class only
            # handles matrices: optimizer.zig:331-441), on the slice this rank owns; the
            # all-gather then publishes them.  Muon matrices are owned whole, round-robin, and
            # broadcast by their owner afterwards (the gather would overwrite them otherwise).
            mat_names = {s.name for s in self._matrix_segs}
            gs = g if g.numel() == f.shard else g[f.lo:f.hi]
            for seg in f.segments:
                if seg.name in mat_names:
                    continue
                a = max(seg.offset, f.lo) - f.lo
                b = min(seg.offset + seg.numel, f.hi) - f.lo
                if b > a:
                    self._lion_range(gs, a, b, seg.decay, lr, grad_scale)
            if self._world() > 1:
                self.comm.all_gather(f.params, f.lo, f.hi)
            for i, seg in enumerate(self._matrix_segs):
                if i % self._world() == f.rank:
                    self._muon_matrix(seg, f.grads, lr, grad_scale)
            if self._world() > 1:
                self.comm.broadcast_segments(f, self._matrix_segs)
        else:
            gs = g if g.numel() == f.shard else g[f.lo:f.hi]
            for a, b, decay in f.owned_ranges():
                if self.kind == "adamw":
                    self._adamw_range(gs, a, b, decay, lr, grad_scale)
                else:
                    self._lion_range(gs, a, b, decay, lr, grad_scale)
            if self._world() > 1:
                self.comm.all_gather(f.params, f.lo, f.hi)
        self._side_update(side, lr, grad_scale)
        f.zero_grads()
        return self._norm

    # -------------------------------------------------------------------- state I/O
    def state_dict(self):
        return {"step": self.step_count, "flat": self.flat.optimizer_state(),
                "muon": self._muon_state, "side": self._side_state}

    def load_state_dict(self, d):
        self.step_count = int(d["step"])
        self.flat.load_optimizer_state(d["flat"])
        for k, st in d.get("muon", {}).items():
            self._muon_state[k] = {n: t.to(self.flat.device) for n, t in st.items()}
        for k, st in d.get("side", {}).items():
            self._side_state[k] = {n: t.to(self.flat.device) for n, t in st.items()}


def build_optimizer(flat: FlatParams, tcfg, comm=None) -> ShardedOptimizer:
    """From a ``TrainingConfig``."""
    return ShardedOptimizer(
        flat, tcfg.optimizer, weight_decay=tcfg.weight_decay, max_grad_norm=tcfg.gradient_clip,
        betas=(tcfg.adam_beta1, tcfg.adam_beta2), eps=tcfg.adam_eps,
        lion_betas=(tcfg.lion_beta1, tcfg.lion_beta2), muon_momentum=tcfg.muon_momentum,
        muon_iterations=tcfg.muon_iterations, comm=comm)

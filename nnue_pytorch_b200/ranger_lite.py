"""`RangerLite`: Adam + positive-negative momentum + lookahead, with the whole
per-tensor update (and the lookahead merge, when one is due) in one kernel.

Mirrors the class of the same name in model/optimizers/ranger_lite.py:216-808
of the reference project: constructor arguments, `step`, `train`/`eval`
weight swap and the state keys `step, grad_ma, variance_ma, neg_grad_ma,
lookahead_params`, so checkpoints load both ways.  The arithmetic follows the
reference's Python path (:592-742).

What differs:
  * CUDA float32 parameters only; there is no CPU path.
  * touched-rows-only update for large 2-D tables: a row that has never
    received a non-zero gradient is skipped, which leaves exactly the bits the
    full update would write (all of its moments are zero).  Used only when
    that identity holds: no weight decay on the group and lookahead blending
    of 0.5 (or no lookahead).
  * `grad_scale`: an optional device scalar every gradient is multiplied by
    inside the kernel, so the trainer's gradient clipping
    (trainer/engine.py:308-311) needs no pass of its own.
  * norm-loss and the legacy scoping mode (`optimizer_name=ranger21`) run as
    plain torch tensor ops, like the reference does for them.
"""

from __future__ import annotations

import collections.abc
import math

import torch

from . import _launch

_ROW_TABLE_MIN_ROWS = 1024


class RangerLite(torch.optim.Optimizer):
    def __init__(
        self,
        params,
        lr=1.0,
        weight_decay=0.0,
        betas=(0.9, 0.999),
        eps=1e-7,
        pnm_activate=True,
        pnm_momentum=1.0,
        lookahead_active=True,
        lookahead_mergetime=5,
        lookahead_blending_alpha=0.5,
        normloss_active=True,
        normloss_factor=1e-4,
        use_legacy_scoping_bug=False,
        touched_rows_only=True,
    ):
        defaults = {
            "lr": lr,
            "weight_decay": weight_decay,
            "betas": betas,
            "eps": eps,
            "pnm_momentum": pnm_momentum,
            "normloss_factor": normloss_factor,
        }
        super().__init__(params, defaults)
        self.lookahead_active = lookahead_active
        self.lookahead_mergetime = lookahead_mergetime
        self.lookahead_alpha = lookahead_blending_alpha
        self.lookahead_step = 0
        self.pnm_active = pnm_activate
        self.normloss_active = normloss_active
        self.eps = eps
        self.param_size = 0
        self.use_legacy_scoping_bug = use_legacy_scoping_bug
        self.touched_rows_only = touched_rows_only
        self.grad_scale: torch.Tensor | None = None
        self._row_active: dict[int, torch.Tensor] = {}
        self._state_was_loaded = False

    # ------------------------------------------------------------------
    def _init_state(self, p):
        state = self.state[p]
        if len(state) == 0:
            state["step"] = 0
            state["grad_ma"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            state["variance_ma"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            if self.lookahead_active:
                state["lookahead_params"] = torch.clone(p.data)
            if self.pnm_active:
                state["neg_grad_ma"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return state

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        # moments of unknown history: every row has to be treated as touched
        self._state_was_loaded = True
        self._row_active.clear()

    def _rows_flag(self, p, group):
        if not self.touched_rows_only or p.dim() != 2 or p.shape[0] < _ROW_TABLE_MIN_ROWS:
            return None
        if p.shape[1] % 4 != 0:
            return None
        if group.get("weight_decay", 0.0) != 0.0:
            return None
        if self.lookahead_active and self.lookahead_alpha != 0.5:
            return None
        flag = self._row_active.get(id(p))
        if flag is None or flag.device != p.device:
            fill = 1 if self._state_was_loaded else 0
            flag = torch.full((p.shape[0],), fill, dtype=torch.uint8, device=p.device)
            self._row_active[id(p)] = flag
        return flag

    def _check_param(self, p):
        if p.grad.is_sparse:
            raise RuntimeError("Sparse matrix not supported")
        if not p.is_cuda or p.dtype != torch.float32:
            raise RuntimeError(
                "nnue_pytorch_b200.RangerLite updates CUDA float32 parameters only (there is no CPU path)"
            )
        if not p.is_contiguous():
            raise RuntimeError("RangerLite needs contiguous parameters")

    def _hparams(self, group, step, merge, phase, wd_keep=1.0):
        beta1, beta2 = group["betas"]
        f = group["pnm_momentum"]
        if self.pnm_active:
            effective = ((step + 1) // 2) * 2
            bc1 = 1 - beta1**effective
            mom, one_minus_mom = beta1**2, 1 - beta1**2
        else:
            bc1 = 1 - beta1**step
            mom, one_minus_mom = beta1, 1 - beta1
        return _launch.hparams_struct(
            beta2=beta2,
            one_minus_beta2=1 - beta2,
            mom=mom,
            one_minus_mom=one_minus_mom,
            one_plus_f=1 + f,
            f=f,
            noise_norm_inv=1 / math.sqrt((1 + f) ** 2 + f**2),
            step_size=group["lr"] / bc1,
            bc2_sqrt=math.sqrt(1 - beta2**step),
            eps=group["eps"],
            wd_keep=wd_keep,
            alpha=self.lookahead_alpha,
            one_minus_alpha=1.0 - self.lookahead_alpha,
            use_pnm=int(self.pnm_active),
            step_is_odd=step % 2,
            do_merge=int(merge),
            phase=phase,
        )

    # ------------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None and isinstance(closure, collections.abc.Callable):
            with torch.enable_grad():
                loss = closure()
        active = [(p, g) for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not active:
            return loss
        if self.normloss_active or self.use_legacy_scoping_bug:
            self._step_tensor_ops()
            self._drop_table_caches(active, ())
            return loss

        for p, _ in active:
            self._check_param(p)
            self._init_state(p)["step"] += 1
        merge = False
        if self.lookahead_active:
            self.lookahead_step += 1
            if self.lookahead_step >= self.lookahead_mergetime:
                self.lookahead_step = 0
                merge = True

        decayed = any(g.get("weight_decay", 0.0) != 0.0 for g in self.param_groups)
        var_norm = None
        if decayed:
            # stable weight decay: second moments first, then their global debiased mean
            total = None
            count = 0
            for p, group in active:
                st = self.state[p]
                hp = self._hparams(group, st["step"], False, phase=1)
                _launch.ranger_update(p.data, self._grad(p), st["grad_ma"], st.get("neg_grad_ma"),
                                      st["variance_ma"], None, None, self.grad_scale, hp)
                part = st["variance_ma"].sum() / (1 - group["betas"][1] ** st["step"])
                total = part if total is None else total + part
                count += p.numel()
            if not self.param_size:
                self.param_size = count
            var_norm = torch.sqrt(total / self.param_size).clamp_min(self.eps).item()

        small = []  # tensors without row flags share launches
        emitted = []  # parameters whose integer table (kept by the forward) the update kernel rewrote
        for p, group in active:
            st = self.state[p]
            wd = group.get("weight_decay", 0.0)
            wd_keep = 1.0 - (wd * group["lr"] / var_norm) if (wd and var_norm is not None) else 1.0
            hp = self._hparams(group, st["step"], merge, phase=2 if decayed else 0, wd_keep=wd_keep)
            rows = self._rows_flag(p, group)
            args = (p.data, self._grad(p), st["grad_ma"], st.get("neg_grad_ma"), st["variance_ma"],
                    st.get("lookahead_params"))
            if rows is None and p.numel() <= self.MULTI_TENSOR_LIMIT and p.data.is_contiguous():
                small.append(args + (hp,))
            else:
                # a feature-transformer table whose integer form the forward keeps: write the new one in the same pass
                cache = getattr(p, "_nnue_q16_cache", None)
                emit = cache.emit_struct(p) if cache is not None else None
                _launch.ranger_update(*args, rows, self.grad_scale, hp, emit=emit)
                if emit is not None:
                    cache.mark(p)
                    emitted.append(p)
        by_device: dict = {}
        for item in small:
            by_device.setdefault(item[0].device, []).append(item)
        for items in by_device.values():
            _launch.ranger_update_multi(items, self.grad_scale)
        self._drop_table_caches(active, emitted)
        return loss

    @staticmethod
    def _drop_table_caches(active, emitted) -> None:
        """The kernels write parameters through raw pointers, which torch's version counter does not see:
        every integer table a forward keeps for a parameter updated here is stale unless the update kernel
        rewrote it."""
        keep = {id(p) for p in emitted}
        for p, _ in active:
            cache = getattr(p, "_nnue_q16_cache", None)
            if cache is not None and id(p) not in keep:
                cache.invalidate()

    MULTI_TENSOR_LIMIT = 1 << 22  # elements; larger tensors get a launch of their own

    @staticmethod
    def _grad(p):
        g = p.grad
        return g if g.is_contiguous() else g.contiguous()

    # ------------------------------------------------------------------
    def _step_tensor_ops(self):
        """Norm-loss / legacy-scoping variants, as tensor ops on the parameters'
        device (same sequence as the reference's Python path)."""
        first = next(p for g in self.param_groups for p in g["params"] if p.grad is not None)
        variance_sum = torch.zeros(1, device=first.device)
        param_size = 0
        leaked = None
        for group in self.param_groups:
            beta2 = group["betas"][1]
            for p in group["params"]:
                if p.grad is None:
                    continue
                leaked = p
                param_size += p.numel()
                st = self._init_state(p)
                st["step"] += 1
                g = p.grad if self.grad_scale is None else p.grad * self.grad_scale
                st["variance_ma"].mul_(beta2).addcmul_(g, g, value=1 - beta2)
                variance_sum += (st["variance_ma"] / (1 - beta2 ** st["step"])).sum()
        if not self.param_size:
            self.param_size = param_size
        var_norm = torch.sqrt(variance_sum / self.param_size).clamp_min(self.eps)

        def regularise(t, group):
            if group["weight_decay"]:
                t.data.mul_(1 - group["weight_decay"] * group["lr"] / var_norm)
            if self.normloss_active:
                n = t.data.norm(p=2.0) if t.dim() <= 1 else t.data.norm(dim=tuple(range(1, t.dim())), keepdim=True, p=2.0)
                t.data.mul_(1 - group["lr"] * 2 * group["normloss_factor"] * (1 - torch.div(1, n + self.eps)))

        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            f = group["pnm_momentum"]
            if self.use_legacy_scoping_bug and leaked is not None:
                regularise(leaked, group)
            for p in group["params"]:
                if self.use_legacy_scoping_bug:
                    leaked = p
                if p.grad is None:
                    continue
                st = self.state[p]
                if not self.use_legacy_scoping_bug:
                    regularise(p, group)
                g = p.grad if self.grad_scale is None else p.grad * self.grad_scale
                step = st["step"]
                denom = (st["variance_ma"].sqrt() / math.sqrt(1 - beta2**step)).add_(group["eps"])
                if self.pnm_active:
                    pos, neg = (st["grad_ma"], st["neg_grad_ma"]) if step % 2 == 1 else (st["neg_grad_ma"], st["grad_ma"])
                    pos.mul_(beta1**2).add_(g, alpha=1 - beta1**2)
                    if self.use_legacy_scoping_bug:
                        bc1 = 1 - beta1**step
                        norm = math.sqrt((1 + beta2) ** 2 + beta2**2)
                    else:
                        bc1 = 1 - beta1 ** (((step + 1) // 2) * 2)
                        norm = math.sqrt((1 + f) ** 2 + f**2)
                    upd = pos.mul(1 + f).add(neg, alpha=-f).mul(1 / norm)
                else:
                    bc1 = 1 - beta1**step
                    st["grad_ma"].mul_(beta1).add_(g, alpha=1 - beta1)
                    upd = st["grad_ma"]
                p.addcdiv_(upd, denom, value=-(group["lr"] / bc1))
        if self.lookahead_active:
            self.lookahead_process_step()

    def lookahead_process_step(self):
        """Every `lookahead_mergetime`-th call blends the fast weights toward the
        slow copy and stores the result as the new slow copy."""
        if not self.lookahead_active:
            return
        self.lookahead_step += 1
        if self.lookahead_step >= self.lookahead_mergetime:
            self.lookahead_step = 0
            for group in self.param_groups:
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    slow = self.state[p]["lookahead_params"]
                    if p.is_cuda and p.dtype == torch.float32 and p.is_contiguous():
                        _launch.lookahead_merge(p.data, slow, self.lookahead_alpha)
                    else:
                        p.data.mul_(self.lookahead_alpha).add_(slow, alpha=1.0 - self.lookahead_alpha)
                        slow.copy_(p.data)

    # ------------------------------------------------------------------
    def train(self):
        if self.lookahead_active:
            self.restore_for_training()

    def eval(self):
        if self.lookahead_active:
            self.swap_for_inference()

    def swap_for_inference(self):
        """Put the slow weights into the parameters (pointer swap, idempotent)."""
        if not self.lookahead_active:
            return
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                if "lookahead_params" in st and "is_swapped" not in st:
                    p.data, st["lookahead_params"] = st["lookahead_params"], p.data
                    st["is_swapped"] = True

    def restore_for_training(self):
        """Undo `swap_for_inference`; whatever the parameters hold now becomes the slow copy."""
        if not self.lookahead_active:
            return
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                if "is_swapped" in st:
                    p.data, st["lookahead_params"] = st["lookahead_params"], p.data
                    del st["is_swapped"]

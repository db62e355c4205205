"""Semi-synchronous training across replica groups: LocalSGD and (streaming) DiLoCo.

* ``LocalSGD``: every ``sync_every`` inner steps the replicas average their parameters.
* ``DiLoCo``: each model *fragment* keeps a copy of the last globally agreed parameters; every ``sync_every`` steps
  (fragments staggered round-robin) the pseudo-gradient ``global - local`` is averaged over live replicas
  (optionally after bf16 quantisation), an outer optimizer (SGD, lr 0.7, Nesterov momentum 0.9 by default) updates the
  global copy, and the local parameters are set to ``alpha * local + (1 - alpha) * global``.

Both are context managers wrapping the training loop and hook the inner optimizer's ``step``; a sync happens only
inside a committed quorum. Counterpart of the torchft ``local_sgd`` module used by
torchtitan/experiments/ft/manager.py:156-216 and diloco/utils.py:14-135.
"""

from __future__ import annotations

import torch
import torch.nn as nn


def _local(p):
    return p.to_local() if hasattr(p, "to_local") else p


class _StepHook:
    def __init__(self, optimizer, fn):
        self.handles = []
        opts = getattr(optimizer, "optimizers", [optimizer])
        for o in opts:
            self.handles.append(o.register_step_post_hook(lambda *_: fn()))
        self._fired = 0
        self._n = len(opts)

    def remove(self):
        for h in self.handles:
            h.remove()


class LocalSGD:
    def __init__(self, manager, model: nn.Module, optimizer, sync_every: int):
        assert sync_every >= 1
        self.manager, self.model, self.optimizer, self.sync_every = manager, model, optimizer, sync_every
        self._local_step = 0
        self._hook = None
        self._calls = 0
        self._n_opts = len(getattr(optimizer, "optimizers", [optimizer]))

    def __enter__(self):
        self._hook = _StepHook(self.optimizer, self._on_step)
        return self

    def __exit__(self, *exc):
        self._hook.remove()
        return False

    def _on_step(self):
        self._calls += 1
        if self._calls % self._n_opts:
            return
        self._local_step += 1
        if self._local_step >= self.sync_every:
            self.sync()

    def sync(self) -> None:
        self.manager.start_quorum()
        with torch.no_grad():
            for p in self.model.parameters():
                self.manager.allreduce(_local(p).data, average=True)
        if self.manager.should_commit():
            self._local_step = 0


class DiLoCo:
    def __init__(self, manager, model_fragments: list[nn.Module], inner_optimizer, outer_optimizer=None, sync_every: int = 1,
                 should_quantize: bool = False, fragment_sync_delay: int = 0, fragment_update_alpha: float = 0.0):
        n = len(model_fragments)
        assert sync_every >= n and sync_every % n == 0, "sync_every must be a multiple of the number of fragments"
        assert fragment_sync_delay < sync_every // n
        self.manager, self.fragments, self.inner = manager, model_fragments, inner_optimizer
        self.sync_every, self.quantize, self.delay, self.alpha = sync_every, should_quantize, fragment_sync_delay, fragment_update_alpha
        self.globals = [[_local(p).detach().clone() for p in f.parameters()] for f in model_fragments]
        if outer_optimizer is None:
            outer_optimizer = [torch.optim.SGD(g, lr=0.7, momentum=0.9, nesterov=True) for g in self.globals]
        elif not isinstance(outer_optimizer, (list, tuple)):
            outer_optimizer = [outer_optimizer]
        # outer optimizers must act on the *global* copies
        self.outer = []
        for g, o in zip(self.globals, outer_optimizer):
            defaults = {k: v for k, v in o.defaults.items()}
            self.outer.append(type(o)(g, **{k: defaults[k] for k in ("lr", "momentum", "nesterov") if k in defaults}))
        self._local_step = 0
        self._calls = 0
        self._n_opts = len(getattr(inner_optimizer, "optimizers", [inner_optimizer]))
        self._hook = None
        self.syncs = 0

    def __enter__(self):
        self._hook = _StepHook(self.inner, self._on_step)
        return self

    def __exit__(self, *exc):
        self._hook.remove()
        return False

    def _on_step(self):
        self._calls += 1
        if self._calls % self._n_opts:
            return
        self._local_step += 1
        per = self.sync_every // len(self.fragments)
        if self._local_step % per == 0:
            frag = (self._local_step // per - 1) % len(self.fragments)
            self.sync_fragment(frag)
        if self._local_step >= self.sync_every:
            self._local_step = 0

    def sync_fragment(self, i: int) -> None:
        self.manager.start_quorum()
        params = [_local(p) for p in self.fragments[i].parameters()]
        with torch.no_grad():
            for g, p in zip(self.globals[i], params):
                pseudo = g - p.data
                if self.quantize:
                    pseudo = pseudo.to(torch.bfloat16)
                    self.manager.allreduce(pseudo, average=True)
                    pseudo = pseudo.to(g.dtype)
                else:
                    self.manager.allreduce(pseudo, average=True)
                g.grad = pseudo
        if self.manager.should_commit():
            self.outer[i].step()
            with torch.no_grad():
                for g, p in zip(self.globals[i], params):
                    p.data.mul_(self.alpha).add_(g, alpha=1 - self.alpha)
            self.syncs += 1
        else:
            with torch.no_grad():   # an uncommitted sync leaves the replica on the last agreed parameters
                for g, p in zip(self.globals[i], params):
                    p.data.copy_(g)
        for g in self.globals[i]:
            g.grad = None

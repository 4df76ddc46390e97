"""``FlatNadam``: all weights, gradients and optimiser state in flat device buffers, one C-ABI
call (two kernel launches) per step.

The reference builds its update from ``tf.clip_by_global_norm(grads, 5.0)``,
``tf.contrib.opt.NadamOptimizer(lr, 0.9, 0.999, 1e-8)`` and
``tf.train.ExponentialMovingAverage(0.9999, global_step)``
(``khan/training/trainer_multi_tower.py:261-266,421-427``).  Here the parameter tensors are
re-pointed at slices of one buffer, their ``.grad`` at slices of another, so that

* ``zero_grad`` is one memset,
* the multi-GPU average is one all-reduce of the gradient buffer with no packing,
* ``step`` is ``ani_nadam_step_f32`` and can sit inside a CUDA graph (the learning rate and the
  step counter live in device memory).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib


class FlatNadam:
    def __init__(self, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, clip_norm=5.0, ema_decay=0.9999):
        self.params = list(params)
        if not self.params:
            raise ValueError("no parameters")
        dev = self.params[0].device
        if dev.type != "cuda" or any(p.dtype != torch.float32 or p.device != dev for p in self.params):
            raise ValueError("FlatNadam needs float32 CUDA parameters on one device")
        self.device = dev
        sizes = [p.numel() for p in self.params]
        self.offsets = [0]
        for s in sizes:
            self.offsets.append(self.offsets[-1] + -(-s // 4) * 4)     # every slice 16-byte aligned
        n = self.offsets[-1]
        self.n = n
        self.flat_params = torch.zeros(n, dtype=torch.float32, device=dev)
        self.flat_grads = torch.zeros(n, dtype=torch.float32, device=dev)
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        with torch.no_grad():
            for p, o, s in zip(self.params, self.offsets, sizes):
                self.flat_params[o:o + s].copy_(p.detach().reshape(-1))
                p.data = self.flat_params[o:o + s].view(p.shape)
                p.grad = self.flat_grads[o:o + s].view(p.shape)
        self.ema = self.flat_params.clone()
        self.state = torch.zeros(8, dtype=torch.int32, device=dev)
        self.hyper_host = [float(lr), float(beta1), float(beta2), float(eps), float(clip_norm), float(ema_decay)]
        self.hyper = torch.tensor(self.hyper_host, dtype=torch.float32, device=dev)
        self.param_groups = [{"lr": float(lr)}]       # what torch optimisers expose; read-only here

    @property
    def lr(self) -> float:
        return self.hyper_host[0]

    def set_lr(self, lr: float) -> None:
        self.hyper_host[0] = float(lr)
        self.param_groups[0]["lr"] = float(lr)
        self.hyper[0:1].fill_(float(lr))               # a device write: later graph replays see it

    def zero_grad(self, set_to_none: bool = False) -> None:
        for p, o in zip(self.params, self.offsets):    # re-attach a gradient that autograd replaced
            if p.grad is None or p.grad.data_ptr() != self.flat_grads.data_ptr() + 4 * o:
                p.grad = self.flat_grads[o:o + p.numel()].view(p.shape)
        self.flat_grads.zero_()

    def step(self) -> None:
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ani_nadam_step_f32(
                self.flat_params.data_ptr(), self.flat_grads.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                self.ema.data_ptr(), self.n, self.hyper.data_ptr(), self.state.data_ptr(), stream),
                "ani_nadam_step_f32")

    def clip_rows(self, indices, max_norm: float = 3.0) -> None:
        """Max-norm constraint on the rows of the matrices ``self.params[k]``, k in ``indices``
        (``tf.clip_by_norm(w, max_norm, axes=1)``): one launch over a row table that is built on the
        first call."""
        key = tuple(indices)
        if getattr(self, "_row_key", None) != key:
            offs, lens = [], []
            for k in key:
                p, o = self.params[k], self.offsets[k]
                rows, cols = (p.shape[0], p.numel() // p.shape[0]) if p.dim() >= 2 else (1, p.numel())
                offs.extend(o + r * cols for r in range(rows))
                lens.extend([cols] * rows)
            self._row_offsets = torch.tensor(offs, dtype=torch.int32, device=self.device)
            self._row_lengths = torch.tensor(lens, dtype=torch.int32, device=self.device)
            self._row_key = key
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ani_clip_rows_f32(self.flat_params.data_ptr(), self._row_offsets.data_ptr(),
                                                    self._row_lengths.data_ptr(), int(self._row_offsets.numel()),
                                                    float(max_norm), stream), "ani_clip_rows_f32")

    def steps_done(self) -> int:
        """The device-side step counter (synchronises)."""
        return int(self.state[0].item())

    def set_steps(self, n: int) -> None:
        """Sets the device-side step counter, which drives the bias corrections of Nadam and the decay of
        the moving average (the other words of the state are scratch of a step and are cleared)."""
        self.state.zero_()
        self.state[0:1].fill_(int(n))

    def slots_of(self, index: int):
        """First moment, second moment and moving average of parameter ``index``, shaped like it (views)."""
        p, o = self.params[index], self.offsets[index]
        return tuple(buf[o:o + p.numel()].view(p.shape) for buf in (self.m, self.v, self.ema))

    def reset_state(self) -> None:
        """Moments to zero, step counter to zero, moving average = the current weights: the state of a
        freshly built optimiser around whatever the weights are now."""
        self.m.zero_()
        self.v.zero_()
        self.ema.copy_(self.flat_params)
        self.set_steps(0)

    def ema_of(self, index: int) -> torch.Tensor:
        """Moving average of parameter ``index``, shaped like it."""
        p, o = self.params[index], self.offsets[index]
        return self.ema[o:o + p.numel()].view(p.shape)

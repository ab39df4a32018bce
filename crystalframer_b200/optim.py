"""AdamW with gradient clipping on flat buffers: one library call per training step.

The reference trains with torch's AdamW and Lightning's ``gradient_clip_val`` (train.py, params "adamw" /
"clip_norm"), i.e. a per-tensor norm, a per-tensor scale and a multi-tensor update for the 60 parameter
tensors of the 4-layer model -- about a millisecond of host work and a dozen launches per step.  Here the
parameters are views into one flat buffer, every parameter owns a slice of one flat gradient buffer (its
"gradient sink"), and ``cfb200_adamw_clip_step`` does norm, clip and update in two launches.  The one-call
encoder layers add their weight gradients straight into the sinks (fused_layer.py); gradients that autograd
delivers in ``p.grad`` (embedding, output head) are added with one multi-tensor call.  With several ranks the
flat gradient buffer is what is all-reduced, so nothing is flattened or copied back."""
import torch
import torch.distributed as dist

from . import _lib

ALIGN = 64          # floats; every parameter starts on a 256-byte boundary of the flat buffers


class FlatAdamW:
    """``FlatAdamW(decay_params, no_decay_params, lr, betas, eps, weight_decay, max_norm)``; ``step()`` takes
    the gradient sinks plus the parameters' ``.grad``.  Same arithmetic as ``clip_grad_norm_(params, max_norm)``
    followed by ``torch.optim.AdamW.step()`` with ``weight_decay`` on ``decay_params`` only.  Both arguments may
    be any iterables (generators included); a parameter may appear only once.

    ``step(average=True)`` also keeps the running average of the weights that the reference maintains over its last
    epochs with ``torch.optim.swa_utils.AveragedModel`` (models/regression.py:150-152), inside the same launch;
    ``averaged_parameters()`` gives it back in the parameters' shapes and ``swap_averaged()`` exchanges it with the
    live weights (to evaluate the averaged model and to return to training)."""

    def __init__(self, decay_params, no_decay_params=(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2,
                 max_norm=0.0, grad_sink=True):
        decay = [p for p in decay_params if p.requires_grad]
        no_decay = [p for p in no_decay_params if p.requires_grad]
        self.params = decay + no_decay
        if len({id(p) for p in self.params}) != len(self.params):
            raise ValueError("FlatAdamW: a parameter appears more than once (tied weights or overlapping groups)")
        if not self.params or not all(p.is_cuda and p.dtype == torch.float32 for p in self.params):
            raise RuntimeError("FlatAdamW needs fp32 CUDA parameters (there is no CPU path)")
        dev = self.params[0].device
        offsets, off = [], 0
        for i, p in enumerate(self.params):
            if i == len(decay):
                self.decay_end = off                 # padding between parameters holds zeros and stays zero
            offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        if len(no_decay) == 0:
            self.decay_end = off
        self.n = off
        self.flat = torch.zeros(self.n, device=dev, dtype=torch.float32)
        self.grad = torch.zeros(self.n, device=dev, dtype=torch.float32)
        self.sinks = []
        for p, o in zip(self.params, offsets):       # parameters become views of the flat buffer
            k = p.numel()
            self.flat[o:o + k].copy_(p.data.reshape(-1))
            p.data = self.flat[o:o + k].view(p.shape)
            sink = self.grad[o:o + k].view(p.shape)
            self.sinks.append(sink)
            if grad_sink:
                p._cf_grad_sink = sink
        self.exp_avg = torch.zeros_like(self.flat)
        self.exp_avg_sq = torch.zeros_like(self.flat)
        self.scratch = torch.zeros(256, device=dev, dtype=torch.float32)
        self.grad_norm = torch.zeros(1, device=dev, dtype=torch.float32)
        self.lr, self.betas, self.eps, self.weight_decay, self.max_norm = lr, betas, eps, weight_decay, max_norm
        self.steps = 0
        self._offsets = offsets
        self.averaged = None          # flat running average of the weights, created by the first step(average=True)
        self.n_averaged = 0
        self.exchange = None          # parallel.GradientExchange once overlap_exchange() has been called

    def overlap_exchange(self, enable=True):
        """With several ranks: start the all-reduce of an encoder layer's slices of the flat gradient buffer as soon
        as that layer's backward has been enqueued, so that it runs beside the backward of the earlier layers;
        ``step(world_sum=True)`` then only sends what is left (embedding, output head, layers that did not take
        the one-call path) and waits.  For steps with ONE backward pass between ``zero_grad`` and ``step``: a
        slice that has been exchanged must not receive further gradients."""
        from . import fused_layer, parallel
        if not enable:
            self.exchange = None
            fused_layer.SINKS_FILLED = None
            return
        self.exchange = parallel.GradientExchange(self.grad)
        base = self.grad.data_ptr()

        def filled(tensors):
            if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
                return
            ranges = []
            for t in tensors:
                a = (t.data_ptr() - base) // 4
                ranges.append((a, a + (t.numel() + ALIGN - 1) // ALIGN * ALIGN))
            self.exchange.send(ranges)

        fused_layer.SINKS_FILLED = filled

    def zero_grad(self, set_to_none=True):
        """Clears the flat gradient buffer (one launch) and drops the parameters' ``.grad``."""
        self.grad.zero_()
        for p in self.params:
            p.grad = None

    def gather_grads(self):
        """Adds every gradient that autograd left in ``p.grad`` to the parameter's slice of the flat buffer (one
        multi-tensor call) and drops it; returns the flat gradient buffer."""
        dst, src = [], []
        for p, s in zip(self.params, self.sinks):
            if p.grad is not None:
                dst.append(s)
                src.append(p.grad)
                p.grad = None
        if dst:
            torch._foreach_add_(dst, src)
        return self.grad

    def step(self, world_sum=False, average=False):
        """One update.  ``world_sum``: sum the gradient buffer over the ranks first (one all-reduce).  ``average``:
        fold the updated weights into the running average (the first such step copies them)."""
        g = self.gather_grads()
        if world_sum and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            if self.exchange is not None:
                self.exchange.finish()
            else:
                dist.all_reduce(g)
        elif self.exchange is not None and self.exchange.work:
            raise RuntimeError("slices of the gradient buffer were exchanged during backward: call step(world_sum=True)")
        self.steps += 1
        b1, b2 = self.betas
        p = _lib.ptr
        if average and self.averaged is None:
            self.averaged = torch.zeros_like(self.flat)
        weight = 1.0 / (self.n_averaged + 1) if average else 0.0
        _lib.invoke("cfb200_adamw_clip_step_avg", 2, self.flat.device, p(self.flat), p(g), p(self.exp_avg), p(self.exp_avg_sq),
                    self.n, self.decay_end, self.lr, b1, b2, self.eps, self.weight_decay, self.max_norm,
                    1.0 - b1 ** self.steps, 1.0 - b2 ** self.steps, p(self.scratch), p(self.grad_norm),
                    p(self.averaged) if average else None, weight)
        if average:
            self.n_averaged += 1

    def averaged_parameters(self):
        """The running average in the parameters' shapes (views of the flat average), in ``self.params`` order."""
        if self.averaged is None:
            raise RuntimeError("no step(average=True) has been taken")
        return [self.averaged[o:o + p.numel()].view(p.shape) for p, o in zip(self.params, self._offsets)]

    def swap_averaged(self):
        """Exchanges the live weights with their running average (the parameters stay views of the same buffer)."""
        if self.averaged is None:
            raise RuntimeError("no step(average=True) has been taken")
        tmp = self.flat.clone()
        self.flat.copy_(self.averaged)
        self.averaged.copy_(tmp)

    def state_dict(self):
        return {"steps": self.steps, "exp_avg": self.exp_avg.clone(), "exp_avg_sq": self.exp_avg_sq.clone(),
                "n_averaged": self.n_averaged, "averaged": None if self.averaged is None else self.averaged.clone()}

    def load_state_dict(self, state):
        self.steps = int(state["steps"])
        self.exp_avg.copy_(state["exp_avg"])
        self.exp_avg_sq.copy_(state["exp_avg_sq"])
        self.n_averaged = int(state.get("n_averaged", 0))
        if state.get("averaged") is not None:
            self.averaged = state["averaged"].clone()

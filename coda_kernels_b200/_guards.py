"""Argument guards shared by the autograd wrappers.

``input_guard`` plays the role of ``fla.utils.input_guard`` in the reference
(e.g. coda/kernels/functional/swiglu.py:10-11): every tensor argument is made
contiguous and the CUDA device of the first tensor becomes current for the
call.  It is also where an expired device-side wait of an earlier launch gets
reported (``ops.lazy_status_check``: one library call that queries an event and
enqueues a 4-byte asynchronous copy, no synchronisation).  ``autocast_custom_fwd`` / ``autocast_custom_bwd`` are
``torch.amp.custom_fwd`` / ``custom_bwd`` bound to CUDA, as in the reference.
"""

from __future__ import annotations

import functools

import torch


def input_guard(fn):
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        first = None
        clean = []
        for a in args:
            if isinstance(a, torch.Tensor):
                a = a.contiguous()
                if first is None:
                    first = a
            clean.append(a)
        for k, v in kwargs.items():
            if isinstance(v, torch.Tensor):
                kwargs[k] = v = v.contiguous()
                if first is None:
                    first = v
        if first is None or not first.is_cuda:
            return fn(*clean, **kwargs)
        _ops().lazy_status_check(first.device)
        if first.device.index == torch.cuda.current_device():
            return fn(*clean, **kwargs)
        with torch.cuda.device(first.device):
            return fn(*clean, **kwargs)

    return wrapper


_ops_module = None


def _ops():
    """``coda_kernels_b200.ops``, imported at first use (it imports this module's users)."""
    global _ops_module
    if _ops_module is None:
        from . import ops

        _ops_module = ops
    return _ops_module


autocast_custom_fwd = functools.partial(torch.amp.custom_fwd, device_type="cuda")
autocast_custom_bwd = functools.partial(torch.amp.custom_bwd, device_type="cuda")

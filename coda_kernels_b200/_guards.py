"""Argument guards shared by the autograd wrappers.

``input_guard`` plays the role of ``fla.utils.input_guard`` in the reference
(e.g. coda/kernels/functional/swiglu.py:10-11): every tensor argument is made
contiguous and the CUDA device of the first tensor becomes current for the
call.  It is also where an expired device-side wait of an earlier launch gets
reported (``ops.lazy_status_check``: an event query and a 4-byte asynchronous
copy, no synchronisation).  ``autocast_custom_fwd`` / ``autocast_custom_bwd`` are
``torch.amp.custom_fwd`` / ``custom_bwd`` bound to CUDA, as in the reference.
"""

from __future__ import annotations

import functools

import torch


def input_guard(fn):
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        args = tuple(a.contiguous() if isinstance(a, torch.Tensor) else a for a in args)
        kwargs = {k: (v.contiguous() if isinstance(v, torch.Tensor) else v) for k, v in kwargs.items()}
        first = next((a for a in list(args) + list(kwargs.values()) if isinstance(a, torch.Tensor)), None)
        if first is not None and first.is_cuda:
            from .ops import lazy_status_check

            with torch.cuda.device(first.device):
                lazy_status_check(first.device)
                return fn(*args, **kwargs)
        return fn(*args, **kwargs)

    return wrapper


autocast_custom_fwd = functools.partial(torch.amp.custom_fwd, device_type="cuda")
autocast_custom_bwd = functools.partial(torch.amp.custom_bwd, device_type="cuda")

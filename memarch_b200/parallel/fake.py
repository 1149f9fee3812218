"""Single-process stand-in for `torch.distributed`: a world of one rank whose collectives are identities.

The reference keeps such a stub for machines without NCCL (race/fake_dist.py:1-31). Here it is a context manager
that swaps the functions of `torch.distributed` the package calls for in-process versions, so the multi-rank code
paths (expert exchange, bucketed gradient all-reduce, control all-reduce, vocab-parallel take / CE, row-sharded
homeostasis) run in one process without a rendezvous:

    with fake_world():
        eng = ParallelEngine(0, 1)
        ...

Everything is restored on exit.  The collectives keep their contracts: in-place ones leave the tensor as it is
(sum, mean and max over one rank), gathers copy the input into slot 0, `async_op=True` returns a finished work handle.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist


class _Done:
    """A finished work handle."""

    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True

    def get_future(self):
        f = torch.futures.Future()
        f.set_result(None)
        return f


class _Group:
    group_name = "fake"

    def size(self):
        return 1

    def rank(self):
        return 0


def _ret(async_op):
    return _Done() if async_op else None


def _identity(t, *a, async_op=False, **k):
    return _ret(async_op)


def _copy_into(out, inp):
    if out.data_ptr() != inp.data_ptr():
        with torch.no_grad():
            out.view(-1)[:inp.numel()].copy_(inp.reshape(-1))


def _all_gather(lst, t, group=None, async_op=False):
    _copy_into(lst[0], t)
    return _ret(async_op)


def _all_gather_into_tensor(out, inp, group=None, async_op=False):
    _copy_into(out, inp)
    return _ret(async_op)


def _reduce_scatter_tensor(out, inp, op=None, group=None, async_op=False):
    _copy_into(out, inp.reshape(-1)[:out.numel()])
    return _ret(async_op)


def _all_to_all_single(out, inp, output_split_sizes=None, input_split_sizes=None, group=None, async_op=False):
    _copy_into(out, inp)
    return _ret(async_op)


def _all_gather_object(lst, obj, group=None):
    lst[0] = obj


def _broadcast_object_list(lst, src=0, group=None, device=None):
    return None


_PATCH = {
    "is_initialized": lambda: True,
    "is_available": lambda: True,
    "get_world_size": lambda group=None: 1,
    "get_rank": lambda group=None: 0,
    "get_backend": lambda group=None: "fake",
    "init_process_group": lambda *a, **k: None,
    "destroy_process_group": lambda *a, **k: None,
    "barrier": lambda *a, async_op=False, **k: _ret(async_op),
    "broadcast": _identity,
    "all_reduce": _identity,
    "reduce": _identity,
    "all_gather": _all_gather,
    "all_gather_into_tensor": _all_gather_into_tensor,
    "reduce_scatter_tensor": _reduce_scatter_tensor,
    "all_to_all_single": _all_to_all_single,
    "all_gather_object": _all_gather_object,
    "broadcast_object_list": _broadcast_object_list,
    "new_group": lambda *a, **k: _Group(),
}


@contextlib.contextmanager
def fake_world():
    """Install the identity collectives into `torch.distributed` for the duration of the block."""
    saved = {k: getattr(dist, k, None) for k in _PATCH}
    try:
        for k, f in _PATCH.items():
            setattr(dist, k, f)
        yield _Group()
    finally:
        for k, f in saved.items():
            if f is None:
                delattr(dist, k)
            else:
                setattr(dist, k, f)

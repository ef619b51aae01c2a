"""
Activation checkpointing that also discards the checkpointed function's OUTPUT
(role of src/olmo_core/nn/output_discard_checkpoint.py:180-353).

Ordinary checkpointing frees what a function computes internally but keeps its output alive for the consumer's
backward pass. When the consumer is a cheap-to-recompute step (e.g. the activation between two expert GEMMs), the
output can be dropped as well::

    ckpt = OutputDiscardCheckpoint()
    h = ckpt.checkpoint(fn, x)            # forward of fn, no graph kept inside
    y = consumer(h)                        # consumer saves ``h`` for its backward
    ckpt.discard_output_and_register_recompute(y)   # free h's memory now

When gradients reach ``y`` the function is re-run, its result is written back into the very tensor object the consumer
saved (so the consumer's backward sees valid data again), and backward of ``fn`` itself runs on the recomputed graph.
The tensor's storage is released with ``resize_(0)``. At recomputation the native helper ``torch.ops.ocb_native.rebind_storage``
(``nn/_csrc/storage_rebind.cpp``, built ahead of time by ``python -m olmo_core_b200.ops.build``) points the emptied
``StorageImpl`` at the recomputed tensor's allocation, so nothing is copied; without the helper library the storage is
re-grown in place and the recomputed bytes are copied into it.
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Tuple

import torch

__all__ = ["OutputDiscardCheckpoint", "native_rebind_available"]

_native_state: Optional[bool] = None


def native_rebind_available() -> bool:
    """Load ``libocb_native.so`` once; True when ``torch.ops.ocb_native.rebind_storage`` can be used."""
    global _native_state
    if _native_state is None:
        from ..ops.build import NATIVE_LIB_PATH

        try:
            if NATIVE_LIB_PATH.exists():
                torch.ops.load_library(str(NATIVE_LIB_PATH))
                _native_state = True
            else:
                _native_state = False
        except OSError:
            _native_state = False
        if not _native_state and torch.cuda.is_available():
            raise RuntimeError(
                f"{NATIVE_LIB_PATH} is missing or unloadable; build it with `python -m olmo_core_b200.ops.build`"
            )
    return _native_state


def _tensors(outputs: Any) -> Tuple[torch.Tensor, ...]:
    if isinstance(outputs, torch.Tensor):
        return (outputs,)
    if isinstance(outputs, (tuple, list)):
        return tuple(t for t in outputs if isinstance(t, torch.Tensor))
    raise TypeError(f"the checkpointed function must return tensors, got {type(outputs)}")


class _Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run, owner, *args):  # type: ignore[override]
        ctx.run, ctx.owner = run, owner
        ctx.inputs = args
        with torch.no_grad():
            outputs = run(*args)
        return outputs

    @staticmethod
    def backward(ctx, *grads):  # type: ignore[override]
        recomputed = ctx.owner._recomputed
        if recomputed is None:  # nobody registered a discard: recompute here, like a plain checkpoint
            recomputed = ctx.owner._rerun(ctx.run, ctx.inputs)
        outs = _tensors(recomputed)
        pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        # the detached copies of the inputs used for the recomputation carry the input gradients
        detached = ctx.owner._detached_inputs
        in_grads = tuple(a.grad if isinstance(a, torch.Tensor) else None for a in detached)
        ctx.owner.clear()
        return (None, None) + in_grads


class OutputDiscardCheckpoint:
    def __init__(self):
        self._run: Optional[Callable[..., Any]] = None
        self._inputs: Optional[Tuple[Any, ...]] = None
        self._outputs: Optional[Tuple[torch.Tensor, ...]] = None
        self._recomputed: Any = None
        self._detached_inputs: Optional[Tuple[Any, ...]] = None
        self._rng_cpu = self._rng_cuda = None

    def checkpoint(self, fn: Callable[..., Any], *args: Any, **kwargs: Any) -> Any:
        """Run ``fn(*args, **kwargs)`` without building a graph inside; tensor arguments must be positional."""
        def run(*inner):
            return fn(*inner, **kwargs)

        self._run, self._inputs = run, args
        self._rng_cpu = torch.get_rng_state()
        self._rng_cuda = torch.cuda.get_rng_state() if torch.cuda.is_available() and torch.cuda.is_initialized() else None
        out = _Function.apply(run, self, *args)
        self._outputs = _tensors(out)
        return out

    def discard_output_and_register_recompute(self, hook_tensor: torch.Tensor) -> None:
        """Free the outputs now; recompute them when the gradient of ``hook_tensor`` (the consumer's result) is ready."""
        assert self._outputs is not None, "call checkpoint() first"
        for t in self._outputs:
            t.untyped_storage().resize_(0)
        if hook_tensor.requires_grad:
            hook_tensor.register_hook(self._recompute)

    def _rerun(self, run, inputs):
        detached = tuple(a.detach().requires_grad_(a.requires_grad) if isinstance(a, torch.Tensor) else a for a in inputs)
        self._detached_inputs = detached
        cpu_state = torch.get_rng_state()
        cuda_state = torch.cuda.get_rng_state() if self._rng_cuda is not None else None
        torch.set_rng_state(self._rng_cpu)
        if self._rng_cuda is not None:
            torch.cuda.set_rng_state(self._rng_cuda)
        try:
            with torch.enable_grad():
                out = run(*detached)
        finally:
            torch.set_rng_state(cpu_state)
            if cuda_state is not None:
                torch.cuda.set_rng_state(cuda_state)
        return out

    def _recompute(self, grad: torch.Tensor) -> torch.Tensor:
        assert self._run is not None and self._inputs is not None and self._outputs is not None
        self._recomputed = self._rerun(self._run, self._inputs)
        native = native_rebind_available()
        with torch.no_grad():
            for old, new in zip(self._outputs, _tensors(self._recomputed)):
                if native and new.is_contiguous() and new.storage_offset() == old.storage_offset():
                    torch.ops.ocb_native.rebind_storage(old, new)  # zero-copy: same StorageImpl, new allocation
                    continue
                old.untyped_storage().resize_(new.numel() * new.element_size())
                # written through `.data`: same memory, but the version counter that autograd checked when the consumer
                # saved `old` is left alone
                old.data.copy_(new)
        return grad

    def clear(self) -> None:
        self._run = self._inputs = self._outputs = self._recomputed = self._detached_inputs = None

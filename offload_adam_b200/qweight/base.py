"""Base class of the weight-only quantized tensor subclasses used for QAT.

A ``QWeightBase`` is a wrapper tensor subclass: it looks like a dense
``(out_features, in_features)`` weight of some float dtype, while holding packed
payload tensors.  ``F.linear`` on it dequantizes on the fly (forward and
backward), its gradient is a plain dense tensor, and ``copy_`` from a dense
tensor re-quantizes in place, which is how the optimizers push the updated fp32
master back into the packed weight
(reference: src/offload_adam/qweight/base.py:13-124 for the public contract).

Unlike the reference, which repeats the autograd function and the five ATen
handlers in every format file, the shared behaviour lives here and is driven by
two per-class declarations:

* ``PAYLOAD``: names of the tensor attributes that make up the packed storage;
* ``META``: names of the non-tensor attributes passed to the constructor after
  the payload tensors.

A subclass provides ``_quantize_into(src)`` (re-quantize a dense tensor into the
existing payload), ``dequantize`` and the state-dict / HF-config methods.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.utils._python_dispatch import return_and_correct_aliasing

aten = torch.ops.aten


class _WeightOnlyLinear(torch.autograd.Function):
    """y = x @ dequant(W)^T (+ b); the packed weight is saved, not the dense one."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: "QWeightBase", bias: Optional[Tensor] = None):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        w = weight.dequantize(dtype=x.dtype)
        y = x @ w.T
        return y if bias is None else y + bias

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        w = weight.dequantize(dtype=gy.dtype)
        gx = gy @ w
        g2 = gy.reshape(-1, weight.shape[0])
        gw = g2.T @ x.reshape(-1, weight.shape[1])
        gb = g2.sum(0) if ctx.has_bias else None
        return gx, gw, gb


class QWeightBase(Tensor):
    PAYLOAD: Tuple[str, ...] = ()
    META: Tuple[str, ...] = ()

    _ATEN_OP_TABLE: dict
    _TORCH_FN_TABLE: dict

    # ------------------------------------------------------------------ registry
    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        cls._ATEN_OP_TABLE = {}
        cls._TORCH_FN_TABLE = {}
        _install_common_handlers(cls)

    @classmethod
    def implements(cls, aten_ops):
        """Decorator: register an ATen op handler ``fn(func, types, args, kwargs)``."""
        ops = aten_ops if isinstance(aten_ops, (list, tuple)) else [aten_ops]

        def deco(fn):
            for op in ops:
                cls._ATEN_OP_TABLE[op] = fn
            return fn

        return deco

    @classmethod
    def implements_torch_function(cls, torch_fns):
        """Decorator: register a ``__torch_function__`` handler."""
        fns = torch_fns if isinstance(torch_fns, (list, tuple)) else [torch_fns]

        def deco(fn):
            for f in fns:
                cls._TORCH_FN_TABLE[f] = fn
            return fn

        return deco

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        handler = cls._ATEN_OP_TABLE.get(func)
        if handler is None:
            raise NotImplementedError(
                f"{cls.__name__} does not support {func}. "
                f"Register a handler via @{cls.__name__}.implements(...)."
            )
        return handler(func, types, args, kwargs)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        handler = cls._TORCH_FN_TABLE.get(func)
        if handler is not None:
            return handler(func, types, args, kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    # --------------------------------------------------------------- flattening
    def __tensor_flatten__(self):
        return list(self.PAYLOAD), [getattr(self, k) for k in self.META]

    @classmethod
    def __tensor_unflatten__(cls, tensors, attrs, outer_size=None, outer_stride=None):
        return cls(*[tensors[k] for k in cls.PAYLOAD], *attrs)

    def _payload(self):
        return [getattr(self, k) for k in self.PAYLOAD]

    def _meta(self):
        return [getattr(self, k) for k in self.META]

    def _rebuild(self, payload, **meta_overrides):
        meta = [meta_overrides.get(k, getattr(self, k)) for k in self.META]
        return type(self)(*payload, *meta)

    # ------------------------------------------------------------- subclass API
    def dequantize(self, dtype=None) -> Tensor:
        """Dense reconstruction at ``dtype`` (default: the outer dtype)."""
        raise NotImplementedError

    def _quantize_into(self, src: Tensor, amax: Optional[Tensor] = None) -> None:
        """Re-quantize dense ``src`` into this instance's payload tensors.  ``amax``
        (a one-element fp32 tensor holding max|x| of the WHOLE weight) is used by
        formats with a per-tensor scale and ignored by the others."""
        raise NotImplementedError

    #: True when quantization needs max|x| over the whole tensor (a per-tensor scale)
    USES_TENSOR_AMAX = False

    #: Format id of the fused optimizer kernels (``csrc/quant.h`` ``QFormat``), and the
    #: names of the two payload tensors those kernels write: packed values, then scales.
    KERNEL_FORMAT = 0
    KERNEL_PAYLOAD: Tuple[str, str] = ("", "")

    def kernel_group(self) -> int:
        """Columns per scale of the fused kernels (NF4 block size, int4 group size)."""
        return 0

    def kernel_scale_dtype(self):
        """Dtype of the stored scales when the format keeps them in the outer dtype."""
        return torch.bfloat16

    def _payload_rows(self, lo: int, hi: int):
        """Per payload tensor, the view that holds output rows ``[lo, hi)`` of the
        weight (the whole tensor for per-tensor quantities)."""
        raise NotImplementedError

    def row_shard(self, lo: int, hi: int):
        """A weight over output rows ``[lo, hi)`` for sharded re-quantization.

        Returns ``(shard, views)``.  ``views[i]`` is where rows ``[lo, hi)`` live in
        payload tensor ``i`` of ``self``.  The shard's payload aliases those views
        when they are contiguous (row-major formats), otherwise it owns contiguous
        temporaries of the same shape (GPTQ's transposed layout) that the caller
        copies or gathers into place.  Quantizing rows separately gives the same
        bits as quantizing the whole weight because no block or group of any format
        spans two output rows; the per-tensor scale of NVFP4 is the exception and
        is handled by passing the global ``amax``."""
        views = self._payload_rows(lo, hi)
        payload = [v if v.is_contiguous() else torch.empty(v.shape, dtype=v.dtype, device=v.device)
                   for v in views]
        return self._rebuild(payload), views

    def _with_outer_dtype(self, payload, dtype):
        """Rebuild with a different outer dtype (used by ``.to(dtype)``)."""
        return self._rebuild(payload)

    @classmethod
    def can_quantize(cls, tensor: Tensor, **kwargs) -> bool:
        """False when this format cannot hold a weight of that shape/dtype."""
        return True

    @classmethod
    def canonical_key_suffixes(cls) -> tuple:
        """Key suffixes of the plain tensors this format saves and loads."""
        raise NotImplementedError

    def to_plain_state_dict(self) -> dict:
        """Plain tensors keyed by ``canonical_key_suffixes()``."""
        raise NotImplementedError

    @classmethod
    def from_plain_state_dict(cls, plain: dict, reference=None) -> "QWeightBase":
        """Inverse of ``to_plain_state_dict``; ``reference`` (the instance
        already on the module) supplies what the plain tensors do not carry."""
        raise NotImplementedError

    @classmethod
    def build_hf_quantization_config(cls, skip_patterns=(), **weight_kwargs) -> dict:
        """``quantization_config`` dict for ``config.json`` so HF / vLLM route
        the checkpoint through the matching loader."""
        raise NotImplementedError

    def __repr__(self):
        extra = "".join(f", {k}={getattr(self, k)}" for k in self.META if k not in ("in_f", "outer_dtype"))
        return (
            f"{type(self).__name__}(shape={tuple(self.shape)}, dtype={self.dtype}, "
            f"device={self.device}{extra}, requires_grad={self.requires_grad})"
        )


def _install_common_handlers(cls):
    """Handlers every format shares; a subclass may override any of them."""

    @cls.implements_torch_function(torch.nn.functional.linear)
    def _linear(func, types, args, kwargs):
        return _WeightOnlyLinear.apply(*args, **kwargs)

    @cls.implements([aten.detach.default, aten.clone.default])
    def _detach_clone(func, types, args, kwargs):
        self = args[0]
        out = self._rebuild([func(t, *args[1:], **kwargs) for t in self._payload()])
        return return_and_correct_aliasing(func, args, kwargs, out)

    @cls.implements(aten._to_copy.default)
    def _to_copy(func, types, args, kwargs):
        self = args[0]
        device = kwargs.get("device", None)
        dtype = kwargs.get("dtype", None)
        payload = [t.to(device=device) for t in self._payload()]
        out = self._with_outer_dtype(payload, dtype) if dtype is not None else self._rebuild(payload)
        return return_and_correct_aliasing(func, args, kwargs, out)

    @cls.implements(aten.copy_.default)
    def _copy_(func, types, args, kwargs):
        dst, src = args[0], args[1]
        if isinstance(dst, cls) and isinstance(src, cls):
            for d, s in zip(dst._payload(), src._payload()):
                d.copy_(s)
        elif isinstance(dst, cls):
            dst._quantize_into(src, None)
        else:
            dst.copy_(src.dequantize())
        return dst

    @cls.implements(aten.zeros_like.default)
    def _zeros_like(func, types, args, kwargs):
        self = args[0]
        return torch.zeros(
            self.shape,
            dtype=kwargs.get("dtype", None) or self.dtype,
            device=kwargs.get("device", None) or self.device,
        )

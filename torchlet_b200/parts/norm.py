"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, float32 inside
(v10_triton_paged_gqa/layer/rms_norm.py:7-25, kernel/rms_norm.py:13-22).

Parameters: ``size``, ``eps``; ``groups`` (default 1): the row is split into that many equal
consecutive parts and each is divided by its own root mean square, the weight covers the whole
row; ``weight_name`` (default "weight"): the tensor's name below the norm's prefix ("" when the
prefix itself is the tensor's name); ``weight_offset`` (default 0): the stored weight lies around
zero and the norm multiplies by ``weight_offset + w`` (1 for a "one plus weight" norm).

``add_normed`` is the norm of a sub-layer's OUTPUT: acc += norm(y) for a float32 side stream y,
one float32 kernel (a sandwich block's second norm)."""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import NORMS, Norm, TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.groups = int(spec.params.get("groups", 1))
        self.weight_offset = float(spec.params.get("weight_offset", 0.0))
        if self.groups <= 0 or self.size % self.groups:
            raise ValueError(f"a norm of {self.size} elements cannot be split into {self.groups} equal parts")
        self.weight = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        init = "zeros" if float(spec.params.get("weight_offset", 0.0)) else "ones"
        return [TensorSpec(prefix + spec.params.get("weight_name", "weight"), (int(spec.params["size"]),), init=init)]

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        name = prefix + self.spec.params.get("weight_name", "weight")
        self.weight = tensors[name].to(device=device, dtype=torch.float32).contiguous()
        if self.weight_offset:
            self.weight += self.weight_offset

    centre = False  # no mean is taken off (what a block that norms inside its own kernel asks)
    fuses_pending = True  # a product's unfinished sum into the stream is completed in the norm's own kernel

    def forward(self, ctx, acc, out=None, rows=None, name="normed"):
        """Normed rows of the float32 stream ``acc`` in the compute dtype; ``rows``
        (int32) selects and orders the rows, default all."""
        count = acc.shape[0] if rows is None else rows.numel()
        if out is None:
            out = ctx.buffer(name, (count, self.size), ctx.dtype)
        if rows is None and out.dtype == torch.bfloat16 and self.groups == 1:
            pending = ctx.take_pending(acc)
            if pending is not None:  # finish the sum and norm in one kernel
                ops.finish_accum_norm(pending.partials, pending.splits, pending.bias, acc, self.weight, self.eps, out)
                return out
        ctx.flush_pending()
        ops.rms_norm(acc, self.weight, self.eps, out, rows, self.groups)
        return out

    def add_normed(self, ctx, y, acc, m: float = 1.0, clear: bool = False) -> None:
        """acc += m * norm(y): both float32 ``[T, size]``; ``y`` is a side stream a sub-layer added its
        output into.  ``clear``: y is zeroed in the same pass, ready for the next sub-layer."""
        if self.groups != 1:
            raise ValueError("the norm of a sub-layer's output is not built for grouped norms")
        pending = ctx.take_pending(y)
        if pending is not None and pending.bias is None:
            # the sub-layer's last product left its split sums: their sum into y, the norm and the residual sum
            # as one kernel
            ops.rms_scaled_add_partials(acc, y, pending.partials, pending.splits, self.weight, m, self.eps, clear)
            return
        if pending is not None:  # finish the split sums into y first
            ops.finish_accum_norm(pending.partials, pending.splits, pending.bias, y)
        else:
            ctx.flush_pending()
        ops.rms_scaled_add(acc, y, self.weight, m, self.eps, clear)


@NORMS.register("layer_norm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(variance + eps) * w + b, the variance being the mean of the squared deviations;
    float32 inside (csrc/hyper.cu).  Parameters: ``size``, ``eps``, ``weight_name`` (default "weight"; "" when the
    prefix itself is the tensor's name), ``bias_name`` (default "bias"; None: no bias)."""

    centre = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = self.bias = None

    @classmethod
    def _names(cls, spec: PartSpec, prefix: str) -> tuple:
        bias = spec.params.get("bias_name", "bias")
        return prefix + spec.params.get("weight_name", "weight"), (prefix + bias if bias is not None else None)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        weight, bias = cls._names(spec, prefix)
        size = int(spec.params["size"])
        return [TensorSpec(weight, (size,), init="ones")] + ([TensorSpec(bias, (size,), init="zeros")] if bias else [])

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        weight, bias = self._names(self.spec, prefix)
        self.weight = tensors[weight].to(device=device, dtype=torch.float32).contiguous()
        self.bias = tensors[bias].to(device=device, dtype=torch.float32).contiguous() if bias else None

    def forward(self, ctx, acc, out=None, rows=None, name="normed"):
        count = acc.shape[0] if rows is None else rows.numel()
        if out is None:
            out = ctx.buffer(name, (count, self.size), ctx.dtype)
        ops.hyper_read_norm(acc, None, self.weight, self.bias, self.eps, out, centre=True, rows=rows)
        return out

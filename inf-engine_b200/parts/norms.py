"""RMSNorm: ``x / sqrt(mean(x^2) + eps) * gain`` (engine/layers.py:11-25), with
float32 statistics whatever the activation dtype, fused with the residual sum
that precedes it in a pre-norm block (engine/llama_block.py:53-62).  With
``unit_offset`` the stored tensor lies around zero and the gain is one plus it
(formed once, in float32); with ``scalar`` the stored tensor is a single number that multiplies every coordinate.
``accumulate`` is the norm of a block that norms its
sublayers' OUTPUTS: the normed rows are added into the residual.
LayerNorm: ``(x - mean) / sqrt(variance + eps) * weight + bias`` with the variance
the mean of the squared deviations, the same way."""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import ExpectedTensor
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    @staticmethod
    def expected_tensors(spec):
        return {spec.weight: ExpectedTensor(() if getattr(spec, "scalar", False) else (spec.size,), init="gain")}

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        self.gain = tensors[spec.weight]
        if getattr(spec, "scalar", False):
            # one number for every coordinate: spread out once, so that the kernels and the products that apply a norm
            # in their prologue see the vector they expect
            self.gain = self.gain.reshape(1).expand(spec.size).contiguous()
        if getattr(spec, "unit_offset", False):
            self.gain = (1.0 + self.gain.float()).contiguous()
        self.eps = float(spec.eps)
        self.size = spec.size

    def accumulate(self, residual: torch.Tensor, y: torch.Tensor, next_in: torch.Tensor | None = None) -> None:
        """residual += norm(y); ``next_in`` (activation type, optional) takes the new residual rows."""
        kernels.outnorm_accumulate(residual, y, self.gain, self.eps, next_in)

    def accumulate_then_norm(self, residual: torch.Tensor, y: torch.Tensor, next_norm, out_name: str = "normed"):
        """residual += norm(y), and in the same kernel the rows that ``next_norm`` (an RMS norm of this size) makes of
        the new residual; None when the two do not go together (the caller then runs them one after the other)."""
        if not isinstance(next_norm, RMSNorm) or next_norm.size != self.size or next_norm.gain.dtype != self.gain.dtype:
            return None
        out = self.rt.ws.take(out_name, tuple(residual.shape), self.rt.act_dtype)
        kernels.outnorm_accumulate_norm(residual, y, self.gain, self.eps, next_norm.gain, next_norm.eps, out)
        return out

    def fusable_rms(self):
        """(gain, eps) for kernels that apply this norm inside a matrix product's prologue."""
        return self.gain, self.eps

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, out_name: str = "normed") -> torch.Tensor:
        out = self.rt.ws.take(out_name, tuple(residual.shape), self.rt.act_dtype)
        kernels.rmsnorm(residual, delta, self.gain, out, self.eps)
        return out

    def gather_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, row_index: torch.Tensor,
                    n_rows: int, out_name: str = "normed_rows") -> torch.Tensor:
        out = self.rt.ws.take(out_name, (n_rows, self.size), self.rt.act_dtype)
        kernels.rmsnorm(residual, delta, self.gain, out, self.eps, row_index=row_index)
        return out


@register_norm("layernorm")
class LayerNorm:
    @staticmethod
    def expected_tensors(spec):
        out = {spec.weight: ExpectedTensor((spec.size,), init="gain")}
        if spec.bias is not None:
            out[spec.bias] = ExpectedTensor((spec.size,))
        return out

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        self.weight = tensors[spec.weight]
        self.bias = tensors[spec.bias].to(self.weight.dtype) if spec.bias is not None else None
        self.eps = float(spec.eps)
        self.size = spec.size

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, out_name: str = "normed") -> torch.Tensor:
        out = self.rt.ws.take(out_name, tuple(residual.shape), self.rt.act_dtype)
        kernels.layernorm(residual, delta, self.weight, self.bias, out, self.eps)
        return out

    def gather_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, row_index: torch.Tensor,
                    n_rows: int, out_name: str = "normed_rows") -> torch.Tensor:
        out = self.rt.ws.take(out_name, (n_rows, self.size), self.rt.act_dtype)
        kernels.layernorm(residual, delta, self.weight, self.bias, out, self.eps, row_index=row_index)
        return out

"""RMSNorm and layer norm, each with the residual add in front of it (one kernel).

Formula of the reference: ``w * x * rsqrt(mean(x^2) + eps)`` in float32
(miniinfer/layers/layernorm.py:27-32), fused with the residual add as in its Triton kernel
(kernels/triton/rms_norm.py:66-108).  The residual stream here is float32.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple, Union

import torch

from ..kernels import ops
from .base import Norm, ParamSpec, whole


Delta = Union[None, torch.Tensor, Tuple[Optional[torch.Tensor], ...]]


def split_delta(delta: Delta) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
  """What is pending for the residual stream as (first, second): a block whose mixer and feed-forward read the same
  normalised rows leaves two outputs to be added, the usual block one."""
  if delta is None or isinstance(delta, torch.Tensor):
    return delta, None
  parts = [d for d in delta if d is not None]
  if len(parts) > 2:
    raise ValueError("at most two outputs can be pending for the residual stream")
  return (parts + [None, None])[0], (parts + [None, None])[1]


class RMSNorm(Norm):
  def __init__(self, name: str, dim: int, eps: float):
    super().__init__(name)
    self.dim = dim
    self.eps = float(eps)

  def param_specs(self) -> Dict[str, ParamSpec]:
    return {"weight": ParamSpec((self.dim,), "vector", [whole(f"{self.name}.weight", (self.dim,))], init="ones_noise")}

  def as_rms(self):
    return self.weight, self.eps

  def add_norm(self, resid: torch.Tensor, delta: Delta, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    if second is not None:
      raise NotImplementedError("RMSNorm adds one pending output; put a LayerNorm behind a block that leaves two")
    out = ctx.ws.buffer("normed", (resid.shape[0], self.dim), ctx.dtype)
    ops.add_rmsnorm(out, resid, first, self.weight, self.eps, None, True)
    return out

  def norm_rows(self, resid: torch.Tensor, delta: Delta, rows: torch.Tensor, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    if second is not None:
      raise NotImplementedError("RMSNorm adds one pending output; put a LayerNorm behind a block that leaves two")
    out = ctx.ws.buffer("normed_rows", (rows.shape[0], self.dim), ctx.dtype)
    ops.add_rmsnorm(out, resid, first, self.weight, self.eps, rows, False)
    return out


class LayerNorm(Norm):
  """``(x - mean) / sqrt(var + eps) * weight + bias`` in float32, the variance being the mean of the squared
  deviations; the residual add (of one or two pending outputs) in front of it, in one kernel.  ``bias_name``: the file
  tensor of the bias (default ``<name>.bias``; the weight is ``<name>.weight`` or, with ``bare_names``, ``<name>``)."""

  def __init__(self, name: str, dim: int, eps: float, weight_name: Optional[str] = None, bias_name: Optional[str] = None):
    super().__init__(name)
    self.dim = dim
    self.eps = float(eps)
    self.weight_name = weight_name or f"{name}.weight"
    self.bias_name = bias_name or f"{name}.bias"

  def param_specs(self) -> Dict[str, ParamSpec]:
    return {"weight": ParamSpec((self.dim,), "vector", [whole(self.weight_name, (self.dim,))], init="ones_noise"),
            "bias": ParamSpec((self.dim,), "vector", [whole(self.bias_name, (self.dim,))])}

  def validate(self, dtype: torch.dtype) -> None:
    if self.dim > 12000:
      raise ValueError(f"{self.name}: rows of {self.dim} values are more than the layer-norm kernel keeps in shared memory (12000)")

  def add_norm(self, resid: torch.Tensor, delta: Delta, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    out = ctx.ws.buffer("normed", (resid.shape[0], self.dim), ctx.dtype)
    ops.add_layernorm(out, resid, first, second, self.weight, self.bias, self.eps, None, True)
    return out

  def norm_rows(self, resid: torch.Tensor, delta: Delta, rows: torch.Tensor, ctx) -> torch.Tensor:
    first, second = split_delta(delta)
    out = ctx.ws.buffer("normed_rows", (rows.shape[0], self.dim), ctx.dtype)
    ops.add_layernorm(out, resid, first, second, self.weight, self.bias, self.eps, rows, False)
    return out

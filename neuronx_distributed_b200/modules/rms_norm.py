"""RMSNorm with fp32 statistics and a sequence-parallel-tagged weight
(reference ``modules/rms_norm.py:10-72``).  Forward/backward run the sm_100a kernels in
``csrc/elementwise.cu`` via :func:`ops.norm.rms_norm`."""
from __future__ import annotations

import numbers
from typing import Optional

import torch
from torch import nn

from ..ops.norm import rms_norm


def manual_rms_norm(input: torch.Tensor, *args) -> torch.Tensor:   # noqa: A002  (reference argument name)
    """Plain-PyTorch form (kept for numerics tests).  ``manual_rms_norm(x, weight, eps)`` or the reference's
    ``manual_rms_norm(input, normalized_shape, weight, eps)`` (rms_norm.py:10-33; statistics over the trailing
    ``len(normalized_shape)`` dims)."""
    if len(args) == 3:
        normalized_shape, weight, eps = args
        dims = tuple(range(-len(tuple(normalized_shape)), 0))
    else:
        (weight, eps), dims = args, (-1,)
    dt = input.dtype
    xf = input.float()
    return (weight.float() * (xf * torch.rsqrt(xf.pow(2).mean(dims, keepdim=True) + eps))).to(dt)


class RMSNorm(nn.Module):
    def __init__(self, normalized_shape=None, eps: float = 1e-5, sequence_parallel_enabled: bool = False,
                 dtype: torch.dtype = torch.float32, device=None, hidden_size: Optional[int] = None, **kwargs):
        """``normalized_shape``: int or shape of the trailing dims (``hidden_size=`` is the same thing by keyword).  Signature
        and the 1e-5 default of reference rms_norm.py:36-62; ``elementwise_affine=False`` is refused as there."""
        super().__init__()
        if kwargs.pop("elementwise_affine", True) is False:
            raise RuntimeError("RMSNorm does not support `elementwise_affine = False`")
        if kwargs:
            raise TypeError(f"unexpected arguments {sorted(kwargs)}")
        shape = normalized_shape if normalized_shape is not None else hidden_size
        assert shape is not None, "normalized_shape (or hidden_size) is required"
        self.normalized_shape = torch.Size((shape,) if isinstance(shape, numbers.Integral) else tuple(shape))
        assert len(self.normalized_shape) == 1, "the kernels normalise over the last dimension"
        self.elementwise_affine = True
        self.weight = nn.Parameter(torch.ones(self.normalized_shape, dtype=dtype, device=device))
        self.eps = self.variance_epsilon = eps
        self.sequence_parallel_enabled = sequence_parallel_enabled
        setattr(self.weight, "sequence_parallel_enabled", sequence_parallel_enabled)

    def reset_parameters(self) -> None:
        """Re-initialise after meta-device materialisation (``reinit_model`` calls it): unit gain."""
        with torch.no_grad():
            self.weight.fill_(1.0)
        setattr(self.weight, "sequence_parallel_enabled", self.sequence_parallel_enabled)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        hidden_states = input      # reference parameter names in the signature
        return rms_norm(hidden_states, self.weight, self.variance_epsilon)

    def extra_repr(self) -> str:
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


class ScalarRMSNorm(nn.Module):
    """RMS norm whose gain is ONE number for all coordinates: ``x / sqrt(mean(x^2) + eps) * g``.  ``add_to(res, y)`` is the
    residual form of a block that normalises the sublayer's OUTPUT: ``res += norm(y)`` with ``res`` a float stream (one kernel,
    ``csrc/seqmix/norms.cu``)."""

    def __init__(self, eps: float = 1e-6, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones((), dtype=torch.float32, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, input: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        from ..ops import seqmix

        x = input
        return seqmix.rms_norm(x.reshape(-1, x.shape[-1]), self.weight.reshape(1), self.eps, None, out_dtype or x.dtype).view(x.shape)

    def add_to(self, res: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        from ..ops import seqmix

        seqmix.add_rms_norm_(res.view(-1, res.shape[-1]), y.reshape(-1, y.shape[-1]), self.weight.reshape(1), self.eps)
        return res


class OffsetRMSNorm(nn.Module):
    """RMS norm whose checkpoint stores the gain's offset from one: ``x / sqrt(mean(x^2) + eps) * (1 + w)``.  The parameter here
    is the gain itself, ``1 + w`` formed once in float (``set_offset``).  ``forward`` gives the sublayer's input in ``out_dtype``;
    ``add_to(res, y)`` is the closing norm of a sandwich block, ``res += norm(y)`` with ``res`` a float stream (one kernel each,
    ``csrc/seqmix/norms.cu``)."""

    def __init__(self, width: int, eps: float = 1e-6, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32, device=device), requires_grad=False)
        self.eps = eps

    @torch.no_grad()
    def set_offset(self, w: torch.Tensor) -> None:
        self.weight.copy_(1.0 + w.to(device=self.weight.device, dtype=torch.float32))

    def forward(self, input: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        from ..ops import seqmix

        x = input
        return seqmix.rms_norm(x.reshape(-1, x.shape[-1]), self.weight, self.eps, None, out_dtype or x.dtype).view(x.shape)

    def add_to(self, res: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        from ..ops import seqmix

        seqmix.add_rms_norm_(res.view(-1, res.shape[-1]), y.reshape(-1, y.shape[-1]), self.weight, self.eps)
        return res


class GainOnlyLayerNorm(nn.Module):
    """Layer norm with a gain and no bias: ``(x - mean) / sqrt(mean((x - mean)^2) + eps) * w``, statistics in float.  ``forward``
    gives the sublayer's input in ``out_dtype``; ``add_to(res, y)`` is the closing norm of a sandwich block, ``res += norm(y)`` with
    ``res`` a float stream (one kernel each: the RMS-norm kernels of ``csrc/seqmix/norms.cu`` with the mean taken off first)."""

    def __init__(self, width: int, eps: float = 1e-6, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, input: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        from ..ops import seqmix

        x = input
        return seqmix.rms_norm(x.reshape(-1, x.shape[-1]), self.weight, self.eps, None, out_dtype or x.dtype, center=True).view(x.shape)

    def add_to(self, res: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        from ..ops import seqmix

        seqmix.add_rms_norm_(res.view(-1, res.shape[-1]), y.reshape(-1, y.shape[-1]), self.weight, self.eps, center=True)
        return res


class GatedPostRMSNorm(nn.Module):
    """The closing step of a block whose norm comes AFTER the residual sum: ``x <- rms_norm(alpha * x + sigmoid(g) * y) * w`` on a
    float stream ``x`` in place, with ``y`` the sublayer's result and ``g`` the logits of a gate per coordinate (``None``: no gate) that
    the caller projects from the sublayer's input.  ``alpha`` weighs the skip path (deep post-norm stacks use ``alpha > 1``).
    ``lowp`` receives the new stream rounded to the sublayers' dtype, ready to be the next sublayer's input (one kernel for all of
    it, ``csrc/seqmix/norms.cu``)."""

    def __init__(self, width: int, alpha: float = 1.0, eps: float = 1e-6, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32, device=device), requires_grad=False)
        self.alpha, self.eps = float(alpha), eps

    def apply_(self, x: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor], lowp: Optional[torch.Tensor] = None) -> torch.Tensor:
        from ..ops import seqmix

        C = x.shape[-1]
        seqmix.postnorm_gated_(x.view(-1, C), y.reshape(-1, C), None if gate is None else gate.reshape(-1, C), self.weight, self.alpha,
                               self.eps, None if lowp is None else lowp.view(-1, C))
        return x

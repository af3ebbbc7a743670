"""Several sequence mixers side by side on the same input, summed with fixed weights: ``sum_i scale_i * mixer_i(h)``.  Every
branch writes its pre-projection features, already times its scale, into its columns of one buffer (``mix(h, ctx, st, out,
out_scale)``), and ONE output projection over the concatenated features — the branches' output matrices side by side — forms the
weighted sum inside the matrix product's float accumulation.  A branch's state entries are prefixed with its name.

``NormedParallelMixers`` is the variant whose branches are each RMS-normed over the model width (a gain per branch) BEFORE they are
summed, ``sum_i scale_i * rms(mixer_i(h)) * w_i``: every branch runs to its own output, and the normed sum is accumulated in
float."""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import seqmix


class ParallelMixers(nn.Module):
    def __init__(self, branches: Dict[str, nn.Module], scales: Sequence[float]):
        super().__init__()
        assert len(branches) == len(scales) and all(hasattr(m, "mix") and hasattr(m, "out_features") for m in branches.values())
        self.branches = nn.ModuleDict(branches)
        self.scales = [float(s) for s in scales]
        self._o = None

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {f"{name}.{k}": v for name, m in self.branches.items() for k, v in m.state_spec().items()}

    def _joint_o(self) -> torch.Tensor:
        mats = [m.o for m in self.branches.values()]
        key = tuple((w.data_ptr(), w._version) for w in mats)
        if self._o is None or self._o[0] != key:
            self._o = (key, torch.cat([w.detach() for w in mats], 1).contiguous())
        return self._o[1]

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        total = sum(m.out_features for m in self.branches.values())
        feats = torch.empty(B * S, total, dtype=h.dtype, device=h.device)
        off = 0
        for (name, m), scale in zip(self.branches.items(), self.scales):
            sub = {k[len(name) + 1:]: v for k, v in st.items() if k.startswith(name + ".")}
            m.mix(h, ctx, sub, feats[:, off:off + m.out_features], scale)
            off += m.out_features
        return F.linear(feats, self._joint_o()).view(B, S, -1)


class NormedParallelMixers(nn.Module):
    def __init__(self, branches: Dict[str, nn.Module], scales: Sequence[float], width: int, eps: float, device=None):
        super().__init__()
        assert len(branches) == len(scales)
        self.branches = nn.ModuleDict(branches)
        self.scales, self.eps = [float(s) for s in scales], eps
        # every branch's gain, already times its scale
        self.out_norms = nn.ParameterDict({name: nn.Parameter(torch.ones(width, dtype=torch.float32, device=device), requires_grad=False)
                                           for name in branches})

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {f"{name}.{k}": v for name, m in self.branches.items() for k, v in m.state_spec().items()}

    @torch.no_grad()
    def set_gain(self, name: str, w: torch.Tensor) -> None:
        """Checkpoint gain of branch ``name`` → the stored gain times the branch's scale."""
        scale = self.scales[list(self.branches).index(name)]
        self.out_norms[name].copy_(w.to(device=self.out_norms[name].device, dtype=torch.float32) * scale)

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        """→ float ``[B,S,width]``."""
        B, S, W = h.shape
        acc = None
        for name, m in self.branches.items():
            sub = {k[len(name) + 1:]: v for k, v in st.items() if k.startswith(name + ".")}
            y = m(h, ctx, sub).view(B * S, W)
            if acc is None:
                acc = seqmix.rms_norm(y, self.out_norms[name], self.eps, None, torch.float32)
            else:
                seqmix.add_rms_norm_(acc, y, self.out_norms[name], self.eps)
        return acc.view(B, S, W)

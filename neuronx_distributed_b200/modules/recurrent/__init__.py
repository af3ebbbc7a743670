"""Recurrent sequence mixers: layers whose memory of the past is a fixed-size state carried from token to token (float), served by
the scan kernels of ``csrc/seqmix/linear_recurrence.cu`` (decay per key channel or fixed per head; real-gated LRU; minGRU) and ``csrc/seqmix/matrix_recurrence.cu``
(matrix memories: gated delta rule with a decay per head or per head and key channel, selective state space)."""
from .gla import GatedLinearAttention  # noqa: F401
from .rglru import RealGatedLRUBlock  # noqa: F401
from .mingru import MinGRU  # noqa: F401
from .delta_rule import GatedDeltaRule  # noqa: F401
from .ssd import SelectiveStateSpace  # noqa: F401
from .retention import Retention  # noqa: F401

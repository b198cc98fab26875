"""pararnn_b200 — B200-native CUDA backend for ParaRNN's parallel training hot path.

Public surface mirrors the part of the reference package that the hot path touches:
``NewtonConfig``, ``NewtonStats``, ``NewtonDivergenceError``, ``newton_apply``,
``sequential_apply``, ``verify_agreement`` / ``AgreementReport``, ``ParaRNN`` and the cells.
"""

from .cells import ParaCfC, ParaGRU, ParaLSTM, ParaNLRU, ParaSLSTM, ParaTitans
from .config import (
    NewtonConfig,
    NewtonDivergenceError,
    NewtonStats,
    compile_safe_config,
    slstm_auto_picard,
    slstm_picard_next,
)
from .decode import can_decode_step, decode_step, decode_wx
from .layers import ParaRNN
from .newton import newton_apply
from .sequential import sequential_apply
from .verify import AgreementError, AgreementReport, default_agreement_atol, verify_agreement
from . import custom_ops  # noqa: E402,F401  registers torch.ops.pararnn_b200.*

__version__ = "0.2.0"
__all__ = [
    "AgreementError", "AgreementReport", "NewtonConfig", "NewtonDivergenceError", "NewtonStats",
    "ParaCfC", "ParaGRU", "ParaLSTM", "ParaNLRU", "ParaRNN", "ParaSLSTM", "ParaTitans", "can_decode_step", "compile_safe_config", "decode_step",
    "decode_wx",
    "default_agreement_atol", "newton_apply", "sequential_apply", "slstm_auto_picard",
    "slstm_picard_next", "verify_agreement",
]

"""pararnn_b200 — B200-native CUDA backend for ParaRNN's parallel training hot path.

Public surface mirrors the part of the reference package that the hot path touches:
``NewtonConfig``, ``NewtonStats``, ``NewtonDivergenceError``, ``newton_apply``,
``sequential_apply``, ``verify_agreement`` / ``AgreementReport``, ``ParaRNN`` and the cells.
"""

from .cells import ParaGRU, ParaNLRU, ParaSLSTM
from .config import (
    NewtonConfig,
    NewtonDivergenceError,
    NewtonStats,
    compile_safe_config,
    slstm_auto_picard,
    slstm_picard_next,
)
from .layers import ParaRNN
from .newton import newton_apply
from .sequential import sequential_apply
from .verify import AgreementError, AgreementReport, default_agreement_atol, verify_agreement

__version__ = "0.1.0"
__all__ = [
    "AgreementError", "AgreementReport", "NewtonConfig", "NewtonDivergenceError", "NewtonStats",
    "ParaGRU", "ParaNLRU", "ParaRNN", "ParaSLSTM", "compile_safe_config",
    "default_agreement_atol", "newton_apply", "sequential_apply", "slstm_auto_picard",
    "slstm_picard_next", "verify_agreement",
]

"""Agreement check between the parallel solve and the sequential unroll
(reference ``verify.py:32-217``): same report fields and default tolerances."""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

import torch
from torch import Tensor, nn

from .config import NewtonConfig, NewtonStats
from .newton import newton_apply
from .sequential import sequential_apply


@dataclass(frozen=True)
class AgreementReport:
    ok: bool
    max_abs: float
    max_rel: float
    mean_abs: float
    atol: float
    rtol: float
    shape: tuple[int, ...]
    dtype: str
    device: str
    newton_iters: int | None = None
    max_residual: float | None = None
    path: str = "cell"

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


class AgreementError(RuntimeError):
    def __init__(self, message: str, report: AgreementReport) -> None:
        super().__init__(message)
        self.report = report


def default_agreement_atol(dtype: torch.dtype) -> float:
    """1e-4 for float32/float64, 1e-2 for float16/bfloat16."""
    return 1e-2 if dtype in (torch.float16, torch.bfloat16) else 1e-4


def verify_agreement(module: nn.Module, x: Tensor, *, config: NewtonConfig | None = None,
                     h0: Tensor | None = None, atol: float | None = None, rtol: float = 0.0,
                     raise_on_fail: bool = False, cu_seqlens: Tensor | None = None) -> AgreementReport:
    if x.dim() < 2:
        raise ValueError(f"x must be at least rank-2 (B, T, ...), got shape {tuple(x.shape)}")
    if cu_seqlens is not None:
        raise NotImplementedError("packed cu_seqlens batches are not covered yet")
    atol_v = float(default_agreement_atol(x.dtype) if atol is None else atol)
    from .layers import ParaRNN

    target = module.rnn if hasattr(module, "rnn") and isinstance(module.rnn, ParaRNN) else module
    with torch.no_grad():
        if isinstance(target, ParaRNN):
            was = target.training
            target.train()
            parallel = target(x)
            stats = target.last_stats
            target.eval()
            sequential = target(x)
            target.train(was)
            path = "para_rnn"
        else:
            if not hasattr(target, "step"):
                raise TypeError(f"verify_agreement needs a cell, ParaRNN or block, got {type(module).__name__}")
            stats = NewtonStats()
            parallel = newton_apply(target, x, config, h0=h0, stats=stats)
            sequential = sequential_apply(target, x, h0)
            path = "cell"
        diff = (parallel.float() - sequential.float()).abs()
        max_abs = float(diff.amax())
        mean_abs = float(diff.mean())
        denom = sequential.float().abs().clamp_min(torch.finfo(sequential.dtype).eps)
        max_rel = float((diff / denom).amax())
        ok = bool(torch.allclose(parallel.float(), sequential.float(), atol=atol_v, rtol=float(rtol)))
    report = AgreementReport(
        ok=ok, max_abs=max_abs, max_rel=max_rel, mean_abs=mean_abs, atol=atol_v, rtol=float(rtol),
        shape=tuple(int(s) for s in parallel.shape), dtype=str(parallel.dtype).replace("torch.", ""),
        device=str(parallel.device),
        newton_iters=None if stats is None else int(stats.iters),
        max_residual=None if stats is None else float(stats.max_residual), path=path)
    if raise_on_fail and not ok:
        raise AgreementError(
            f"parallel vs sequential max_abs={max_abs:.3e} exceeds atol={atol_v:.3e} "
            f"(rtol={rtol:.3e}); shape={report.shape} dtype={report.dtype} path={path}", report)
    return report

"""Python faces of the kernels in ``csrc/parallel.cu``: the sum of a layer's scaled branches into the residual stream,
fused with one or two RMS norms of the same row, and a scale of float32 rows in place."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ._lib import KernelError, c_float, c_int, c_longlong, check, dt_code, fn, ptr, require_cuda, stream


def _terms(h: torch.Tensor, terms: Sequence):
    terms = list(terms)
    if len(terms) > 2:
        raise KernelError("at most two scaled terms are added in one pass")
    out = []
    for x, s in terms:
        require_cuda(x, s)
        if x.shape != h.shape:
            raise KernelError("a term must have the residual stream's shape")
        if s is not None and (s.dtype != torch.float32 or s.numel() != h.shape[1]):
            raise KernelError("a term's factor is a float32 vector over the width")
        out.append((x, s))
    while len(out) < 2:
        out.append((None, None))
    return out


def add_scaled_rmsnorm(h: torch.Tensor, terms: Sequence, gains: Sequence[torch.Tensor], eps: float, out_dtype: torch.dtype,
                       rows: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """``h += sum_i s_i * x_i`` (``terms``: up to two ``(x_i [T, width], s_i float32 [width] or None)``; written back
    unless ``rows`` is given), then one RMS norm per entry of ``gains`` (one or two float32 vectors) of the same rows:
    ``rmsnorm(h) * gain`` in ``out_dtype``, for all rows or for ``rows`` (int32) only."""
    require_cuda(h, rows, *gains)
    if h.dtype != torch.float32 or any(g.dtype != torch.float32 or g.numel() != h.shape[1] for g in gains):
        raise KernelError("the residual stream and norm gains are float32, one gain per column")
    if not 1 <= len(gains) <= 2:
        raise KernelError("one or two norms")
    (a, sa), (b, sb) = _terms(h, terms)
    T, H = h.shape
    R = T if rows is None else rows.numel()
    ys = [torch.empty((R, H), dtype=out_dtype, device=h.device) for _ in gains]
    check(fn("parallel", "sx_add_scaled_rmsnorm")(
        ptr(h), ptr(a), c_int(dt_code(a.dtype) if a is not None else 0), ptr(sa),
        ptr(b), c_int(dt_code(b.dtype) if b is not None else 0), ptr(sb), ptr(gains[0]),
        ptr(gains[1] if len(gains) > 1 else None), c_float(eps), ptr(ys[0]), ptr(ys[1] if len(ys) > 1 else None), ptr(rows),
        c_int(R), c_int(H), c_int(dt_code(out_dtype)), c_int(1 if rows is None else 0), stream()), "add_scaled_rmsnorm")
    return ys


def add_scaled(h: torch.Tensor, terms: Sequence) -> None:
    """``h += sum_i s_i * x_i`` in place (float32 ``h``)."""
    require_cuda(h)
    if h.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    (a, sa), (b, sb) = _terms(h, terms)
    check(fn("parallel", "sx_add_scaled")(ptr(h), ptr(a), c_int(dt_code(a.dtype) if a is not None else 0), ptr(sa), ptr(b),
                                          c_int(dt_code(b.dtype) if b is not None else 0), ptr(sb), c_int(h.shape[0]),
                                          c_int(h.shape[1]), stream()), "add_scaled")


def scale_rows(x: torch.Tensor, s: float) -> None:
    """``x *= s`` in place (float32)."""
    require_cuda(x)
    if x.dtype != torch.float32:
        raise KernelError("scale_rows takes float32")
    check(fn("parallel", "sx_scale_rows")(ptr(x), c_longlong(x.numel()), c_float(s), stream()), "scale_rows")

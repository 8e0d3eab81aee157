"""Python face of the kernels in ``csrc/mlstm.cu``: a matrix memory per head with exponential gates."""
from __future__ import annotations

import torch

from ._lib import KernelError, c_float, c_int, check, dt_code, fn, ptr, require_cuda, stream


_PIECE = [0]

# portions of at least this many tokens (the longest of a step) run in pieces
PIECES_MIN_TOKENS = 32


def mlstm(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, g_off: int, gates: torch.Tensor, bias: torch.Tensor,
          cap: float, q_scale: float, heads: int, dim: int, vdim: int, gain: torch.Tensor, eps: float, den_eps: float,
          S: torch.Tensor, n: torch.Tensor, m: torch.Tensor, ctx) -> torch.Tensor:
    """The recurrence over the step's tokens, per head: ``i = cap tanh(zi / cap)``, ``f = logsigmoid(cap tanh(zf / cap))``,
    ``m' = max(f + m, i)``, ``S' = exp(f + m - m') S + exp(i - m') k v^T``, ``n'`` likewise with ``k`` alone,
    ``o = S'^T q / (max(|n' . q|, exp(-m')) + den_eps)``; the result is ``o / rms(o) * gain * sigmoid(g)``
    ``[T, heads * vdim]`` in ``proj``'s dtype.

    ``proj [T, row]`` holds q, k (``heads * dim`` columns each from ``q_off``, ``k_off``; q is multiplied by ``q_scale``),
    v and the output gate's pre-activation (``heads * vdim`` from ``v_off``, ``g_off``); ``gates`` float32
    ``[T, 2 * heads]`` the pre-activations ``zi`` (first) and ``zf`` without their biases ``bias`` float32 ``[2 * heads]``.
    ``S [slots, heads, dim, vdim]``, ``n [slots, heads, dim]``, ``m [slots, heads]`` float32 are moved on."""
    require_cuda(proj, gates, bias, gain, S, n, m)
    for t in (gates, bias, gain, S, n, m):
        if t.dtype != torch.float32:
            raise KernelError("mlstm: gates, biases, gains and states are float32")
    T, row = proj.shape
    if (tuple(S.shape[1:]) != (heads, dim, vdim) or tuple(n.shape[1:]) != (heads, dim) or tuple(m.shape[1:]) != (heads,)
            or tuple(gates.shape) != (T, 2 * heads) or bias.numel() != 2 * heads or gain.numel() != heads * vdim):
        raise KernelError("mlstm: the states, gates or gains do not fit the heads")
    if max(q_off, k_off) + heads * dim > row or max(v_off, g_off) + heads * vdim > row:
        raise KernelError("mlstm: the columns do not fit the projection")
    out = torch.empty((T, heads * vdim), dtype=proj.dtype, device=proj.device)
    # long portions run in pieces of 64 tokens (four kernels); single tokens and short portions walk the tokens
    tok = info = st = None
    pieces, launches = 0, 1
    if ctx.max_new >= PIECES_MIN_TOKENS and fn("mlstm", "sx_mlstm_pieces_fit")(c_int(dim), c_int(vdim)):
        if _PIECE[0] == 0:
            _PIECE[0] = int(fn("mlstm", "sx_mlstm_piece_tokens")())
        pieces, launches = (ctx.max_new + _PIECE[0] - 1) // _PIECE[0], 4
        tok = torch.empty((T, heads, 2), dtype=torch.float32, device=proj.device)
        info = torch.empty((ctx.n_seqs, pieces, heads, 4), dtype=torch.float32, device=proj.device)
        st = torch.empty((ctx.n_seqs, pieces, heads, dim * vdim + dim), dtype=torch.float32, device=proj.device)
    check(fn("mlstm", "sx_mlstm")(ptr(proj), c_int(row), c_int(q_off), c_int(k_off), c_int(v_off), c_int(g_off), ptr(gates),
                                  ptr(bias), c_float(cap), c_float(q_scale), ptr(gain), c_float(eps), c_float(den_eps),
                                  ptr(S), ptr(n), ptr(m), ptr(out), ptr(ctx.cu_seqlens), ptr(ctx.seq_slots), c_int(ctx.n_seqs),
                                  c_int(heads), c_int(dim), c_int(vdim), c_int(dt_code(proj.dtype)), ptr(tok), ptr(info), ptr(st),
                                  c_int(pieces), stream()), "mlstm", launches=launches)
    return out

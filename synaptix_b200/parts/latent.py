"""Attention over a cached latent: keys and values of all heads are made from one small vector per token.

Per token the layer keeps ``c = rmsnorm(Wdkv x)[:kv_rank] * gain`` and one rotated key part of ``rot_dim`` elements
that all heads share (the last rows of ``Wdkv``, not normed).  Head ``h`` has the key ``[Wuk_h c | k_rot]`` and the
value ``Wuv_h c``; its query ``[q_h | q_rot_h]`` comes through a latent of its own,
``Wuq (rmsnorm(Wdq x) * gain)``.  Scores are ``(q_h . Wuk_h c + q_rot_h . k_rot) * scale`` over the visible keys
(causal, optionally a sliding window of ``window`` positions, the query's own included), ordinary softmax; head
``h``'s result is multiplied by ``sigmoid(Wg x)_h`` and the heads go through ``Wo``.

The per-head keys and values are never formed.  ``q_h . Wuk_h c = (Wuk_h^T q_h) . c``, so the query is taken into the
latent's space once (``q' = [Wuk_h^T q_h | q_rot_h]``, ``kv_rank + rot_dim`` elements), attention runs with ONE key
row ``[c | k_rot]`` per token for all heads, its weights are applied to ``c`` itself, and ``Wuv_h`` is applied to the
weighted latent afterwards.  The cache therefore holds keys only (``KVRequest(keys_only=True)``), one head of
``kv_rank + rot_dim`` elements; the values are its first ``kv_rank`` elements.  Queries in the latent's space and the
weighted latents stay 32-bit.

A layer built with ``own_kv=False`` has no ``Wdkv``: the schedule gives it the cache entry of the layer whose latent
it reads (``LayerRun(..., write_cache=False)``); its ``Wuk``, ``Wuv``, queries, window and gate are its own.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from .. import ops
from ..cache.store import KVRequest, KVView
from ..weights.loader import TensorSpec
from .base import Mixer, Part, PositionEncoding, Runtime, StepContext, to_device_f32, to_device_matrix
from .linear import Linear


class LatentAttention(Mixer):
    accepts_lazy_input = False
    can_defer_output = False

    NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
             "g": "g", "o": "o"}

    def __init__(self, prefix: str, width: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, *,
                 scale: float, position: PositionEncoding, norm_eps: float, window: Optional[int] = None,
                 keep_window="own", own_kv: bool = True, gated: bool = True,
                 names: Optional[Mapping[str, str]] = None):
        """``keep_window``: how many latest keys the cache entry must keep (the largest window of the layers that read
        it, ``None`` for all); ``"own"``: this layer's ``window``."""
        self.prefix, self.width = prefix, width
        self.heads, self.dim, self.rot_dim, self.vdim = heads, dim, rot_dim, vdim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.scale = float(scale)
        self.position = position
        self.norm_eps = float(norm_eps)
        self.window = window
        self.keep_window = window if keep_window == "own" else keep_window
        self.own_kv, self.gated = bool(own_kv), bool(gated)
        self.names = n = dict(self.NAMES, **(names or {}))
        p = prefix
        parts = [(p + n["dq"], q_rank)]
        self.col_dkv = self.col_g = -1
        if own_kv:
            self.col_dkv = q_rank
            parts.append((p + n["dkv"], kv_rank + rot_dim))
        if gated:
            self.col_g = sum(o for _, o in parts)
            parts.append((p + n["g"], heads))
        self.proj = Linear([x for x, _ in parts], width, [o for _, o in parts])
        self.uq = Linear(p + n["uq"], q_rank, heads * (dim + rot_dim))
        self.o = Linear(p + n["o"], heads * vdim, width)
        self.dq_gain = self.dkv_gain = self.uk = self.uv = None

    def children(self) -> List[Part]:
        return [self.proj, self.uq, self.o, self.position]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, n = self.prefix, self.names
        specs = {p + n["dq_norm"]: TensorSpec((self.q_rank,), "gain"),
                 p + n["uk"]: TensorSpec((self.heads * self.dim, self.kv_rank), "matrix"),
                 p + n["uv"]: TensorSpec((self.heads * self.vdim, self.kv_rank), "matrix")}
        if self.own_kv:
            specs[p + n["dkv_norm"]] = TensorSpec((self.kv_rank,), "gain")
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        p, n = self.prefix, self.names
        self.dq_gain = to_device_f32(tensors[p + n["dq_norm"]], rt)
        if self.own_kv:
            self.dkv_gain = to_device_f32(tensors[p + n["dkv_norm"]], rt)
        self.uk = to_device_matrix(tensors[p + n["uk"]], rt)          # [heads * dim, kv_rank]
        self.uv = to_device_matrix(tensors[p + n["uv"]], rt)          # [heads * vdim, kv_rank]

    def cache_request(self):
        if not self.own_kv:
            return None
        return KVRequest(1, self.kv_rank + self.rot_dim, self.keep_window, keys_only=True)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_view: KVView, write_cache: bool = True):
        if write_cache != self.own_kv:
            raise ValueError("a latent attention layer writes the cache exactly when it has a key/value latent of its own")
        rot = self.position.rotation()
        inv_freq, rot_dims = rot if rot is not None else (None, 0)
        pairs = bool(getattr(self.position, "pairs", False))
        bt = ctx.block_tables[cache_view.group]
        p = self.proj.forward(x)
        cq = ops.latent_prepare(p, self.q_rank, self.col_dkv, self.kv_rank, self.rot_dim, self.dq_gain, self.dkv_gain,
                                self.norm_eps, inv_freq, rot_dims, pairs, ctx, bt, cache_view.k if write_cache else None)
        q = self.uq.forward(cq)
        qa = ops.latent_query(q, self.uk, self.heads, self.dim, self.rot_dim, self.kv_rank, inv_freq, rot_dims, pairs, ctx)
        ol = ops.latent_attention(qa, cache_view.k, ctx, bt, self.heads, self.kv_rank, self.rot_dim, self.scale, self.window)
        y = ops.latent_output(ol, self.uv, self.heads, self.vdim, self.kv_rank, p, self.col_g, x.dtype)
        return self.o.forward(y)

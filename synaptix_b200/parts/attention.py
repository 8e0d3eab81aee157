"""Grouped-query attention over the paged cache: the mixer of the Qwen3 dense decoder.

In the reference's order (crates/synaptix-models/llm/common/src/model.rs:1715-1734,
1781-1782, 1872-1878):
``q,k,v = x Wq^T, x Wk^T, x Wv^T`` -> per-head RMSNorm of q and k (optional) ->
rotation of q and k (optional) -> k, v appended to the cache ->
``softmax(q k^T * scale + causal mask) v`` with query head ``h`` reading kv head
``h // (nh / nkv)`` -> ``Wo``.  Key ``j`` is visible to the query at position ``p``
iff ``j <= p`` and, with a window ``w``, ``j > p - w``.

Sizes and constants are parameters: heads, kv heads, head size, norm eps, scale,
window, the position encoding.  The three projections run as one product.

Further options, all off by default: ``v_head_dim`` (values of another size than
keys), ``softcap`` (``score <- softcap * tanh(score / softcap)`` after the scale),
``sinks`` (a learned number per query head whose exponential joins the softmax's
denominator; it has no key and no value and is neither scaled nor capped), ``chunk``
(position ``p`` sees key ``j <= p`` only if ``j // chunk == p // chunk``, chunks
counted from position 0 of the sequence).  ``names`` maps q, k, v, o, q_norm, k_norm
and sink to the tensor names behind the prefix.

An attention can also run as one of several mixers that share an input product
(``input_parts``, ``output_part``, ``mix``): the owner stacks the projections of
all of them, and each writes what its output projection reads into its columns of
one buffer.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

from .. import ops
from ..cache.store import KVRequest, KVView
from ..weights.loader import TensorSpec
from .base import Mixer, Part, PositionEncoding, Runtime, StepContext, to_device_f32
from .linear import Linear


class Attention(Mixer):
    accepts_lazy_input = True      # x goes straight into the fused q/k/v product
    can_defer_output = True        # the output projection may be handed on unrun

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sinks"}

    def __init__(self, prefix: str, width: int, n_heads: int, n_kv_heads: int, head_dim: int, *,
                 position: PositionEncoding, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, scale: Optional[float] = None,
                 v_head_dim: Optional[int] = None, softcap: Optional[float] = None, sinks: bool = False,
                 chunk: Optional[int] = None, names: Optional[Mapping[str, str]] = None, shared: bool = False):
        """``shared``: the part owns no projections; an owner stacks ``input_parts()`` / ``output_part()`` of
        several mixers and calls ``mix``."""
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if chunk is not None and chunk <= 0:
            raise ValueError("chunk must be > 0")
        self.prefix = prefix
        self.width = width
        self.nh, self.nkv, self.hd = n_heads, n_kv_heads, head_dim
        self.vd = head_dim if v_head_dim is None else v_head_dim
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.softcap = None if not softcap else float(softcap)
        self.has_sinks = bool(sinks)
        self.chunk = chunk
        self.names = dict(self.NAMES, **(names or {}))
        self.shared = bool(shared)
        # the plain form: what the kernels that take the projection as it is (or prepare the heads in its epilogue) assume
        self.is_plain = (self.vd == head_dim and self.softcap is None and not self.has_sinks and chunk is None)
        self.qkv = self.o = None
        if not shared:
            names_in, outs = zip(*self.input_parts())
            self.qkv = Linear(list(names_in), width, list(outs))
            self.o = Linear(self.output_part()[0], self.output_part()[1], width)
        self.wq: Optional[torch.Tensor] = None
        self.wk: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None

    def input_parts(self):
        """``(tensor name, outputs)`` of the projections, in the order of their columns."""
        n, p = self.names, self.prefix
        return [(p + n["q"], self.nh * self.hd), (p + n["k"], self.nkv * self.hd), (p + n["v"], self.nkv * self.vd)]

    def output_part(self):
        """``(tensor name, inputs)`` of the output projection."""
        return self.prefix + self.names["o"], self.nh * self.vd

    def children(self) -> List[Part]:
        return ([] if self.shared else [self.qkv, self.o]) + [self.position]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {}
        if self.qk_norm_eps is not None:
            specs[self.prefix + self.names["q_norm"]] = TensorSpec((self.hd,), "gain")
            specs[self.prefix + self.names["k_norm"]] = TensorSpec((self.hd,), "gain")
        if self.has_sinks:
            specs[self.prefix + self.names["sink"]] = TensorSpec((self.nh,), "bias")
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        if self.qk_norm_eps is not None:
            self.wq = to_device_f32(tensors[self.prefix + self.names["q_norm"]], rt)
            self.wk = to_device_f32(tensors[self.prefix + self.names["k_norm"]], rt)
        if self.has_sinks:
            self.sinks = to_device_f32(tensors[self.prefix + self.names["sink"]], rt)

    def cache_request(self):
        return KVRequest(self.nkv, self.hd, self.window, None if self.vd == self.hd else self.vd, self.chunk)

    def mix(self, proj: torch.Tensor, col: int, ctx: StepContext, cache_view: KVView, write_cache: bool = True,
            out: Optional[torch.Tensor] = None, out_col: int = 0, out_scale: float = 1.0) -> torch.Tensor:
        """Head preparation, cache write and attention from a projection ``proj [T, row]`` whose columns from ``col``
        on are this part's q, k and v heads; what the output projection reads goes, times ``out_scale``, into the
        columns of ``out`` from ``out_col`` on (default: a new ``[T, nh * vd]``)."""
        T = proj.shape[0]
        rot = self.position.rotation()
        inv_freq, rotary_dim = rot if rot is not None else (None, 0)
        bt = ctx.block_tables[cache_view.group]
        q = torch.empty((T, self.nh * self.hd), dtype=proj.dtype, device=proj.device)
        ops.qkv_prepare(proj, q, cache_view.k if write_cache else None, cache_view.v if write_cache else None,
                        self.wq, self.wk, inv_freq, rotary_dim,
                        self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                        ctx.positions, ctx.seq_of_token, bt, self.nh, self.nkv, self.hd, vd=self.vd, col=col)
        return ops.attention(q, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd, self.scale, self.window,
                             vd=self.vd, softcap=self.softcap, sinks=self.sinks, chunk=self.chunk,
                             out=out, out_col=out_col, out_scale=out_scale)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_view: KVView, write_cache: bool = True,
                defer_output: bool = False) -> torch.Tensor:
        out = self.o.deferred if defer_output else self.o.forward
        if not self.is_plain:
            return out(self.mix(self.qkv.forward(x), 0, ctx, cache_view, write_cache))
        T = x.shape[0]
        rot = self.position.rotation()
        inv_freq, rotary_dim = rot if rot is not None else (None, 0)
        bt = ctx.block_tables[cache_view.group]
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        if (isinstance(x, torch.Tensor)
                and ops.projection_prepares_heads(T, x.shape[1], x.dtype, self.qkv.weight.dtype, self.nh, self.nkv, self.hd,
                                                  rotary_dim)
                and not ctx.all_single):
            # prompt steps: the projection's epilogue prepares the heads and writes the cache
            q = ops.project_and_prepare(x, self.qkv.weight, cache_view.k if write_cache else None,
                                        cache_view.v if write_cache else None, self.wq, self.wk, inv_freq, eps, ctx, bt,
                                        self.nh, self.nkv, self.hd)
            return out(ops.attention(q, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd, self.scale, self.window))
        qkv = self.qkv.forward(x)
        if ops.decode_attention_takes_projection(qkv.dtype, self.nh, self.nkv, self.hd, rotary_dim, ctx):
            # single-token steps: the attention kernel prepares the heads and writes the cache itself
            a = ops.attention_from_projection(qkv, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd,
                                              self.scale, self.window, self.wq, self.wk, inv_freq,
                                              self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, write_cache)
            return out(a)
        q = torch.empty((T, self.nh * self.hd), dtype=qkv.dtype, device=qkv.device)
        ops.qkv_prepare(qkv, q, cache_view.k if write_cache else None, cache_view.v if write_cache else None,
                        self.wq, self.wk, inv_freq, rotary_dim,
                        self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                        ctx.positions, ctx.seq_of_token, bt, self.nh, self.nkv, self.hd,
                        pages_like=cache_view.k)
        a = ops.attention(q, cache_view.k, cache_view.v, ctx, bt, self.nh, self.nkv, self.hd,
                          self.scale, self.window)
        return out(a)

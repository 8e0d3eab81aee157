"""The Pidutar decoder put together from parts.

A layer is a ``ParallelBlock``: mixer and feed-forward read the same stream, each behind an RMS norm of its own whose
gain is stored around zero (``1 + w``), each times a learned vector over the width, and the stream takes
``residual_mult`` times their sum.  Mixers by layer type:

* ``mlstm``: ``MLSTM``, a matrix memory per head with capped exponential gates;
* ``latent_attention``: ``LatentAttention``: keys and values made from a cached latent, queries through a latent of
  their own, a rotated part of ``rot_dim`` elements with neighbouring elements paired (``RotaryPairs``), a sliding
  window, a gate per head.  A layer with ``kv_from`` has no key/value latent: its run in the schedule names the cache
  entry of the layer it reads and writes nothing (``LayerRun(layer, entry, write_cache=False)``); that entry keeps as
  many keys as the largest window among its readers.

The feed-forward is a ``MixtureOfExperts`` (absent in layers whose ``mlp`` is null).  The embedding's rows are
multiplied by ``embedding.scale``, the logits by ``logit_scale``; the final norm's gain is ``1 + w`` as well.

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1|norm2``, ``l<i>.ls1|ls2``,
``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``.
"""
from __future__ import annotations

from ..config.pidutar import PidutarConfig
from ..config.registry import register_architecture
from ..parts import (Embedding, LatentAttention, MixtureOfExperts, MLSTM, NoPosition, OutputHead, ParallelBlock, RMSNorm,
                     RotaryPairs)
from .decoder import DecoderModel, LayerRun

NORM_OFFSET = 1.0           # the norms' stored weights lie around zero: gain = 1 + w


def build_pidutar(cfg: PidutarConfig) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    embedding = Embedding("embed", cfg.vocab, W, scale=cfg.embedding_scale)
    # a cache entry keeps what the widest window among its readers needs (None: everything)
    keep = {}
    for i, spec in enumerate(cfg.layers):
        if spec.type == "latent_attention":
            owner = i if spec.attention.kv_from is None else spec.attention.kv_from
            w = spec.attention.window
            if owner not in keep:
                keep[owner] = w
            elif keep[owner] is not None:
                keep[owner] = None if w is None else max(keep[owner], w)
    layers, schedule, entry_of = [], [], {}
    for i, spec in enumerate(cfg.layers):
        p = f"l{i}."
        if spec.type == "mlstm":
            m = spec.memory
            mixer = MLSTM(p + "mix.", W, m.heads, m.dim, m.vdim, gate_cap=m.gate_cap, unit_norm_eps=eps)
        else:
            a = spec.attention
            position = RotaryPairs(a.rot_dim, a.rot_base, rotary_dim=a.rot_dims) if a.rot_dims else NoPosition()
            own = a.kv_from is None
            mixer = LatentAttention(p + "mix.", W, a.heads, a.dim, a.rot_dim, a.vdim, a.q_rank, a.kv_rank, scale=a.scale,
                                    position=position, norm_eps=eps, window=a.window,
                                    keep_window=keep[i] if own else "own", own_kv=own)
        norm2 = ffn = None
        if spec.mlp is not None:
            f = spec.mlp
            norm2 = RMSNorm(p + "norm2", W, eps, offset=NORM_OFFSET)
            ffn = MixtureOfExperts(p + "mlp.", W, f.ff, f.experts, f.top, scale=f.scale)
        layers.append(ParallelBlock(RMSNorm(p + "norm1", W, eps, offset=NORM_OFFSET), mixer, norm2, ffn,
                                    scale_names=(p + "ls1", p + "ls2"), mult=cfg.residual_mult))
        if spec.type == "latent_attention" and spec.attention.kv_from is not None:
            schedule.append(LayerRun(i, entry_of[spec.attention.kv_from], write_cache=False))
        else:
            entry_of[i] = len(entry_of)
            schedule.append(LayerRun(i, entry_of[i]))
    return DecoderModel(cfg, embedding, layers, RMSNorm("final.norm", W, eps, offset=NORM_OFFSET),
                        OutputHead("head", cfg.vocab, W, False, embedding, scale=cfg.logit_scale), schedule=schedule)


register_architecture(PidutarConfig, build_pidutar)

"""The Vemedra decoder put together from parts.

A layer is ``ConvPreNormBlock``: RMS norm, a short causal convolution over time added to its input, the mixer; then
the same in front of a capped gated feed-forward (absent in layers whose ``mlp`` is null).  Mixers by layer type:

* ``mingru``: ``MinGRU``;
* ``parallel``: ``ParallelMixers`` of softmax attention (grouped heads, rotate-half rotation of the first ``rot.dims``
  elements of a head, scores scaled, then capped by ``softcap * tanh(. / softcap)``, chunks of ``mask.size`` positions,
  a sink per head in the denominator) and ``Retention`` (fixed decay per head, k scaled by ``dim^-1/2``, unit norm
  per head, ``silu`` gate), added with the two scales of the configuration.

A stretch of layers may run several times with the same weights (``loop``): every pass has cache entries of its own;
before each pass but the first the embedding output is added to the stream again, and before every pass a learned
vector of that pass (``loop.step[t]``).  The schedule says all of that as data (``LayerRun``, ``Inject``).

Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.step``, and per layer ``l<i>.norm1|norm2``,
``l<i>.canon1|canon2``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vemedra import VemedraConfig
from ..parts import (Attention, CappedGLU, ConvPreNormBlock, Embedding, MinGRU, NoPosition, OutputHead, ParallelMixers,
                     Retention, RMSNorm, RotaryHalf, TokenConv)
from .decoder import DecoderModel, Inject, LayerRun, StreamVectors

GLU_ALPHA = 1.702          # g * sigmoid(1.702 g): the sigmoid form of GELU


def build_vemedra(cfg: VemedraConfig) -> DecoderModel:
    W, eps, taps = cfg.width, cfg.norm_eps, cfg.canon_taps
    embedding = Embedding("embed", cfg.vocab, W)
    layers = []
    for i, spec in enumerate(cfg.layers):
        p = f"l{i}."
        if spec.type == "mingru":
            mixer = MinGRU(p + "mix.", W, spec.mingru_width)
        else:
            a, r = spec.left, spec.right
            position = RotaryHalf(a.dim, a.rot_base, rotary_dim=a.rot_dims) if a.rot_dims else NoPosition()
            left = Attention(p + "mix.left.", W, a.heads, a.kv_heads, a.dim, position=position, scale=a.scale,
                             v_head_dim=a.vdim, softcap=a.softcap, sinks=True, chunk=a.chunk, shared=True,
                             names={"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink"})
            right = Retention(p + "mix.right.", W, r.heads, r.dim, r.vdim, r.decay, unit_norm_eps=eps, gated=True,
                              shared=True)
            mixer = ParallelMixers(W, [left, right], [spec.left_scale, spec.right_scale])
        if spec.ff is None:
            layers.append(ConvPreNormBlock(RMSNorm(p + "norm1", W, eps), TokenConv(p + "canon1", W, taps), mixer))
        else:
            layers.append(ConvPreNormBlock(
                RMSNorm(p + "norm1", W, eps), TokenConv(p + "canon1", W, taps), mixer,
                RMSNorm(p + "norm2", W, eps), TokenConv(p + "canon2", W, taps),
                CappedGLU(p + "mlp.", W, spec.ff, limit=spec.ff_limit, alpha=GLU_ALPHA)))
    schedule = []
    for entry, (layer, opens_pass) in enumerate(cfg.runs()):
        if opens_pass is not None:
            schedule.append(Inject(embedding=opens_pass > 0, row=opens_pass))
        schedule.append(LayerRun(layer, entry))
    vectors = StreamVectors("loop.step", cfg.loop_times, W) if cfg.has_loop else None
    return DecoderModel(cfg, embedding, layers, RMSNorm("final.norm", W, eps),
                        OutputHead("head", cfg.vocab, W, False, embedding), schedule=schedule, stream_vectors=vectors)


register_architecture(VemedraConfig, build_vemedra)

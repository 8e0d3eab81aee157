"""Several mixers side by side on the same input, their outputs added with a weight each:
``sum_i scale_i * mixer_i(x)``.

The mixers are built ``shared`` (see ``Attention``, ``Retention``): this part stacks all their input projections
into ONE product, lets each mixer write what its output projection reads, times its scale, into its columns of one
buffer, and runs the output projections as ONE product over the joined inputs.  The cache entry is the bundle of the
mixers' requests, in their order.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..cache.store import BundleRequest
from .base import Mixer, Part, StepContext
from .linear import JoinedLinear, Linear


class ParallelMixers(Mixer):
    accepts_lazy_input = False
    can_defer_output = True

    def __init__(self, width: int, mixers: Sequence[Mixer], scales: Sequence[float]):
        if len(mixers) != len(scales) or not mixers:
            raise ValueError("one scale per mixer")
        self.width = width
        self.mixers = list(mixers)
        self.scales = [float(s) for s in scales]
        names, outs, self.cols = [], [], []
        for m in self.mixers:
            self.cols.append(sum(outs))
            for n, o in m.input_parts():
                names.append(n)
                outs.append(o)
        self.proj = Linear(names, width, outs)
        o_names, o_ins = zip(*[m.output_part() for m in self.mixers])
        self.out_cols = [sum(o_ins[:i]) for i in range(len(o_ins))]
        self.o = JoinedLinear(list(o_names), list(o_ins), width)

    def children(self) -> List[Part]:
        return [self.proj, self.o] + self.mixers

    def cache_request(self):
        return BundleRequest(tuple(m.cache_request() for m in self.mixers))

    def forward(self, x: torch.Tensor, ctx: StepContext, views, write_cache: bool = True, defer_output: bool = False):
        a = self.proj.forward(x)
        y = torch.empty((a.shape[0], self.o.in_features), dtype=a.dtype, device=a.device)
        for m, col, view, oc, sc in zip(self.mixers, self.cols, views, self.out_cols, self.scales):
            m.mix(a, col, ctx, view, write_cache, out=y, out_col=oc, out_scale=sc)
        return self.o.deferred(y) if defer_output else self.o.forward(y)

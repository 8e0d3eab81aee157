"""Small Vemedra configurations for the tests: they differ in every size and option."""
import functools
import tempfile

import torch

import plain_vemedra as PV


def _soft(heads, kv, dim, vdim, scale, softcap, chunk, rot_dims, rot_base):
    d = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, softcap=softcap, mask=dict(size=chunk))
    if rot_dims:
        d["rot"] = dict(dims=rot_dims, base=rot_base)
    return d


def _par(left, right, ls, rs, ff, limit=1.5):
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=ls, right_scale=rs),
                mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


def _gru(width, ff=None, limit=1.0):
    return dict(type="mingru", mixer=dict(width=width), mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


# grouped heads (2 query heads a kv head), values smaller than keys, half of a head rotated, chunks of 10 positions
# (no multiple or divisor of a page), 3 retention heads with key and value sizes that differ, a loop over layers 1..2
# that does not begin at layer 0, a minGRU layer with a feed-forward and a parallel layer without
VA = dict(architecture="Vemedra", vocab=97, width=48, norm=dict(eps=1e-5), canon=dict(taps=3),
          layers=[_par(_soft(4, 2, 16, 8, 0.3, 4.0, 10, 8, 1.0e4), dict(heads=3, dim=8, vdim=12, decay=[0.9, 0.99, 0.5]), 0.7, 1.3, 64),
                  _gru(40, ff=56),
                  _par(_soft(2, 1, 24, 24, 0.2, 30.0, 37, 24, 5.0e5), dict(heads=1, dim=16, vdim=16, decay=[0.97]), 1.0, 0.25, None),
                  _gru(24)],
          loop=dict(start=1, stop=3, times=2))
VA_INIT = dict(seed=3, std_matrix=0.1, std_embedding=0.6, std_gain=0.1, std_bias=0.3)

# 4 taps, one query head a kv head, a chunk of 70, no rotation in the second attention, a loop of one pass over all layers
VB = dict(architecture="Vemedra", vocab=131, width=64, norm=dict(eps=1e-6), canon=dict(taps=4),
          layers=[_gru(80),
                  _par(_soft(3, 3, 32, 16, 0.18, 8.0, 70, 16, 1.0e6), dict(heads=2, dim=32, vdim=8, decay=[0.999, 0.9375]), 0.6, 0.5, 96, limit=2.0),
                  _par(_soft(2, 2, 8, 40, 0.4, 2.5, 64, 0, 0), dict(heads=2, dim=12, vdim=20, decay=[0.8, 0.995]), 0.5, 0.75, 40)],
          loop=dict(start=0, stop=3, times=1))
VB_INIT = dict(seed=7, std_matrix=0.09, std_embedding=0.5, std_gain=0.2, std_bias=0.3)

# a single tap (the convolution adds w * y of the token itself), no loop at all, head size 64 for keys and values
# with two query heads a kv head (the sizes the fast bfloat16 attention kernels take), chunks of 100
VF = dict(architecture="Vemedra", vocab=203, width=128, norm=dict(eps=1e-5), canon=dict(taps=1),
          layers=[_par(_soft(4, 2, 64, 64, 0.125, 20.0, 100, 64, 4.0e5), dict(heads=2, dim=64, vdim=64, decay=[0.95, 0.998]), 0.8, 0.4, 256),
                  _gru(128),
                  _par(_soft(2, 2, 64, 64, 0.15, 50.0, 130, 32, 1.0e4), dict(heads=4, dim=32, vdim=32, decay=[0.9, 0.95, 0.99, 0.999]), 1.0, 1.0, 128)])
VF_INIT = dict(seed=11, std_matrix=0.06, std_embedding=0.5, std_gain=0.1, std_bias=0.3)

CONFIGS = {"VA": (VA, VA_INIT), "VB": (VB, VB_INIT), "VF": (VF, VF_INIT)}

_FOLDERS = {}


def folder(name: str) -> str:
    if name not in _FOLDERS:
        from synaptix_b200.config import VemedraConfig
        from synaptix_b200.weights import write_model_folder
        cfg_dict, init = CONFIGS[name]
        init = dict(init)
        _FOLDERS[name] = write_model_folder(VemedraConfig.from_dict(cfg_dict), tempfile.mkdtemp(prefix=f"sx_{name}_"),
                                            init.pop("seed"), **init)
    return _FOLDERS[name]


@functools.lru_cache(maxsize=None)
def oracle(name: str):
    return PV.load_folder(folder(name))


@functools.lru_cache(maxsize=256)
def oracle_logits(name: str, tokens: tuple) -> torch.Tensor:
    cfg, W = oracle(name)
    return PV.forward(cfg, W, list(tokens)).float()

"""Small Pidutar configurations for the tests: they differ in every size and option."""
import functools
import tempfile

import torch

import plain_pidutar as PP


def _mem(heads, dim, vdim, cap, mlp):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap), mlp=mlp)


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, rot, mlp, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale)
    if window:
        m["mask"] = dict(size=window)
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def _moe(ff, experts, top, scale):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale))


# attention first, read by two later layers with windows of their own (70 and 9 against the owner's 23: the entry keeps
# 70 keys), a layer without feed-forward, one expert of one (top = experts = 1), odd sizes that no fast product takes
PA = dict(architecture="Pidutar", vocab=101, width=52, norm=dict(eps=1e-5), embedding=dict(scale=2.5), residual_mult=0.4,
          logit_scale=0.5,
          layers=[_lat(3, 12, 8, 10, 20, 28, 0.3, 23, (8, 1.0e4), _moe(24, 5, 2, 1.5)),
                  _mem(2, 12, 20, 6.0, None),
                  _lat(2, 6, 8, 14, 12, 28, 0.45, 70, (8, 1.0e4), _moe(16, 1, 1, 0.7), kv_from=0),
                  _mem(1, 16, 8, 15.0, _moe(40, 7, 7, 2.0)),
                  _lat(5, 4, 8, 6, 36, 28, 0.25, 9, (8, 1.0e4), _moe(8, 9, 3, 1.0), kv_from=0)])
PA_INIT = dict(seed=5, std_matrix=0.12, std_embedding=0.5, std_gain=0.2, std_bias=0.5)

# memory layers first, a window of one page and one token (65), part of the rotated elements left unrotated
# (rot.dims 4 of rot_dim 12), a window of 1 (a token sees itself alone), nine heads (more than a block of the attention
# kernel takes), scales of 1
PB = dict(architecture="Pidutar", vocab=77, width=64, norm=dict(eps=1e-6), embedding=dict(scale=1.0), residual_mult=1.0,
          logit_scale=1.0,
          layers=[_mem(4, 8, 8, 9.0, _moe(32, 4, 2, 1.0)),
                  _mem(2, 24, 12, 11.0, _moe(32, 6, 1, 3.0)),
                  _lat(9, 8, 12, 8, 40, 36, 0.2, 65, (4, 5.0e5), _moe(48, 3, 2, 1.0)),
                  _lat(1, 16, 4, 32, 16, 24, 0.35, 1, (4, 100.0), None),
                  _lat(2, 8, 12, 16, 24, 36, 0.3, 130, (4, 5.0e5), _moe(16, 8, 4, 0.5), kv_from=2)])
PB_INIT = dict(seed=9, std_matrix=0.1, std_embedding=0.7, std_gain=0.15, std_bias=0.4)

# sizes the fast bfloat16 products take (multiples of 32), no window (every key is seen) in the owner and a window in
# its reader, no rotation at all in another pair, rot_dim 0 is not used but dim 0 is: a head of rotated elements alone
PF = dict(architecture="Pidutar", vocab=256, width=128, norm=dict(eps=1e-5), embedding=dict(scale=4.0), residual_mult=0.25,
          logit_scale=0.125,
          layers=[_lat(4, 32, 32, 32, 64, 64, 0.11, None, (32, 2.0e5), _moe(64, 8, 2, 1.5)),
                  _mem(2, 32, 64, 10.0, _moe(64, 8, 2, 1.5)),
                  _lat(4, 32, 32, 32, 64, 64, 0.11, 100, (32, 2.0e5), _moe(64, 8, 2, 1.5), kv_from=0),
                  _lat(2, 0, 64, 64, 32, 96, 0.2, 40, None, _moe(32, 16, 4, 1.0)),
                  _mem(4, 64, 32, 8.0, _moe(96, 4, 3, 1.0))])
PF_INIT = dict(seed=13, std_matrix=0.08, std_embedding=0.4, std_gain=0.1, std_bias=0.3)

# head sizes that the tensor-core attention over per-head keys and values takes (dim + rot_dim = vdim = 64 and 128):
# whole prompts of 256 tokens and more run that form in bfloat16; a reader with wider heads than its owner and no window
PT = dict(architecture="Pidutar", vocab=160, width=128, norm=dict(eps=1e-5), embedding=dict(scale=2.0), residual_mult=0.35,
          logit_scale=0.5,
          layers=[_lat(4, 32, 32, 64, 64, 64, 0.13, 100, (32, 3.0e5), _moe(64, 4, 2, 1.25)),
                  _mem(2, 32, 32, 10.0, _moe(64, 4, 2, 1.25)),
                  _lat(2, 96, 32, 128, 32, 64, 0.09, None, (32, 3.0e5), _moe(64, 4, 2, 1.25), kv_from=0),
                  _lat(3, 48, 16, 64, 48, 40, 0.12, 64, (8, 1.0e4), None)])
PT_INIT = dict(seed=17, std_matrix=0.08, std_embedding=0.4, std_gain=0.1, std_bias=0.3)

CONFIGS = {"PA": (PA, PA_INIT), "PB": (PB, PB_INIT), "PF": (PF, PF_INIT), "PT": (PT, PT_INIT)}

_FOLDERS = {}


def folder(name: str) -> str:
    if name not in _FOLDERS:
        from synaptix_b200.config import PidutarConfig
        from synaptix_b200.weights import write_model_folder
        cfg_dict, init = CONFIGS[name]
        init = dict(init)
        _FOLDERS[name] = write_model_folder(PidutarConfig.from_dict(cfg_dict), tempfile.mkdtemp(prefix=f"sx_{name}_"),
                                            init.pop("seed"), **init)
    return _FOLDERS[name]


@functools.lru_cache(maxsize=None)
def oracle(name: str):
    return PP.load_folder(folder(name))


@functools.lru_cache(maxsize=256)
def oracle_logits(name: str, tokens: tuple) -> torch.Tensor:
    cfg, W = oracle(name)
    return PP.forward(cfg, W, list(tokens)).float()

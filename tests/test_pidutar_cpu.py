"""What needs no GPU of the Pidutar decoder: its configuration, the model as data (tensor names, schedule, cache
requests), and the plain implementation against other forms of its own equations."""
import copy
import math

import pytest
import torch

import plain_pidutar as PP
from tiny_pidutar import CONFIGS


def cfg_of(name):
    from synaptix_b200.config import PidutarConfig
    return PidutarConfig.from_dict(CONFIGS[name][0])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_registry(name):
    from synaptix_b200.config import PidutarConfig, resolve_architecture
    d = CONFIGS[name][0]
    cfg = cfg_of(name)
    assert PidutarConfig.from_dict(cfg.to_dict()) == cfg
    assert resolve_architecture(d).config_cls is PidutarConfig
    assert cfg.embedding_scale == d["embedding"]["scale"] and cfg.logit_scale == d["logit_scale"]
    assert [l.type for l in cfg.layers] == [l["type"] for l in d["layers"]]


def test_configuration_errors():
    from synaptix_b200.config import ConfigError, PidutarConfig
    base = CONFIGS["PA"][0]

    def broken(change):
        d = copy.deepcopy(base)
        change(d)
        with pytest.raises(ConfigError):
            PidutarConfig.from_dict(d)
    broken(lambda d: d.pop("residual_mult"))
    broken(lambda d: d["layers"][0].update(type="other"))
    broken(lambda d: d["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda d: d["layers"][0]["mlp"]["router"].update(top=9))
    broken(lambda d: d["layers"][2]["mixer"].update(kv_from=1))            # not an attention layer
    broken(lambda d: d["layers"][2]["mixer"].update(kv_from=4))            # not an earlier one
    broken(lambda d: d["layers"][4]["mixer"].update(kv_from=2))            # has no latent of its own
    broken(lambda d: d["layers"][2]["mixer"].update(kv_rank=30))           # differs from its owner's
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=10))       # more than rot_dim
    broken(lambda d: d["layers"][1]["mixer"].pop("gate_cap"))


def test_model_as_data():
    from synaptix_b200.cache.store import BundleRequest, KVRequest
    from synaptix_b200.models import model_skeleton
    m = model_skeleton(cfg_of("PA"))
    runs = [(r.layer, r.cache_entry, r.write_cache) for r in m.schedule]
    assert runs == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 2, True), (4, 0, False)]
    reqs = m.cache_requests()
    assert reqs[0] == KVRequest(1, 28 + 8, 70, keys_only=True)             # the widest window among the three readers
    assert isinstance(reqs[1], BundleRequest) and [tuple(i.shape) for i in reqs[1].items] == [(2, 12, 20), (2, 12), (2,)]
    specs = m.all_tensor_specs()
    assert "l2.mix.dkv" not in specs and "l0.mix.dkv" in specs and "l1.norm2" not in specs and "l1.ls2" not in specs
    assert tuple(specs["l0.mix.dkv"].shape) == (36, 52) and tuple(specs["l3.mlp.e6.down"].shape) == (52, 40)
    assert tuple(specs["l4.mix.uq"].shape) == (5 * 12, 36) and tuple(specs["l1.mix.i.b"].shape) == (2,)
    m = model_skeleton(cfg_of("PF"))
    assert m.cache_requests()[0] == KVRequest(1, 96, None, keys_only=True)    # the owner sees every key


def test_keys_only_storage_and_window_release():
    from synaptix_b200.cache.store import Cache, KVRequest
    c = Cache([KVRequest(1, 36, 70, keys_only=True)], max_tokens=640, max_seqs=2, dtype=torch.float32, device="cpu")
    v = c.view(0)
    assert tuple(v.k.shape[1:]) == (1, 64, 36) and v.v.shape[-1] == 0
    s = c.open()
    c.slots.reserve(s, 300)
    c.slots.advance(s, 300)
    assert c.slots.table(s, 0)[:3] == [-1, -1, -1] and c.slots.table(s, 0)[3] > 0    # keys up to 230 are behind the window


def test_plain_matrix_memory_equals_the_sum_over_the_past():
    """The recurrence with its running maximum against the closed form: weights exp(sum of later f + i_j) over the past,
    normalised by max(|.|, 1) in unstabilised terms (m starts at 0, which the closed form has as exp(-m) = 1 ... )."""
    g = torch.Generator().manual_seed(1)
    T, K, H, D, Dv, cap = 40, 12, 2, 6, 5, 7.0
    m = dict(heads=H, dim=D, vdim=Dv, gate_cap=cap)
    W = {"p." + k: torch.randn(n, K, generator=g).double() for k, n in
         [("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv), ("i", H), ("f", H)]}
    W["p.i.b"], W["p.f.b"] = torch.randn(H, generator=g).double(), torch.randn(H, generator=g).double() + 1
    W["p.norm"], W["p.o"] = torch.ones(H * Dv, dtype=torch.float64), torch.eye(H * Dv, dtype=torch.float64)
    x = torch.randn(T, K, generator=g).double()
    got = PP.mlstm(x, W, "p.", m, 1e-5)
    q = (x @ W["p.q"].T).view(T, H, D) * D ** -0.5
    k = (x @ W["p.k"].T).view(T, H, D)
    v = (x @ W["p.v"].T).view(T, H, Dv)
    gi = cap * torch.tanh((x @ W["p.i"].T + W["p.i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((x @ W["p.f"].T + W["p.f.b"]) / cap))
    ref = torch.zeros(T, H, Dv, dtype=torch.float64)
    for h in range(H):
        for t in range(T):
            logw = torch.stack([gf[j + 1:t + 1, h].sum() + gi[j, h] for j in range(t + 1)])
            mt = max(float(gf[:t + 1, h].sum()), float(logw.max()))         # the running maximum, unrolled, from m_0 = 0
            w = torch.exp(logw - mt)
            num = (w[:, None] * (k[:t + 1, h] @ q[t, h])[:, None] * v[:t + 1, h]).sum(0)
            den = max(abs(float((w * (k[:t + 1, h] @ q[t, h])).sum())), math.exp(-mt)) + 1e-6
            ref[t, h] = num / den
    ref = PP.rms_unit(ref, 1e-5).reshape(T, H * Dv) * torch.sigmoid(x @ W["p.g"].T)
    assert torch.allclose(got, ref, atol=1e-9, rtol=1e-7)


def test_plain_rotation_keeps_relative_angles():
    g = torch.Generator().manual_seed(2)
    a, b = torch.randn(1, 10, generator=g).double(), torch.randn(1, 10, generator=g).double()
    def dot(p, q):
        return float((PP.rotate_pairs(a, torch.tensor([p]), 6, 100.0) * PP.rotate_pairs(b, torch.tensor([q]), 6, 100.0)).sum())
    assert abs(dot(17, 5) - dot(112, 100)) < 1e-9 and abs(dot(17, 5) - dot(18, 5)) > 1e-3
    r = PP.rotate_pairs(a, torch.tensor([3]), 6, 100.0)
    assert torch.equal(r[:, 6:], a[:, 6:])                                   # elements from rot.dims on pass unchanged
    assert abs(float(r[0, 0]) - float(a[0, 0] * math.cos(3.0) - a[0, 1] * math.sin(3.0))) < 1e-12


def test_plain_experts_top_equal_to_all_is_the_softmax_mixture():
    g = torch.Generator().manual_seed(3)
    E, K, F = 4, 10, 6
    W = {"p.router": torch.randn(E, K, generator=g).double()}
    for e in range(E):
        W[f"p.e{e}.gate"], W[f"p.e{e}.up"] = torch.randn(F, K, generator=g).double(), torch.randn(F, K, generator=g).double()
        W[f"p.e{e}.down"] = torch.randn(K, F, generator=g).double()
    x = torch.randn(5, K, generator=g).double()
    got = PP.experts(x, W, "p.", dict(router=dict(experts=E, top=E, scale=3.0)))
    s = torch.softmax(x @ W["p.router"].T, -1)
    ref = sum(3.0 * s[:, e:e + 1] * ((torch.nn.functional.silu(x @ W[f"p.e{e}.gate"].T) * (x @ W[f"p.e{e}.up"].T)) @ W[f"p.e{e}.down"].T)
              for e in range(E))
    assert torch.allclose(got, ref, atol=1e-10)

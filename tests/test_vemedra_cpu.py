"""What of the Vemedra decoder runs without a GPU: its configuration, its model as names and shapes, the cache's
bookkeeping for its requests, and the plain implementation's mechanisms against naive loops."""
import json
import os

import pytest
import torch

import plain_vemedra as PV
from tiny_vemedra import CONFIGS, VA, VB, VF, folder


def test_config_round_trips_and_is_chosen_by_its_name(tmp_path):
    from synaptix_b200.config import VemedraConfig, load_config
    for name, (d, _) in CONFIGS.items():
        p = tmp_path / f"{name}.json"
        p.write_text(json.dumps(d))
        cfg = load_config(str(p))
        assert isinstance(cfg, VemedraConfig)
        again = VemedraConfig.from_dict(cfg.to_dict())
        assert again == cfg
    cfg = VemedraConfig.from_dict(VA)
    assert cfg.layers[0].left.chunk == 10 and cfg.layers[0].left.rot_dims == 8 and cfg.layers[1].mingru_width == 40
    assert cfg.layers[2].ff is None and cfg.layers[1].ff == 56
    # layers 1 and 2 run twice; each pass opens at layer 1
    assert cfg.runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert VemedraConfig.from_dict(VF).runs() == [(0, None), (1, None), (2, None)]


@pytest.mark.parametrize("breaker", [
    lambda d: d["layers"][0].update(type="conv"),
    lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.5]),
    lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3),
    lambda d: d["layers"][0]["mlp"].update(kind="experts"),
    lambda d: d["loop"].update(stop=9),
    lambda d: d.pop("width"),
    lambda d: d["canon"].update(taps=0),
    lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=7),
])
def test_config_errors(breaker):
    from synaptix_b200.config import ConfigError, VemedraConfig
    d = json.loads(json.dumps(VA))
    breaker(d)
    with pytest.raises(ConfigError):
        VemedraConfig.from_dict(d)


def test_model_names_shapes_and_schedule():
    from synaptix_b200.config import VemedraConfig
    from synaptix_b200.models import Inject, LayerRun, model_skeleton
    m = model_skeleton(VemedraConfig.from_dict(VA))
    specs = m.all_tensor_specs()
    assert specs["l0.mix.left.q"].shape == (64, 48) and specs["l0.mix.left.v"].shape == (16, 48)
    assert specs["l0.mix.left.sink"].shape == (4,) and specs["l0.mix.left.o"].shape == (48, 32)
    assert specs["l0.mix.right.k"].shape == (24, 48) and specs["l0.mix.right.g"].shape == (36, 48)
    assert specs["l1.mix.z.b"].shape == (40,) and specs["l1.canon2"].shape == (48, 3) and specs["loop.step"].shape == (2, 48)
    assert "l2.norm2" not in specs and "l2.canon2" not in specs and "l3.mlp.gate" not in specs
    kinds = [(type(s).__name__, getattr(s, "layer", None), getattr(s, "cache_entry", None)) for s in m.steps]
    assert kinds == [("LayerRun", 0, 0), ("Inject", None, None), ("LayerRun", 1, 1), ("LayerRun", 2, 2),
                     ("Inject", None, None), ("LayerRun", 1, 3), ("LayerRun", 2, 4), ("LayerRun", 3, 5)]
    injects = [s for s in m.steps if isinstance(s, Inject)]
    assert [(s.embedding, s.row) for s in injects] == [(False, 0), (True, 1)]
    assert len(m.cache_requests()) == 6
    # a model without a loop has no table of stream vectors
    assert "loop.step" not in model_skeleton(VemedraConfig.from_dict(VF)).all_tensor_specs()


def test_cache_bundles_value_sizes_and_state_rows():
    from synaptix_b200.cache import BundleRequest, Cache, KVRequest, StateRequest
    reqs = [BundleRequest((BundleRequest((KVRequest(2, 16, None, 8, 10), StateRequest((3, 8, 12)))), StateRequest((2, 48)),
                           StateRequest((2, 48)))),
            BundleRequest((StateRequest((40,)), StateRequest((2, 48)))),
            KVRequest(2, 16, None, 8, 10)]
    c = Cache(reqs, max_tokens=256, max_seqs=3, dtype=torch.float32, device="cpu")
    (kv, ret), h1, h2 = c.view(0)
    assert kv.k.shape == (5, 2, 64, 16) and kv.v.shape == (5, 2, 64, 8) and ret.shape == (4, 3, 8, 12)
    assert h1.shape == (4, 2, 48) and h1.data_ptr() != h2.data_ptr()
    gru, h = c.view(1)
    assert gru.shape == (4, 40) and h.shape == (4, 2, 48)
    assert c.view(2).group == kv.group and c.view(2).k.data_ptr() != kv.k.data_ptr()
    s = c.open()
    for t in (ret, h1, gru):
        t[s] = 1.0
    c.close(s)
    assert c.open() == s and float(ret[s].abs().sum() + h1[s].abs().sum() + gru[s].abs().sum()) == 0.0


def test_pages_before_the_chunk_a_sequence_has_reached_are_given_back():
    from synaptix_b200.cache import PagePool, SequenceSlots
    pool = PagePool(8, first=1)
    slots = SequenceSlots(2, [pool], [None], [100])
    s = slots.open()
    slots.reserve(s, 150)
    slots.advance(s, 150)                       # position 150 lies in chunk 100..199: page 0 (keys 0..63) is dead
    assert slots.table(s, 0) == [-1, 2, 3] and pool.n_free == 6
    slots.reserve(s, 50)
    slots.advance(s, 50)                        # at 200: keys below 200 are dead, pages 0..2 (keys up to 191) go
    assert slots.table(s, 0) == [-1, -1, -1, 1] and pool.n_free == 7
    slots.reserve(s, 56)
    slots.advance(s, 56)                        # 256 tokens: still chunk 200..299; page 3 holds keys 192..255
    assert slots.table(s, 0)[3] == 1
    slots.close(s)
    assert pool.n_free == 8


def test_plain_convolution_and_retention_against_naive_loops():
    g = torch.Generator().manual_seed(0)
    h = torch.randn(9, 5, generator=g, dtype=torch.float64)
    w = torch.randn(5, 3, generator=g, dtype=torch.float64)
    out = PV.token_conv(h, w)
    for t in range(9):
        for c in range(5):
            ref = h[t, c] + sum(w[c, j] * h[t - 2 + j, c] for j in range(3) if t - 2 + j >= 0)
            assert abs(out[t, c] - ref) < 1e-12
    # retention as a sum over earlier tokens: o_t = sum_j decay^(t-j) (q_t . k_j / sqrt(D)) v_j
    W = {"p.q": torch.randn(4, 6, generator=g, dtype=torch.float64), "p.k": torch.randn(4, 6, generator=g, dtype=torch.float64),
         "p.v": torch.randn(3, 6, generator=g, dtype=torch.float64), "p.g": torch.randn(3, 6, generator=g, dtype=torch.float64),
         "p.o": torch.eye(3, dtype=torch.float64)}
    x = torch.randn(7, 6, generator=g, dtype=torch.float64)
    got = PV.retention(x, W, "p.", dict(heads=1, dim=4, vdim=3, decay=[0.8]), 1e-5)
    q, k, v, gate = x @ W["p.q"].T, x @ W["p.k"].T / 2.0, x @ W["p.v"].T, x @ W["p.g"].T
    for t in range(7):
        o = sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1))
        o = o / torch.sqrt((o * o).mean() + 1e-5) * torch.nn.functional.silu(gate[t])
        assert torch.allclose(got[t], o, atol=1e-10)


def test_folder_of_random_weights_holds_every_tensor():
    cfg, W = PV.load_folder(folder("VA"))
    assert cfg["loop"] == VA["loop"] and W["l0.canon1"].shape == (48, 3) and float(W["l0.mix.left.sink"].abs().sum()) > 0
    lg = PV.forward(cfg, W, [1, 2, 3, 4])
    assert lg.shape == (4, 97) and torch.isfinite(lg).all()

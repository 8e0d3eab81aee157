"""The Vemedra decoder on the GPU against the plain implementation: each mechanism's kernel alone, then whole models
through the engine under every way of cutting the work into steps, portions and batches, and greedy generation through
the library's entry point.  Configurations and weights are made here (``tiny_vemedra``)."""
import math

import pytest
import torch

import plain_vemedra as PV
from helpers import assert_close
from tiny import random_tokens
from tiny_vemedra import CONFIGS, folder, oracle, oracle_logits

pytestmark = pytest.mark.gpu

NAMES = ["VA", "VB", "VF"]
DTYPES = ["float32", "bfloat16"]
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def step_ctx(past, new, slots, tables=None, dtype=torch.float32):
    """A step's context for kernels called directly: sequences with ``past`` tokens held bring ``new`` tokens each."""
    from synaptix_b200.parts import Runtime, StepContext
    i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    return StepContext(
        positions=i32([p + j for p, n in zip(past, new) for j in range(n)]),
        seq_of_token=i32([i for i, n in enumerate(new) for _ in range(n)]),
        cu_seqlens=i32(cu), seq_past=i32(past), seq_lens=i32([p + n for p, n in zip(past, new)]), seq_slots=i32(slots),
        block_tables=tables, n_tokens=sum(new), n_seqs=len(new), max_new=max(new), max_len=max(p + n for p, n in zip(past, new)),
        all_single=all(n == 1 for n in new), runtime=Runtime(torch.device("cuda:0"), dtype),
        host={"cu_seqlens": cu, "seq_past": list(past), "seq_lens": [p + n for p, n in zip(past, new)], "seq_slots": list(slots)})


def portions(lengths, cuts):
    """Steps for sequences of ``lengths``: every sequence advances by ``cuts[k]`` tokens in step k (as far as it goes)."""
    at = [0] * len(lengths)
    for c in cuts:
        past, new, who = [], [], []
        for i, n in enumerate(lengths):
            m = min(c, n - at[i])
            if m > 0:
                past.append(at[i]); new.append(m); who.append(i)
        if not who:
            break
        yield past, new, who
        for i, m in zip(who, new):
            at[i] += m


# ---------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,taps", [(40, 3), (300, 2), (48, 1), (1100, 5)])
def test_norm_and_short_convolution_over_portions(width, taps, dtype):
    """Sum, RMS norm and y + conv(y), with the last inputs carried in each sequence's slot: portions of many sizes, down to
    single tokens (the one-kernel form) and portions shorter than the taps reach back."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(width + taps)
    lengths, slots = [23, 41, 5], [2, 0, 3]
    h0 = [torch.randn(n, width, generator=g) * 2 for n in lengths]
    delta = [torch.randn(n, width, generator=g).to(DT[dtype]) for n in lengths]
    gain = 1 + 0.3 * torch.randn(width, generator=g)
    cw = 0.5 * torch.randn(width, taps, generator=g)
    hist = torch.full((5, taps - 1, width), float("nan")).cuda()
    hist[slots] = 0.0                                     # what opening a slot does; other slots must not be read
    ref = [PV.token_conv(PV.rms_norm(a.double() + d.double(), gain.double(), 1e-5), cw.double()) for a, d in zip(h0, delta)]
    got = [torch.zeros(n, width) for n in lengths]
    for past, new, who in portions(lengths, [3, 1, 1, 2, 7, 1, 64]):
        ctx = step_ctx(past, new, [slots[i] for i in who], dtype=DT[dtype])
        h = torch.cat([h0[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        d = torch.cat([delta[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        out = ops.add_rmsnorm_conv(h, d, gain.cuda(), 1e-5, cw.cuda(), hist, ctx, DT[dtype]).float().cpu()
        hsum = torch.cat([h0[i][p:p + n] + delta[i][p:p + n].float() for i, p, n in zip(who, past, new)])
        assert torch.allclose(h.cpu(), hsum, atol=1e-6)   # the sum went into the stream in place
        t = 0
        for i, p, n in zip(who, past, new):
            got[i][p:p + n] = out[t:t + n]
            t += n
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == "float32" else dict(atol=3e-2, rtol=2e-2)
    for a, b in zip(got, ref):
        assert torch.allclose(a.double(), b, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N", [70, 200])
def test_mingru_recurrence_over_portions(dtype, N):
    """Short portions (a thread walks the tokens) and long ones (pieces composed, then carried; with 200 channels through
    tiles in shared memory, with 70 a thread fetching its own channel), the state going on."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(5)
    K = 24
    W = {"p.z": torch.randn(N, K, generator=g) * 0.5, "p.x": torch.randn(N, K, generator=g), "p.g": torch.randn(N, K, generator=g),
         "p.z.b": torch.randn(N, generator=g), "p.x.b": torch.randn(N, generator=g), "p.o": torch.eye(N)}
    W = {k: v.double() for k, v in W.items()}
    lengths, slots = [330, 9, 150], [1, 3, 0]
    xs = [torch.randn(n, K, generator=g).double() for n in lengths]
    ref = [PV.mingru(x, W, "p.") for x in xs]
    stacked = torch.cat([W["p.g"], W["p.z"], W["p.x"]])                   # the kernel takes the columns by offset
    proj = [(x @ stacked.T).to(DT[dtype]) for x in xs]
    if dtype == "bfloat16":                                                # the oracle sees the rounded projections
        ref = []
        for pr in proj:
            a = pr.double()
            z = torch.sigmoid(a[:, N:2 * N] + W["p.z.b"]); u = a[:, 2 * N:] + W["p.x.b"]
            c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            S, rows = torch.zeros(N, dtype=torch.float64), []
            for t in range(a.shape[0]):
                S = (1 - z[t]) * S + z[t] * c[t]
                rows.append(S * torch.nn.functional.silu(a[t, :N]))
            ref.append(torch.stack(rows))
    state = torch.full((5, N), float("nan")).cuda()
    state[slots] = 0.0
    got = [torch.zeros(n, N) for n in lengths]
    for past, new, who in portions(lengths, [200, 1, 2, 1, 129, 64]):
        ctx = step_ctx(past, new, [slots[i] for i in who])
        a = torch.cat([proj[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        out = ops.mingru(a, N, 2 * N, 0, N, W["p.z.b"].float().cuda(), W["p.x.b"].float().cuda(), state, ctx).float().cpu()
        t = 0
        for i, p, n in zip(who, past, new):
            got[i][p:p + n] = out[t:t + n]
            t += n
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == "float32" else dict(atol=2e-2, rtol=1e-2)
    for a, b in zip(got, ref):
        assert torch.allclose(a.double(), b, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,D,E", [(3, 8, 12), (2, 64, 32), (1, 20, 100), (1, 12, 300)])
def test_retention_over_portions(heads, D, E, dtype):
    """A key far back must still count with a slow decay: token 3 of the long sequence has a key and a value ten times
    the others', and the last queries point at it."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(heads * D + E)
    K = 16
    decay = [0.999, 0.9, 0.5][:heads]
    W = {k: torch.randn(n, K, generator=g).double() * 0.4 for k, n in
         (("p.q", heads * D), ("p.k", heads * D), ("p.v", heads * E), ("p.g", heads * E))}
    W["p.o"] = torch.eye(heads * E, dtype=torch.float64)
    lengths, slots = [300, 7, 66], [0, 2, 1]
    xs = [torch.randn(n, K, generator=g).double() for n in lengths]
    xs[0][3] *= 10.0
    xs[0][-5:] = xs[0][3] / 10.0 + 0.1 * xs[0][-5:]
    m = dict(heads=heads, dim=D, vdim=E, decay=decay)
    stacked = torch.cat([W["p.q"], W["p.k"], W["p.v"], W["p.g"]])
    proj = [(x @ stacked.T).to(DT[dtype]) for x in xs]
    if dtype == "float32":
        ref = [PV.retention(x, W, "p.", m, 1e-5) for x in xs]
    else:                                                                  # the oracle on the rounded projections
        eye = {"p.q": torch.eye(heads * D), "p.k": torch.eye(heads * D), "p.v": torch.eye(heads * E), "p.g": torch.eye(heads * E)}
        ref = []
        for pr in proj:
            a = pr.double()
            hq, hv = heads * D, heads * E
            parts = {"p.q": a[:, :hq], "p.k": a[:, hq:2 * hq], "p.v": a[:, 2 * hq:2 * hq + hv], "p.g": a[:, 2 * hq + hv:]}
            T = a.shape[0]
            q = parts["p.q"].view(T, heads, D); k = parts["p.k"].view(T, heads, D) * D ** -0.5; v = parts["p.v"].view(T, heads, E)
            S, rows = torch.zeros(heads, D, E, dtype=torch.float64), []
            dc = torch.tensor(decay, dtype=torch.float64)
            for t in range(T):
                S = dc[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
                rows.append(torch.einsum("hdv,hd->hv", S, q[t]))
            o = PV.rms_unit(torch.stack(rows), 1e-5).reshape(T, hv)
            ref.append(o * torch.nn.functional.silu(parts["p.g"]))
    state = torch.full((4, heads, D, E), float("nan")).cuda()
    state[slots] = 0.0
    got = [torch.zeros(n, heads * E) for n in lengths]
    hq, hv = heads * D, heads * E
    for past, new, who in portions(lengths, [130, 1, 1, 2, 100, 64, 64]):
        ctx = step_ctx(past, new, [slots[i] for i in who])
        a = torch.cat([proj[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        out = torch.zeros(a.shape[0], hv + 5, dtype=DT[dtype]).cuda()
        ops.retention(a, 0, hq, 2 * hq, 2 * hq + hv, heads, D, E, torch.tensor(decay).cuda(), D ** -0.5, 1e-5, True, state, ctx,
                      out=out, out_col=5, out_scale=0.5)
        assert float(out[:, :5].abs().sum()) == 0.0
        o = out[:, 5:].float().cpu() * 2.0
        t = 0
        for i, p, n in zip(who, past, new):
            got[i][p:p + n] = o[t:t + n]
            t += n
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=2e-2)
    for a, b in zip(got, ref):
        assert torch.allclose(a.double(), b, **tol), float((a.double() - b).abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,vd,chunk,cap", [(4, 2, 16, 8, 10, 30.0), (2, 2, 64, 64, 100, 30.0), (4, 2, 64, 64, 37, None),
                                                      (3, 1, 32, 48, 64, 30.0), (2, 1, 128, 128, 70, 40.0), (6, 2, 32, 32, 110, 20.0)])
def test_attention_with_chunks_cap_and_sink(nh, nkv, hd, vd, chunk, cap, dtype):
    """Softmax attention over the paged cache with chunks of positions, capped scores, a sink per head and values of their
    own size, in a prompt portion and token by token.  Keys at the first and last place of a chunk, at page borders and far
    back are made ten times larger and the queries after them point at them, so that a key seen one place too far or not
    far enough changes the result by much more than the tolerance; one sink is large, so that leaving it out shows."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(nh * hd + chunk)
    T, cut = 230, 150                                       # a portion of 150 tokens, then single tokens
    q = torch.randn(T, nh, hd, generator=g) * 0.5
    k = torch.randn(T, nkv, hd, generator=g) * 0.5
    v = torch.randn(T, nkv, vd, generator=g)
    spikes = sorted({j for c in range(0, T, chunk) for j in (c - 1, c, c + 1) if 0 <= j < T} | {63, 64, 127, 128, 191, 192, 2})
    for j in spikes:
        k[j] *= 6.0
        for t in range(j, min(T, j + 3)):                   # the next queries look for that key
            q[t] = 0.4 * q[t] + k[j].repeat_interleave(nh // nkv, dim=0) / 6.0
    sinks = torch.randn(nh, generator=g)
    sinks[0] = 4.0
    scale = 1.3 / math.sqrt(hd)
    dt = DT[dtype]
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    ref = PV.chunk_sink_heads(q.double(), k.double(), v.double(), torch.arange(T), sinks.double(), scale, cap, chunk)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).cuda()
    pages = 6
    kp = torch.full((pages, nkv, 64, hd), float("nan"), dtype=dt).cuda()
    vp = torch.full((pages, nkv, 64, vd), float("nan"), dtype=dt).cuda()
    table = torch.tensor([[4, 2, 5, 1]], dtype=torch.int32).cuda()
    got = []
    for past, new in [(0, cut)] + [(p, 1) for p in range(cut, T)]:
        ctx = step_ctx([past], [new], [0], [table], dtype=dt)
        a = proj[past:past + new].contiguous()
        qq = torch.empty(new, nh * hd, dtype=dt).cuda()
        ops.qkv_prepare(a, qq, kp, vp, None, None, None, 0, 0.0, ctx.positions, ctx.seq_of_token, table, nh, nkv, hd, vd=vd)
        oc = 4 if hd == vd else 3              # (the tensor-core kernels of bfloat16 want even columns)
        out = torch.zeros(new, nh * vd + oc, dtype=dt).cuda()
        ops.attention(qq, kp, vp, ctx, table, nh, nkv, hd, scale, None, vd=vd, softcap=cap, sinks=sinks.cuda(), chunk=chunk,
                      out=out, out_col=oc, out_scale=2.0)
        assert float(out[:, :oc].abs().sum()) == 0.0
        got.append(out[:, oc:].float().cpu() / 2.0)
    got = torch.cat(got).view(T, nh, vd)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=4e-2, rtol=3e-2)
    assert torch.allclose(got.double(), ref, **tol), float((got.double() - ref).abs().max())
    if dtype == "bfloat16" and hd == vd:           # the same through the plain kernel
        with ops.options(attn_options_fast=False):
            ctx = step_ctx([0], [T], [0], [table], dtype=dt)
            qq = torch.empty(T, nh * hd, dtype=dt).cuda()
            ops.qkv_prepare(proj, qq, kp, vp, None, None, None, 0, 0.0, ctx.positions, ctx.seq_of_token, table, nh, nkv, hd, vd=vd)
            o2 = ops.attention(qq, kp, vp, ctx, table, nh, nkv, hd, scale, None, vd=vd, softcap=cap, sinks=sinks.cuda(), chunk=chunk)
        assert torch.allclose(o2.float().cpu().view(T, nh, vd).double(), ref, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_capped_gated_activation_and_stream_sums(dtype):
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(1)
    gu = (torch.randn(7, 2 * 33, generator=g) * 3).to(DT[dtype])
    a = gu.double()
    gate, up = torch.clamp(a[:, :33], max=1.5), torch.clamp(a[:, 33:], -1.5, 1.5)
    ref = gate * torch.sigmoid(1.702 * gate) * (up + 1)
    got = ops.capped_glu(gu.cuda(), 1.702, 1.5).float().cpu().double()
    assert torch.allclose(got, ref, atol=1e-5 if dtype == "float32" else 3e-2, rtol=1e-5 if dtype == "float32" else 1e-2)
    h = torch.randn(7, 33, generator=g)
    d = torch.randn(7, 33, generator=g).to(DT[dtype])
    rows, vec = torch.randn(7, 33, generator=g), torch.randn(33, generator=g)
    hd = h.clone().cuda()
    ops.stream_add(hd, d.cuda(), rows.cuda(), vec.cuda())
    assert torch.allclose(hd.cpu(), h + d.float() + rows + vec, atol=1e-6)
    hd = h.clone().cuda()
    ops.stream_add(hd, None, None, vec.cuda())
    assert torch.allclose(hd.cpu(), h + vec, atol=1e-6)


@pytest.mark.parametrize("rows", [1, 2, 8, 16, 40, 160, 300, 700])
def test_capped_gated_activation_in_the_products_epilogues(rows):
    """Every bfloat16 product with the gated epilogue (the weight-streaming ones of few rows, the tile product of prompt
    steps with its cut tiles) applies the capped form inside ``gate_activation`` and SiLU * up outside of it."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(rows)
    K, I = 256, 640
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.15).to(torch.bfloat16)
    a = x.double() @ w.double().T
    gate, up = torch.clamp(a[:, :I], max=1.25), torch.clamp(a[:, I:], -1.25, 1.25)
    capped = gate * torch.sigmoid(1.702 * gate) * (up + 1)
    plain = torch.nn.functional.silu(a[:, :I]) * a[:, I:]
    with ops.gate_activation(1.702, 1.25):
        got = ops.linear(x.cuda(), w.cuda(), epilogue="silu_mul").float().cpu().double()
    assert torch.allclose(got, capped, atol=3e-2, rtol=2e-2), float((got - capped).abs().max())
    got = ops.linear(x.cuda(), w.cuda(), epilogue="silu_mul").float().cpu().double()
    assert torch.allclose(got, plain, atol=6e-2, rtol=2e-2), float((got - plain).abs().max())
    with ops.gate_activation(1.702, 1.25):                   # and in 32-bit, through the plain kernels
        got = ops.linear(x.float().cuda(), w.float().cuda(), epilogue="silu_mul").cpu().double()
    assert torch.allclose(got, capped, atol=1e-4, rtol=1e-4)


# ---------------------------------------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def engines():
    from synaptix_b200.engine import Engine
    from synaptix_b200.models import load_model
    made = {}

    def get(name, dtype, max_tokens=2048, max_seqs=None):
        key = (name, dtype, max_tokens, max_seqs)
        if key not in made:
            eng = Engine(load_model(folder(name), dtype=dtype), max_tokens=max_tokens, max_seqs=max_seqs)
            for t in eng.cache._k + eng.cache._v:          # a kernel that reads a place no step wrote shows at once
                t.fill_(float("nan"))
            made[key] = eng
        assert made[key].cache.slots.n_live == 0
        return made[key]
    return get


def vocab(name):
    return CONFIGS[name][0]["vocab"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_every_place(engines, name, dtype):
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    assert type(eng.model.config).__name__ == "VemedraConfig" and eng.use_graphs
    for i, n in enumerate([1, 2, 3, 17, 64, 65, 150, 301]):
        toks = random_tokens(vocab(name), n, 100 + i)
        s = eng.open()
        got = eng.step([Entry(s, toks, list(range(n)))])
        eng.close(s)
        assert_close(got, oracle_logits(name, tuple(toks)), dtype, f"{name} {dtype} whole n={n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first_token(engines, name, dtype):
    """Every token a step of its own (captured steps): the first tokens of a sequence, whose convolutions and states
    begin from zeros, and on across chunk and page borders."""
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    # (with a single token behind it, retention's unit norm leaves sign(q . k) v / rms(v): where q . k is nearly zero,
    # rounding to bfloat16 may flip it, so the sequence begins with a token for which it is not)
    toks = random_tokens(vocab(name), 150, 8)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = torch.cat([eng.step([Entry(s, [t], [0])]) for t in toks])
    eng.close(s)
    assert_close(got, ref, dtype, f"{name} {dtype} token by token")
    assert any(c.graph is not None for c in eng._captured.values())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("size", [2, 3, 7, 64, 100])
def test_prompts_in_portions(engines, name, dtype, size):
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    toks = random_tokens(vocab(name), 277, 20 + size)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = [eng.step([Entry(s, toks[a:a + size], list(range(len(toks[a:a + size]))))]) for a in range(0, len(toks), size)]
    eng.close(s)
    assert_close(torch.cat(got), ref, dtype, f"{name} {dtype} portions of {size}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_in_slots_and_pages_used_again(engines, name, dtype):
    """Batches of unequal prompts decoded together, shorter requests ending earlier; the cache holds little more than one
    batch and three slots, so every batch runs in slots, states and pages that the batch before gave back."""
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype, max_tokens=512, max_seqs=3)
    V = vocab(name)
    for b, (lens, decodes) in enumerate([([5, 130, 1], [3, 40, 12]), ([64, 9, 200], [10, 30, 2]), ([2, 3, 100], [25, 1, 70])]):
        seqs = [random_tokens(V, n + d, 300 + 10 * b + i) for i, (n, d) in enumerate(zip(lens, decodes))]
        refs = [oracle_logits(name, tuple(s)) for s in seqs]
        slots = [eng.open() for _ in seqs]
        got = eng.step([Entry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)])
        assert_close(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), dtype, f"{name} batch {b} prompts")
        live = list(range(len(seqs)))
        for j in range(max(decodes)):
            live = [i for i in live if j < decodes[i]]
            got = eng.step([Entry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in live])
            assert_close(got, torch.stack([refs[i][lens[i] + j] for i in live]), dtype, f"{name} batch {b} decode {j}")
            for i in live:
                if j == decodes[i] - 1:
                    eng.close(slots[i])
    assert eng.cache.slots.n_live == 0


@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_gives_pages_of_passed_chunks_back(engines, name):
    """400 tokens one by one behind a prompt, in a cache of 5 pages: it only fits because pages that lie before the
    chunk a sequence has reached are given back (chunks of 10 to 130 positions in these models)."""
    from synaptix_b200.engine import Entry
    eng = engines(name, "float32", max_tokens=320)
    toks = random_tokens(vocab(name), 90 + 400, 77)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = [eng.step([Entry(s, toks[:90], [89])])]
    for t in toks[90:]:
        got.append(eng.step([Entry(s, [t], [0])]))
    assert -1 in eng.cache.slots.table(s, 0)
    eng.close(s)
    assert_close(torch.cat(got), ref[89:], "float32", f"{name} long decoding")


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(name):
    """``LLM.generate`` (scheduler, decode sessions, sampling on the device): greedy tokens of unequal prompts in one
    batch equal the plain implementation's, each computed alone."""
    import synaptix_b200
    llm = synaptix_b200.LLM(folder(name), compute_dtype="float32", max_tokens=1024)
    V = vocab(name)
    prompts = [random_tokens(V, n, 900 + n) for n in (3, 41, 1, 18)]
    out = llm.generate(prompts, max_new_tokens=12, temperature=0.0)
    cfg, W = oracle(name)
    for p, new in zip(prompts, out):
        seq = list(p)
        for tok in new:
            lg = PV.forward(cfg, W, seq)[-1]
            top2 = lg.topk(2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(lg.abs().max()):       # a near tie may fall either way
                assert tok == int(lg.argmax()), f"{name}: token {len(seq) - len(p)} of prompt of {len(p)}"
            seq.append(tok)
        assert len(new) == 12
    out2 = llm.generate(prompts, max_new_tokens=12, temperature=0.0, prefill_batch=5)
    assert out2 == out


@pytest.mark.parametrize("dtype", DTYPES)
def test_replay_program_with_a_batch_whose_requests_end_at_different_times(tmp_path, dtype):
    """``bin/trace_run`` as a user drives it (a subprocess fed JSON lines): three requests of unequal lengths begin in one
    step, go on one token a step, the shorter ones end earlier, and a fourth runs afterwards in what they gave back."""
    from test_gpu_trace_run import Replay
    name = "VA"
    V = vocab(name)
    seqs = {f"q{i}": random_tokens(V, n, 800 + i) for i, n in enumerate([31, 75, 12, 50])}
    refs = {k: oracle_logits(name, tuple(v)) for k, v in seqs.items()}
    r = Replay(folder(name), dtype, str(tmp_path), 192)
    heads = {"q0": 20, "q1": 60, "q2": 11}
    got = r.step([{"id": k, "tokens": seqs[k][:h], "want": [0, h - 1]} for k, h in heads.items()])
    assert_close(got, torch.stack([refs[k][j] for k, h in heads.items() for j in (0, h - 1)]), dtype, "replay: prompts")
    at = dict(heads)
    while at:
        live = list(at)
        ends = [k for k in live if at[k] + 1 == len(seqs[k])]
        got = r.step([{"id": k, "tokens": [seqs[k][at[k]]], "want": [0]} for k in live], end=ends)
        assert_close(got, torch.stack([refs[k][at[k]] for k in live]), dtype, f"replay: decode {sorted(at.values())}")
        for k in live:
            at[k] += 1
            if k in ends:
                del at[k]
    got = r.step([{"id": "q3", "tokens": seqs["q3"], "want": [49]}], end=["q3"])
    assert_close(got, refs["q3"][49:50], dtype, "replay: afterwards")
    r.finish()


def test_command_line_run_and_inspect(tmp_path):
    """``python -m synaptix_b200 run`` chooses the model by config.json and generates greedily; ``inspect`` lists its layers."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "VB"
    cfg, W = oracle(name)
    prompt = random_tokens(vocab(name), 9, 1300)
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "synaptix_b200", "run", folder(name), ",".join(map(str, prompt)),
                        "--max-tokens", "6", "--temperature", "0", "--compute-dtype", "f32", "--stop-ids", "", "--json"],
                       capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    seq = list(prompt)
    for tok in out["outputs"][0]["tokens"]:
        lg = PV.forward(cfg, W, seq)[-1]
        top2 = lg.topk(2).values
        if float(top2[0] - top2[1]) > 1e-3 * float(lg.abs().max()):
            assert tok == int(lg.argmax())
        seq.append(tok)
    assert out["prompt_tokens"] == 9 and out["new_tokens"] == 6
    r = subprocess.run([sys.executable, "-m", "synaptix_b200", "inspect", folder(name)], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "architecture: Vemedra" in r.stdout and "layer 1: parallel, feed-forward 96" in r.stdout

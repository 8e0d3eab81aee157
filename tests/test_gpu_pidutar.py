"""The Pidutar decoder on the GPU against the plain implementation: each mechanism's kernels alone, then whole models
through the engine under every way of cutting the work into steps, portions and batches, and greedy generation through
the library's entry point.  Configurations and weights are made here (``tiny_pidutar``)."""
import math

import pytest
import torch

import plain_pidutar as PP
import helpers
from test_gpu_vemedra import portions, step_ctx
from tiny import random_tokens
from tiny_pidutar import CONFIGS, folder, oracle, oracle_logits

pytestmark = pytest.mark.gpu

NAMES = ["PA", "PB", "PF", "PT"]
DTYPES = ["float32", "bfloat16"]
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def i32(x):
    return torch.tensor(x, dtype=torch.int32).cuda()


def assert_close(got, ref, dtype, what=""):
    """Logits against the oracle's.  32-bit: every row within the shared tolerance.  bfloat16: these small models have
    routers with random weights, and where two experts' scores nearly tie, rounding may choose the other one; that row
    is then off by far more than rounding alone and the rows behind it by a little more.  So the bfloat16 comparison is
    one over many rows (callers gather the rows of single-token steps first): 85 in 100 within the shared tolerance."""
    if dtype == "float32":
        return helpers.assert_close(got, ref, dtype, what)
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    rel = (got - ref).abs().max(dim=1).values / ref.abs().max()
    within = float((rel <= helpers.BF16_REL).float().mean())
    assert within >= 0.85, f"{what}: only {within:.2f} of {rel.numel()} rows are within {helpers.BF16_REL}"


class Gathered:
    """Rows of many small steps, compared at once (see ``assert_close``); 32-bit rows are compared as they come."""

    def __init__(self, dtype, what):
        self.dtype, self.what, self.got, self.ref = dtype, what, [], []

    def add(self, got, ref, what=""):
        if self.dtype == "float32":
            return helpers.assert_close(got, ref, self.dtype, f"{self.what} {what}")
        self.got.append(got.detach().float().cpu())
        self.ref.append(ref.detach().float().cpu())

    def check(self):
        if self.got:
            assert_close(torch.cat(self.got), torch.cat(self.ref), self.dtype, self.what)


def near(got, ref, dtype, f32=1e-4, bf16=2e-2):
    """Elementwise, against the largest magnitude of the reference."""
    scale = float(ref.abs().max())
    err = float((got.double() - ref.double()).abs().max())
    assert err <= (f32 if dtype == "float32" else bf16) * scale, f"off by {err:.3e} at scale {scale:.3e}"


# ---------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [52, 328, 1000, 13000])
def test_scaled_branches_summed_and_two_norms_of_one_row(width, dtype):
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(width)
    T = 7
    h = torch.randn(T, width, generator=g) * 3
    a = torch.randn(T, width, generator=g).to(DT[dtype])
    b = torch.randn(T, width, generator=g)                       # a 32-bit term beside one of the compute dtype
    sa, sb = torch.randn(width, generator=g), torch.randn(width, generator=g)
    w1, w2 = 0.2 * torch.randn(width, generator=g), 0.2 * torch.randn(width, generator=g)
    x = h.double() + sa.double() * a.double() + sb.double() * b.double()
    ref1, ref2 = PP.norm_around_zero(x, w1.double(), 1e-5), PP.norm_around_zero(x, w2.double(), 1e-5)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == "float32" else dict(atol=3e-2, rtol=1e-2)
    hd = h.cuda()
    y1, y2 = ops.add_scaled_rmsnorm(hd, [(a.cuda(), sa.cuda()), (b.cuda(), sb.cuda())], [(1 + w1).cuda(), (1 + w2).cuda()],
                                    1e-5, DT[dtype])
    assert torch.allclose(hd.cpu().double(), x, atol=1e-5)       # the sum went into the stream in place
    assert torch.allclose(y1.float().cpu().double(), ref1, **tol) and torch.allclose(y2.float().cpu().double(), ref2, **tol)
    # chosen rows only, one term without a factor, one norm: the stream stays as it is
    hd = h.cuda()
    rows = [5, 0, 3]
    (y,) = ops.add_scaled_rmsnorm(hd, [(b.cuda(), None)], [(1 + w1).cuda()], 1e-5, DT[dtype], rows=i32(rows))
    assert torch.equal(hd.cpu(), h)
    assert torch.allclose(y.float().cpu().double(), PP.norm_around_zero(h.double() + b.double(), w1.double(), 1e-5)[rows], **tol)
    hd = h.cuda()
    ops.add_scaled(hd, [(a.cuda(), sa.cuda())])
    assert torch.allclose(hd.cpu().double(), h.double() + sa.double() * a.double(), atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,D,Dv,cap", [(3, 8, 12, 6.0), (2, 64, 32, 15.0), (1, 20, 100, 9.0), (1, 128, 128, 13.0), (1, 260, 200, 8.0)])
def test_matrix_memory_over_portions(heads, D, Dv, cap, dtype):
    """Portions of many sizes down to single tokens, the three states going on in each sequence's slot; the other slots
    hold NaN.  Gate biases push the forget gate both ways, so that the running maximum is led by either of its arms."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(heads * D + Dv)
    K = 16
    m = dict(heads=heads, dim=D, vdim=Dv, gate_cap=cap)
    W = {"p.q": torch.randn(heads * D, K, generator=g) * 0.5, "p.k": torch.randn(heads * D, K, generator=g) * 0.5,
         "p.v": torch.randn(heads * Dv, K, generator=g) * 0.5, "p.g": torch.randn(heads * Dv, K, generator=g) * 0.5,
         "p.i": torch.randn(heads, K, generator=g) * 2, "p.f": torch.randn(heads, K, generator=g) * 2,
         "p.i.b": torch.randn(heads, generator=g) * 3, "p.f.b": torch.randn(heads, generator=g) * 3 + 2,
         "p.norm": 1 + 0.2 * torch.randn(heads * Dv, generator=g), "p.o": torch.eye(heads * Dv)}
    W = {k: v.double() for k, v in W.items()}
    lengths, slots = [210, 9, 77], [1, 3, 0]
    xs = [torch.randn(n, K, generator=g).double() for n in lengths]
    stacked = torch.cat([W["p.g"], W["p.q"], W["p.v"], W["p.k"]])                # the kernel takes the columns by offset
    proj = [(x @ stacked.T).to(DT[dtype]) for x in xs]
    gates = [(x @ torch.cat([W["p.i"], W["p.f"]]).T).float() for x in xs]
    if dtype == "bfloat16":            # the oracle sees the rounded projections: weights that pick them out of the row
        hv, hq = heads * Dv, heads * D
        ref = []
        for pr, x in zip(proj, xs):
            z = torch.cat([pr.double(), x], dim=1)
            n_in = z.shape[1]
            def pick(a, n):
                w = torch.zeros(n, n_in, dtype=torch.float64)
                w[torch.arange(n), a + torch.arange(n)] = 1.0
                return w
            Wp = dict(W)
            Wp["p.g"], Wp["p.q"], Wp["p.v"], Wp["p.k"] = pick(0, hv), pick(hv, hq), pick(hv + hq, hv), pick(2 * hv + hq, hq)
            for nm in ("p.i", "p.f"):
                Wp[nm] = torch.cat([torch.zeros(heads, pr.shape[1], dtype=torch.float64), W[nm]], dim=1)
            ref.append(PP.mlstm(z, Wp, "p.", m, 1e-5))
    else:
        ref = [PP.mlstm(x, W, "p.", m, 1e-5) for x in xs]
    S = torch.full((5, heads, D, Dv), float("nan")).cuda()
    nn = torch.full((5, heads, D), float("nan")).cuda()
    mm = torch.full((5, heads), float("nan")).cuda()
    for t in (S, nn, mm):
        t[slots] = 0.0
    bias = torch.cat([W["p.i.b"], W["p.f.b"]]).float().cuda()
    hv, hq = heads * Dv, heads * D
    got = [torch.zeros(n, hv) for n in lengths]
    for past, new, who in portions(lengths, [70, 1, 2, 1, 65, 64, 3, 200]):
        ctx = step_ctx(past, new, [slots[i] for i in who])
        a = torch.cat([proj[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        gt = torch.cat([gates[i][p:p + n] for i, p, n in zip(who, past, new)]).cuda()
        out = ops.mlstm(a, hv, 2 * hv + hq, hv + hq, 0, gt, bias, cap, D ** -0.5, heads, D, Dv, W["p.norm"].float().cuda(),
                        1e-5, 1e-6, S, nn, mm, ctx).float().cpu()
        t = 0
        for i, p, n in zip(who, past, new):
            got[i][p:p + n] = out[t:t + n]
            t += n
    for a, b in zip(got, ref):
        near(a, b, dtype)
    assert torch.isnan(S[2]).all() and torch.isnan(mm[4]).all()


def latent_pages(rows_by_seq, tables, n_pages, E, dtype):
    """Cache pages [n_pages, 1, 64, E] filled with NaN except the rows of the given sequences at their positions."""
    pages = torch.full((n_pages, 1, 64, E), float("nan"), dtype=dtype)
    for rows, table in zip(rows_by_seq, tables):
        for j in range(rows.shape[0]):
            pages[table[j // 64], 0, j % 64] = rows[j].to(dtype)
    return pages.cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,R,Dr,window", [(3, 28, 8, 23), (9, 88, 24, 75), (2, 40, 0, 64), (1, 300, 20, None), (4, 64, 64, 1), (2, 30, 6, 17), (1, 70, 2, 40)])
def test_latent_attention_sees_the_windows_edge_and_a_key_far_back(heads, R, Dr, window, dtype):
    """Cache rows and queries made here: for each probed query one key is made to stand out (its row is the query's
    direction, scaled), placed just inside the window, just outside it, at position 0 and across page borders; queries
    in prompts and single ones.  Pages are scattered and unused ones hold NaN."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(heads + R)
    E, scale = R + Dr, 0.3
    n = 300
    rows = torch.randn(n, E, generator=g) * 0.3
    qa = torch.randn(n, heads, E, generator=g) * 0.3
    w = window if window else n
    probes = {}            # query position -> position of the key that stands out
    for p, j in [(299, 299 - w + 1), (298, 298 - w), (150, max(0, 150 - w + 1)), (200, 200 - w), (64, 64 - min(w, 64) + 1),
                 (128, 63), (5, 0), (0, 0), (72, 1)]:
        if j >= 0:
            probes[p] = j
    for p, j in probes.items():
        rows[j] = 0.2 * torch.randn(E, generator=g)
    for p, j in probes.items():
        qa[p] = rows[j][None, :] * (8.0 + torch.arange(heads)[:, None]) / (rows[j].norm() ** 2 * scale) * 2.0
    rows = rows.to(DT[dtype]).double()                       # what the cache holds
    pos = torch.arange(n)
    diff = pos[:, None] - pos[None, :]
    see = (diff >= 0) & (diff < w)
    ref = torch.zeros(n, heads, R, dtype=torch.float64)
    for h in range(heads):
        s = (qa[:, h].double() @ rows.T) * scale
        ref[:, h] = torch.softmax(s.masked_fill(~see, -math.inf), dim=-1) @ rows[:, :R]
    table = [7, 2, 9, 4, 1]
    pages = latent_pages([rows], [table], 11, E, DT[dtype])
    bt = i32([table])
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == "float32" else dict(atol=2e-3, rtol=2e-3)
    ctx = step_ctx([0], [n], [0], tables=[bt])                  # the whole prompt
    got = ops.latent_attention(qa.cuda(), pages, ctx, bt, heads, R, Dr, scale, window).merged().cpu().double()
    assert torch.allclose(got, ref, **tol), float((got - ref).abs().max())
    standout = [p for p, j in probes.items() if 0 <= p - j < w and p != j]
    assert (standout or w == 1) and all(float((ref[p] - rows[probes[p], :R]).abs().max()) < 0.05 for p in standout)
    for p in probes:                                            # single queries behind p cached tokens
        ctx = step_ctx([p], [1], [0], tables=[bt])
        for splits in (None, 1, 3, 16):                         # the window in parts, merged (more parts than key tiles too)
            got = ops.latent_attention(qa[p:p + 1].cuda(), pages, ctx, bt, heads, R, Dr, scale, window, splits=splits)
            assert torch.allclose(got.merged().cpu().double(), ref[p:p + 1], **tol), (p, splits)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairs", [True, False])
def test_latent_attention_layer_against_per_head_keys_and_values(dtype, pairs):
    """The four kernels in a row (prepare and cache write, queries into the latent's space, attention, values and gate)
    against the form that makes every head's keys and values; two sequences in scattered pages, a prompt and portions."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(3)
    K, H, D, Dr, Dv, Rq, R, window, dims = 24, 3, 12, 8, 10, 20, 28, 37, 6
    m = dict(heads=H, dim=D, rot_dim=Dr, vdim=Dv, q_rank=Rq, kv_rank=R, scale=0.4, mask=dict(size=window), rot=dict(dims=dims, base=1.0e4))
    shapes = {"dq": (Rq, K), "uq": (H * (D + Dr), Rq), "dkv": (R + Dr, K), "uk": (H * D, R), "uv": (H * Dv, R), "g": (H, K)}
    W = {"p." + k: (torch.randn(*s, generator=g) * 0.4).to(DT[dtype]).double() for k, s in shapes.items()}
    W["p.dq.norm"] = 1 + 0.2 * torch.randn(Rq, generator=g).double()
    W["p.dkv.norm"] = 1 + 0.2 * torch.randn(R, generator=g).double()
    W["p.o"] = torch.eye(H * Dv, dtype=torch.float64)
    lengths = [150, 70]
    xs = [torch.randn(n, K, generator=g).to(DT[dtype]).double() for n in lengths]
    if pairs:
        ref = []
        for x in xs:
            pos = torch.arange(x.shape[0])
            ref.append(PP.latent_attention(x, W, "p.", m, pos, 1e-5, PP.latent_keys(x, W, "p.", m, pos, 1e-5)))
    tables = [[5, 1, 8], [3, 6, 0]]
    pages = torch.full((9, 1, 64, R + Dr), float("nan"), dtype=DT[dtype]).cuda()
    bt = i32(tables)
    stacked = torch.cat([W["p.dq"], W["p.g"], W["p.dkv"]]).to(DT[dtype]).cuda()
    inv_freq = torch.tensor([1.0e4 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32).cuda()
    got = [torch.zeros(n, H * Dv) for n in lengths]
    for past, new, who in portions(lengths, [64, 1, 1, 30, 2, 100]):
        ctx = step_ctx(past, new, who, tables=[bt[who]])
        x = torch.cat([xs[i][p:p + n] for i, p, n in zip(who, past, new)]).to(DT[dtype]).cuda()
        proj = ops.gemm_generic(x, stacked)
        cq = ops.latent_prepare(proj, Rq, Rq + H, R, Dr, W["p.dq.norm"].float().cuda(), W["p.dkv.norm"].float().cuda(), 1e-5,
                                inv_freq, dims, pairs, ctx, bt[who].contiguous(), pages)
        q = ops.gemm_generic(cq, W["p.uq"].to(DT[dtype]).cuda())
        qa = ops.latent_query(q, W["p.uk"].to(DT[dtype]).cuda(), H, D, Dr, R, inv_freq, dims, pairs, ctx)
        ol = ops.latent_attention(qa, pages, ctx, bt[who].contiguous(), H, R, Dr, 0.4, window)
        y = ops.latent_output(ol, W["p.uv"].to(DT[dtype]).cuda(), H, Dv, R, proj, Rq, DT[dtype]).float().cpu()
        t = 0
        for i, p, n in zip(who, past, new):
            got[i][p:p + n] = y[t:t + n]
            t += n
    if not pairs:      # the other pairing has no plain counterpart here: rotating queries and keys alike keeps relative angles
        assert all(torch.isfinite(a).all() for a in got)
        return
    for a, b in zip(got, ref):
        near(a, b, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,experts,top,ff,width", [(1, 5, 2, 24, 52), (3, 1, 1, 16, 40), (70, 7, 7, 40, 64), (300, 16, 4, 100, 130), (9, 10, 3, 72, 328), (400, 6, 2, 136, 264), (700, 5, 3, 200, 328)])
def test_mixture_of_experts(T, experts, top, ff, width, dtype):
    """Router, sort by expert, grouped products and the weighted sum against the plain form; one token's input is made
    to fall on a near tie of the router, which the comparison leaves out."""
    from synaptix_b200 import ops
    g = torch.Generator().manual_seed(T + experts)
    W = {"p.router": torch.randn(experts, width, generator=g).double() * 0.5}
    for e in range(experts):
        W[f"p.e{e}.gate"] = (torch.randn(ff, width, generator=g) * 0.2).to(DT[dtype]).double()
        W[f"p.e{e}.up"] = (torch.randn(ff, width, generator=g) * 0.2).to(DT[dtype]).double()
        W[f"p.e{e}.down"] = (torch.randn(width, ff, generator=g) * 0.2).to(DT[dtype]).double()
    x = torch.randn(T, width, generator=g).to(DT[dtype])
    f = dict(router=dict(experts=experts, top=top, scale=1.7))
    ref = PP.experts(x.double(), W, "p.", f)
    s = torch.softmax(x.double() @ W["p.router"].T, dim=-1).sort(dim=-1, descending=True).values
    clear = torch.ones(T, dtype=torch.bool) if top == experts else (s[:, top - 1] - s[:, top]) > 1e-4
    gate_up = torch.stack([torch.cat([W[f"p.e{e}.gate"], W[f"p.e{e}.up"]]) for e in range(experts)]).to(DT[dtype]).cuda()
    down = torch.stack([W[f"p.e{e}.down"] for e in range(experts)]).to(DT[dtype]).cuda()
    ids, weights = ops.moe_route(x.cuda(), W["p.router"].float().cuda(), top, 1.7, 1e-20)
    assert torch.allclose(weights.sum(-1).cpu(), torch.full((T,), 1.7), atol=1e-5)
    plan = ops.moe_sort(ids, experts)
    off = plan.offsets.cpu().tolist()
    assert off[0] == 0 and off[-1] == T * top and sorted(plan.order.cpu().tolist()) == list(range(T * top))
    flat = ids.cpu().flatten().tolist()
    for e in range(experts):
        assert all(flat[i] == e for i in plan.order.cpu().tolist()[off[e]:off[e + 1]])
    z = ops.moe_gate_up(x.cuda(), gate_up, plan, top)
    y = ops.moe_down(z, down, plan)
    got = ops.moe_combine(y, plan, weights, DT[dtype]).float().cpu().double()
    near(got[clear], ref[clear], dtype)


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
    assert type(eng.model.config).__name__ == "PidutarConfig" and eng.use_graphs
    for i, n in enumerate([1, 2, 3, 17, 64, 65, 150, 301, 700]):
        toks = random_tokens(vocab(name), n, 100 + i)
        s = eng.open()
        got = eng.step([Entry(s, toks, list(range(n)))])
        eng.close(s)
        assert_close(got, oracle_logits(name, tuple(toks)), dtype, f"{name} {dtype} whole n={n}")


def test_whole_prompts_in_bfloat16_take_the_per_head_form(engines, monkeypatch):
    """Head sizes a tensor-core attention kernel takes: a whole prompt of 256 tokens and more goes through per-head keys
    and values in pages of the step's own (all three attention layers of this model), a shorter one, a portion
    behind cached tokens and single tokens through the latent form; all agree with the plain implementation."""
    from synaptix_b200 import ops
    from synaptix_b200.engine import Entry
    calls = []
    orig = ops.latent_expand
    monkeypatch.setattr(ops, "latent_expand", lambda *a, **k: (calls.append(1), orig(*a, **k))[1])
    eng = engines("PT", "bfloat16")
    toks = random_tokens(vocab("PT"), 400, 5)
    ref = oracle_logits("PT", tuple(toks))
    s = eng.open()
    got = [eng.step([Entry(s, toks[:300], list(range(300)))])]
    n_first = len(calls)
    got.append(eng.step([Entry(s, toks[300:399], list(range(99)))]))
    got.append(eng.step([Entry(s, toks[399:], [0])]))
    eng.close(s)
    assert n_first == 3 and len(calls) == 3
    assert_close(torch.cat(got), ref, "bfloat16", "PT: per-head form, then the latent form")


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(engines, name):
    """The residual stream behind each layer (the branches' sum included) against the plain implementation's."""
    from synaptix_b200.engine import Entry
    eng = engines(name, "float32")
    toks = random_tokens(vocab(name), 90, 4)
    cfg, W = oracle(name)
    ref = []
    PP.forward(cfg, W, toks, ref)
    seen = []
    s = eng.open()
    entries = [Entry(s, toks, [0])]
    past, new = eng._check(entries)
    ctx = eng.plan(entries, past, new)
    ctx.observe = lambda n, h, pending: seen.append((h + pending.float()).cpu() if pending is not None else h.cpu().clone())
    eng._forward(ctx)
    eng.cache.slots.advance(s, len(toks))
    eng.close(s)
    assert len(seen) == len(ref)
    for i, (a, b) in enumerate(zip(seen, ref)):
        assert torch.allclose(a.double(), b, atol=2e-4 * float(b.abs().max())), f"{name}: layer {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first_token(engines, name, dtype):
    """Every token a step of its own (captured steps): the first tokens of a sequence, whose states begin from zeros,
    and on across window and page borders."""
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    toks = random_tokens(vocab(name), 150, 8)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = torch.cat([eng.step([Entry(s, [t], [0])]) for t in toks])
    eng.close(s)
    assert_close(got, ref, dtype, f"{name} {dtype} token by token")
    assert any(c.graph is not None for c in eng._captured.values())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["PA", "PT"])
def test_branches_on_two_streams_change_no_bit(name, dtype):
    """Single-token steps run the feed-forward on a second stream beside the mixer (captured: two branches of the graph).
    The same steps with the branches one after the other, and a second time on two streams in slots and pages used again,
    give the same bits: nothing of one branch is read or overwritten by the other before the streams have met."""
    from synaptix_b200 import ops
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    toks = [random_tokens(vocab(name), n, 60 + n) for n in (90, 37, 64)]

    def run(eng):
        slots = [eng.open() for _ in toks]
        out = [eng.step([Entry(s, t[:20], [19]) for s, t in zip(slots, toks)])]
        for j in range(20, 37):
            out.append(eng.step([Entry(s, [t[j]], [0]) for s, t in zip(slots, toks)]))
        for j in range(37, 64):                                  # the shorter requests end earlier
            out.append(eng.step([Entry(s, [t[j]], [0]) for s, t in zip(slots[::2], toks[::2])]))
        for s in slots:
            eng.close(s)
        return torch.cat(out).cpu()
    with ops.options(branch_streams=False):
        eng = Engine(load_model(folder(name), dtype=dtype), max_tokens=1024, max_seqs=3)
        ref = run(eng)
    eng = Engine(load_model(folder(name), dtype=dtype), max_tokens=1024, max_seqs=3)
    first, second = run(eng), run(eng)
    assert any(c.graph is not None for c in eng._captured.values())
    assert torch.equal(first, ref) and torch.equal(second, ref)


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
        rows = Gathered(dtype, f"{name} batch {b}")
        got = eng.step([Entry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)])
        rows.add(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), "prompts")
        live = list(range(len(seqs)))
        for j in range(max(decodes)):
            live = [i for i in live if j < decodes[i]]
            got = eng.step([Entry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in live])
            rows.add(got, torch.stack([refs[i][lens[i] + j] for i in live]), f"decode {j}")
            for i in live:
                if j == decodes[i] - 1:
                    eng.close(slots[i])
        rows.check()
    assert eng.cache.slots.n_live == 0


@pytest.mark.parametrize("name", ["PA", "PB"])
def test_long_decoding_gives_pages_behind_the_window_back(engines, name):
    """400 tokens one by one behind a prompt, in a cache of 5 pages: it only fits because pages behind the widest window
    that reads an entry are given back (70 and 130 positions in these models)."""
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
            lg = PP.forward(cfg, W, seq)[-1]
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
    name = "PA"
    V = vocab(name)
    seqs = {f"q{i}": random_tokens(V, n, 800 + i) for i, n in enumerate([31, 75, 12, 50])}
    refs = {k: oracle_logits(name, tuple(v)) for k, v in seqs.items()}
    r = Replay(folder(name), dtype, str(tmp_path), 192)
    heads = {"q0": 20, "q1": 60, "q2": 11}
    rows = Gathered(dtype, "replay")
    got = r.step([{"id": k, "tokens": seqs[k][:h], "want": [0, h - 1]} for k, h in heads.items()])
    rows.add(got, torch.stack([refs[k][j] for k, h in heads.items() for j in (0, h - 1)]), "prompts")
    at = dict(heads)
    while at:
        live = list(at)
        ends = [k for k in live if at[k] + 1 == len(seqs[k])]
        got = r.step([{"id": k, "tokens": [seqs[k][at[k]]], "want": [0]} for k in live], end=ends)
        rows.add(got, torch.stack([refs[k][at[k]] for k in live]), f"decode {sorted(at.values())}")
        for k in live:
            at[k] += 1
            if k in ends:
                del at[k]
    got = r.step([{"id": "q3", "tokens": seqs["q3"], "want": [45, 46, 47, 48, 49]}], end=["q3"])
    rows.add(got, refs["q3"][45:50], "afterwards")
    rows.check()
    r.finish()


def test_command_line_run_and_inspect(tmp_path):
    """``python -m synaptix_b200 run`` chooses the model by config.json and generates greedily; ``inspect`` lists its layers."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "PB"
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
        lg = PP.forward(cfg, W, seq)[-1]
        top2 = lg.topk(2).values
        if float(top2[0] - top2[1]) > 1e-3 * float(lg.abs().max()):
            assert tok == int(lg.argmax())
        seq.append(tok)
    assert out["prompt_tokens"] == 9 and out["new_tokens"] == 6
    r = subprocess.run([sys.executable, "-m", "synaptix_b200", "inspect", folder(name)], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "architecture: Pidutar" in r.stdout, r.stdout + r.stderr

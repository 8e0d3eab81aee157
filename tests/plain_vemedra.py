"""A plain, slow implementation of the Vemedra decoder on the CPU: one function per mechanism, straight from the
equations, whole sequences only, no cache and no batching.  It shares nothing with the package (it reads model
folders with the ``safetensors`` package) and is what the GPU tests compare the engine with.

Notation: ``x`` is the residual stream ``[T, width]``, ``h`` what a sublayer reads, positions count from 0.
"""
import json
import os

import torch


def load_folder(path, dtype=torch.float64):
    from safetensors.torch import load_file
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    W = {k: v.to(dtype) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}
    return cfg, W


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def token_conv(h, w):
    """h + causal depthwise convolution over time: out_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j] * h[:T - back]
    return out


def mingru(h, W, p):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t with z = sigmoid(Wz h + bz), c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0),
    u = Wx h + bx; out = Wo (S_t * silu(Wg h))."""
    z = torch.sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ W[p + "g"].T
    S = torch.zeros(z.shape[1], dtype=h.dtype)
    rows = []
    for t in range(h.shape[0]):
        S = (1 - z[t]) * S + z[t] * c[t]
        rows.append(S)
    return (torch.stack(rows) * torch.nn.functional.silu(g)) @ W[p + "o"].T


def rotate_half(x, pos, dims, base):
    """x [T, heads, dim]: the first ``dims`` elements of each head rotated, element i paired with i + dims/2."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = pos.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def chunk_sink_heads(q, k, v, pos, sinks, scale, cap, size):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of ONE sequence at positions ``pos``: softmax attention in which position i
    sees j <= i of its own chunk of ``size`` positions (None: all), scores capped by ``cap * tanh(. / cap)`` (None: not),
    and exp(sink_h) in the denominator (None: no sink).  Returns [T, H, Dv]."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    see = pos[None, :] <= pos[:, None]
    if size is not None:
        see = see & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * scale
        if cap is not None:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~see, float("-inf"))
        top = s.max(dim=-1).values
        if sinks is not None:
            top = torch.maximum(top, sinks[hh])
        e = torch.exp(s - top[:, None])
        den = e.sum(dim=-1)
        if sinks is not None:
            den = den + torch.exp(sinks[hh] - top)
        out[:, hh] = (e / den[:, None]) @ v[:, g]
    return out


def chunk_sink_attention(h, W, p, m):
    """Grouped-query softmax attention inside chunks of ``mask.size`` positions, with capped scores and a sink."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, G, D)
    v = (h @ W[p + "v"].T).view(T, G, Dv)
    pos = torch.arange(T)
    if m.get("rot"):
        q = rotate_half(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"])
    out = chunk_sink_heads(q, k, v, pos, W[p + "sink"], m["scale"], m.get("softcap"), (m.get("mask") or {}).get("size"))
    return out.reshape(T, H * Dv) @ W[p + "o"].T


def retention(h, W, p, m, eps):
    """Per head S_t = decay S_(t-1) + k_t v_t^T with k scaled by dim^-1/2, o_t = S_t^T q_t; o / rms(o), gated, projected."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, H, D) * D ** -0.5
    v = (h @ W[p + "v"].T).view(T, H, Dv)
    g = h @ W[p + "g"].T
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    rows = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        rows.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = rms_unit(torch.stack(rows), eps).reshape(T, H * Dv)
    return (o * torch.nn.functional.silu(g)) @ W[p + "o"].T


def capped_glu(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + "down"].T


def mixer(h, W, layer, i, eps):
    p = f"l{i}.mix."
    if layer["type"] == "mingru":
        return mingru(h, W, p)
    if layer["type"] == "parallel":
        m = layer["mixer"]
        return (m["left_scale"] * chunk_sink_attention(h, W, p + "left.", m["left"])
                + m["right_scale"] * retention(h, W, p + "right.", m["right"], eps))
    raise ValueError(layer["type"])


def run_layer(x, W, layer, i, eps):
    x = x + mixer(token_conv(rms_norm(x, W[f"l{i}.norm1"], eps), W[f"l{i}.canon1"]), W, layer, i, eps)
    if layer["mlp"] is not None:
        h = token_conv(rms_norm(x, W[f"l{i}.norm2"], eps), W[f"l{i}.canon2"])
        x = x + capped_glu(h, W, f"l{i}.mlp.", layer["mlp"]["limit"])
    return x


def forward(cfg, W, tokens, streams=None):
    """Logits ``[T, vocab]`` of one whole sequence; ``streams`` (a list) collects the residual stream after each layer run."""
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][torch.tensor(tokens)]
    x = x0.clone()
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    order += [(i, None) for i in range(loop["stop"], len(cfg["layers"]))]
    for i, first_of_pass in order:
        if first_of_pass is not None:
            if first_of_pass > 0:
                x = x + x0
            x = x + W["loop.step"][first_of_pass]
        x = run_layer(x, W, cfg["layers"][i], i, eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T

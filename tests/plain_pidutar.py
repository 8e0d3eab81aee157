"""A plain, slow implementation of the Pidutar decoder on the CPU: one function per mechanism, straight from the
equations, whole sequences only, no cache and no batching.  It shares nothing with the package (it reads model
folders with the ``safetensors`` package) and is what the GPU tests compare the engine with.

Notation: ``x`` is the residual stream ``[T, width]``, ``h`` what a sublayer reads, positions count from 0.
"""
import json
import math
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


def norm_around_zero(x, w, eps):
    """The layers' norm: the stored weight lies around zero and the gain is 1 + w."""
    return rms_unit(x, eps) * (1.0 + w)


def rotate_pairs(x, pos, dims, base):
    """x [T, ..., n]: the first ``dims`` elements rotated, element 2i paired with element 2i + 1, by the angle
    pos * base^(-2i / dims); elements from ``dims`` on pass unchanged."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = pos.to(x.dtype)[:, None] * f[None, :]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def capped(z, cap):
    return cap * torch.tanh(z / cap)


def mlstm(h, W, p, m, eps):
    """The matrix memory with a running maximum that starts at 0.  Per head: log input gate i, log forget gate f,
    M_t = max(f + M_(t-1), i), S_t = exp(f + M_(t-1) - M_t) S_(t-1) + exp(i - M_t) k v^T, n_t the same with k alone,
    o = S_t^T q / (max(|n_t . q|, exp(-M_t)) + 1e-6); each head's o over its root mean square, times the gain over
    all heads, times sigmoid(Wg h), then Wo."""
    T = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ W[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, Dv)
    gi = capped(h @ W[p + "i"].T + W[p + "i.b"], cap)
    gf = torch.nn.functional.logsigmoid(capped(h @ W[p + "f"].T + W[p + "f.b"], cap))
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    M = torch.zeros(H, dtype=h.dtype)
    rows = []
    for t in range(T):
        M_new = torch.maximum(gf[t] + M, gi[t])
        a = torch.exp(gf[t] + M - M_new)
        b = torch.exp(gi[t] - M_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        M = M_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-M)) + 1e-6
        rows.append(num / den[:, None])
    o = rms_unit(torch.stack(rows), eps).reshape(T, H * Dv) * W[p + "norm"]
    return (o * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def latent_keys(h, W, p, m, pos, eps):
    """What a latent attention layer keeps per token: the normed latent c [T, kv_rank] and the rotated key part
    [T, rot_dim] that all heads share."""
    R = m["kv_rank"]
    d = h @ W[p + "dkv"].T
    c = rms_unit(d[:, :R], eps) * W[p + "dkv.norm"]
    kr = d[:, R:]
    if m.get("rot"):
        kr = rotate_pairs(kr, pos, m["rot"]["dims"], m["rot"]["base"])
    return c, kr


def latent_attention(h, W, p, m, pos, eps, kept):
    """Attention whose keys and values are made per head from the kept latent: q through a normed latent of its own,
    score = (q_plain . (Wuk c) + q_rot . k_rot) * scale over the keys of the window, softmax, values Wuv c, each head
    times sigmoid(Wg h) of that head, then Wo."""
    T = h.shape[0]
    H, D, Dr, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kept
    cq = rms_unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, D + Dr)
    qp, qr = q[..., :D], q[..., D:]
    if m.get("rot"):
        qr = rotate_pairs(qr, pos, m["rot"]["dims"], m["rot"]["base"])
    kp = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, Dv)
    diff = pos[:, None] - pos[None, :]
    see = diff >= 0
    if m.get("mask"):
        see = see & (diff < m["mask"]["size"])
    g = torch.sigmoid(h @ W[p + "g"].T)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for hh in range(H):
        s = (qp[:, hh] @ kp[:, hh].T + qr[:, hh] @ kr.T) * m["scale"]
        s = s.masked_fill(~see, -math.inf)
        out[:, hh] = torch.softmax(s, dim=-1) @ v[:, hh]
    out = out * g[:, :, None]
    return out.reshape(T, H * Dv) @ W[p + "o"].T


def experts(h, W, p, f):
    """A mixture of small gated feed-forwards: softmax of the router's logits over all experts, the ``top`` largest
    chosen, their scores divided by their sum (+ 1e-20) and multiplied by router.scale, the weighted sum of the chosen
    experts' outputs down(silu(gate h) * (up h))."""
    r = f["router"]
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    top, idx = torch.topk(s, r["top"], dim=-1)
    w = top / (top.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = p + "e%d." % int(idx[t, j])
            z = torch.nn.functional.silu(h[t] @ W[e + "gate"].T) * (h[t] @ W[e + "up"].T)
            out[t] += w[t, j] * (z @ W[e + "down"].T)
    return out


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that takes the stream after every layer."""
    dtype = W["embed"].dtype
    eps = cfg["norm"]["eps"]
    pos = torch.arange(len(tokens))
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = layer["mixer"]
        h = norm_around_zero(x, W[p + "norm1"], eps)
        if layer["type"] == "mlstm":
            a = mlstm(h, W, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_keys(h, W, p + "mix.", m, pos, eps)
                mine = kept[i]
            else:
                mine = kept[m["kv_from"]]
            a = latent_attention(h, W, p + "mix.", m, pos, eps, mine)
        else:
            raise ValueError(layer["type"])
        branch = a * W[p + "ls1"]
        if layer.get("mlp") is not None:
            b = experts(norm_around_zero(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
            branch = branch + b * W[p + "ls2"]
        x = x + cfg["residual_mult"] * branch
        if layers_out is not None:
            layers_out.append(x.clone())
    y = norm_around_zero(x, W["final.norm"], eps)
    return (y @ W["head"].T) * cfg["logit_scale"]

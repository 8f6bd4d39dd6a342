"""A plain, slow implementation of the Kebudra design in float32 on the CPU: one function per mechanism, whole
sequences at once, no cache.  It shares no code with the package; tests compare the package with it.

Notation: T tokens, W model width, H query heads, G key/value heads, D key size, Dv value size.  Weights are given
as a dict of float32 tensors by their checkpoint names; linear weights are [out, in]."""
from __future__ import annotations

import math

import torch


def lin(x, w):
    return x @ w.t()


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def dyt(x, alpha, w, b):
    """Dynamic tanh: an elementwise squashing in place of a norm; no statistics of the row."""
    return torch.tanh(alpha * x) * w + b


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x, pos, dims, base):
    """Rotates the first ``dims`` entries of the last axis; entry 2i goes with 2i + 1.  x [T, ..., n], pos [T]."""
    i = torch.arange(dims // 2, dtype=torch.float32)
    f = base ** (-2.0 * i / dims)
    ang = pos.to(torch.float32)[:, None] * f[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_softmax(scores):
    """scores [H, T, T] -> weights; a query sees keys at its own and earlier positions."""
    T = scores.shape[-1]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), -1)


# --------------------------------------------------------------------------- mixers

def differential_attention(h, p, m, eps, kv=None):
    """Two softmax maps per head over the same values, subtracted.  ``p``: the mixer's tensors (q, k, v, lq1, lk1,
    lq2, lk2, g, o), ``m``: its sizes and constants.  ``kv`` = (k, v) of another layer for a layer that borrows them.
    Returns (output, (k, v))."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, p["q"]).view(T, H, 2, D)
    if kv is None:
        k = lin(h, p["k"]).view(T, G, 2, D)
        v = lin(h, p["v"]).view(T, G, Dv)
    else:
        k, v = kv
    rep = H // G
    kk = k.repeat_interleave(rep, 1)                    # head h reads key/value head h // rep
    vv = v.repeat_interleave(rep, 1)
    outs = []
    for j in range(2):
        s = torch.einsum("thd,uhd->htu", q[:, :, j], kk[:, :, j]) * m["scale"]
        outs.append(torch.einsum("htu,uhe->the", causal_softmax(s), vv))
    lam = math.exp(float((p["lq1"] * p["lk1"]).sum())) - math.exp(float((p["lq2"] * p["lk2"]).sum())) + m["diff"]
    o = outs[0] - lam * outs[1]
    o = rms(o, eps) * (1 - m["diff"])
    o = o * torch.sigmoid(lin(h, p["g"]))[:, :, None]
    return lin(o.reshape(T, H * Dv), p["o"]), (k, v)


def latent_attention(h, p, m, eps, pos):
    """Queries and keys/values through low-rank latents; a rotated key part shared by all heads."""
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(lin(h, p["dq"]), eps) * p["dq.norm"]
    q = lin(cq, p["uq"]).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    dkv = lin(h, p["dkv"])
    c = rms(dkv[:, :C], eps) * p["dkv.norm"]
    k_rot = rotate_pairs(dkv[:, C:], pos, m["rot"]["dims"], m["rot"]["base"])          # [T, R], one for all heads
    k_plain = lin(c, p["uk"]).view(T, H, D)
    v = lin(c, p["uv"]).view(T, H, Dv)
    s = (torch.einsum("thd,uhd->htu", q_plain, k_plain) + torch.einsum("thr,ur->htu", q_rot, k_rot)) * m["scale"]
    o = torch.einsum("htu,uhe->the", causal_softmax(s), v).reshape(T, H * Dv)
    o = o * torch.sigmoid(lin(h, p["g"]))
    return lin(o, p["o"])


def short_conv_silu(x, taps):
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, j] x_{t - (K-1) + j}, zeros before the start; then silu."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C), x], 0)
    y = torch.zeros(T, C)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y * torch.sigmoid(y)


def channel_delta(h, p, m, eps):
    """The gated delta rule with one decay per head and key channel, token by token."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(lin(h, p["q"]), p["q.conv"]).view(T, G, D)
    k = short_conv_silu(lin(h, p["k"]), p["k.conv"]).view(T, G, D)
    v = short_conv_silu(lin(h, p["v"]), p["v.conv"]).view(T, H, Dv)
    unit = lambda x: x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * D ** -0.5, unit(k)
    beta = torch.sigmoid(lin(h, p["b"]))                                                # [T, H]
    dt = torch.nn.functional.softplus(lin(lin(h, p["a1"]), p["a2"]) + p["dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(p["A_log"])[None, :, None] * dt)                       # [T, H, D]
    gate = torch.sigmoid(lin(lin(h, p["g1"]), p["g2"])).view(T, H, Dv)
    rep = H // G
    S = torch.zeros(H, D, Dv)
    out = torch.zeros(T, H, Dv)
    for t in range(T):
        kt, qt = k[t].repeat_interleave(rep, 0), q[t].repeat_interleave(rep, 0)          # [H, D]
        S = decay[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, qt)
    out = rms(out, eps) * p["norm"] * gate
    return lin(out.reshape(T, H * Dv), p["o"])


# --------------------------------------------------------------------------- feed-forward

def routed_experts(h, p, m):
    """Each token goes to the ``top`` experts with the largest router logits, weighted by the softmax over those
    logits alone.  An expert is down(relu(up h)^2)."""
    top = m["router"]["top"]
    z = lin(h, p["router"])
    val, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(val, -1)
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0])
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            a = torch.relu(lin(h[t], p[f"e{e}.up"])) ** 2
            out[t] += w[t, j] * lin(a, p[f"e{e}.down"])
    return out


# --------------------------------------------------------------------------- the model

def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, layer_outputs: list | None = None):
    """Logits [T, vocab] of one sequence.  ``layer_outputs`` (a list) receives the sum of the streams after every layer."""
    w = {k: v.float() for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.numel()
    pos = torch.arange(T)
    S = int(cfg.get("streams", 1))
    x = (w["embed"][tokens] * cfg["embedding"]["scale"]).unsqueeze(0).repeat(S, 1, 1)    # [S, T, W]
    norm = lambda name, u: dyt(u, w[name + ".alpha"], w[name], w[name + ".b"])
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        for qn, name in ((1, "mixer"), (2, "mlp")):
            if name == "mlp" and layer.get("mlp") is None:
                continue
            if S > 1 or (L + f"hc{qn}.in") in w:
                cin, cout, cmix = w[L + f"hc{qn}.in"], w[L + f"hc{qn}.out"], w[L + f"hc{qn}.mix"]
            else:
                cin, cout, cmix = torch.ones(1), torch.ones(1), torch.ones(1, 1)
            u = torch.einsum("s,stw->tw", cin, x)
            hin = norm(L + f"norm{qn}", u)
            if name == "mlp":
                y = routed_experts(hin, sub(w, L + "mlp."), layer["mlp"])
            else:
                m, p = layer["mixer"], sub(w, L + "mix.")
                if layer["type"] == "attention":
                    src = m.get("kv_from")
                    y, kv = differential_attention(hin, p, m, eps, kept[src] if src is not None else None)
                    kept[i] = kv
                elif layer["type"] == "latent_attention":
                    y = latent_attention(hin, p, m, eps, pos)
                elif layer["type"] == "channel_delta":
                    y = channel_delta(hin, p, m, eps)
                else:
                    raise ValueError(layer["type"])
            x = torch.einsum("sr,stw->rtw", cmix, x) + cout[:, None, None] * y[None]
        if layer_outputs is not None:
            layer_outputs.append(x.sum(0))
    xs = norm("final.norm", x.sum(0))
    return lin(xs, w["head"])

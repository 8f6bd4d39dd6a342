"""Plain, slow Getizen: the oracle that the engine tests of this design compare with.

Whole sequences, no cache, no batching, float32 on the CPU, one function per mechanism, written from the
design's equations and sharing no code with the package.  ``cfg`` is the parsed config.json, ``W`` a
``{tensor name: float32 tensor}`` dict.

The design in this file's notation (t: token index = position, x_t: residual stream, d: model width):

  embedding          x_t = gnorm(E[token_t]; w_embed_norm)
  layer              x <- gnorm(alpha x + mixer(x); w_norm1);  x <- gnorm(alpha x + ff(x); w_norm2)
  gnorm(v; w)        v cut into ``groups`` equal consecutive parts, each part / sqrt(mean(part^2) + eps); times w
  ff(h)              g = min(Wg h, L), u = clip(Wu h, -L, L);  Wd (g sigmoid(1.702 g) (u + 1))
  rotation           pairs (i, i + n/2) of the first n dims of a head turn by the angle t f_i, f_i = base^(-2i/n);
                     optionally f_i rescaled by wavelength (long waves divided by ``factor``, a linear blend between)
  retention          per head S_t = gamma S_{t-1} + k_t v_t^T, o_t = S_t^T q_t (k scaled by dim^-1/2 after rotation);
                     o / rms(o) per head, times silu(Wg h), then Wo
  chunked attention  softmax attention with grouped key/value heads, q and k RMS-normed over the whole projection,
                     rotated, score scaled by ``scale`` and a per-head temperature; key j visible to query t when
                     j <= t and both lie in the same block of ``mask.size`` positions; output gated by sigmoid(Wg h)
  gated recurrence   y = gelu_tanh(Wy h + by); u = causal_conv(Wx h + bx); per block of channels r = sigmoid(Ra u + ra),
                     i = sigmoid(Ri u + ri); a = exp(-8 r softplus(lam)); s_t = a s_{t-1} + sqrt(1 - a^2) (i u); Wo (s y)
  parallel mixer     (rms(attention(h)) w_left + rms(recurrence(h)) w_right) / 2
  head               logits = E gnorm(x; w_final)
"""
from __future__ import annotations

import math

import torch


def rms_scale(v: torch.Tensor, eps: float) -> torch.Tensor:
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def group_norm(v: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    parts = v.reshape(*v.shape[:-1], groups, v.shape[-1] // groups)
    return rms_scale(parts, eps).reshape(v.shape) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def feed_forward(h: torch.Tensor, W: dict, p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def frequencies(rot: dict) -> torch.Tensor:
    """f_i for i < dims/2, rescaled by wavelength where the config asks for it."""
    n = rot["dims"]
    f = [rot["base"] ** (-2.0 * i / n) for i in range(n // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float32)


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]: the first ``dims`` dimensions of every head turn, the rest pass."""
    n = rot["dims"]
    if n == 0:
        return x
    ang = positions.float()[:, None] * frequencies(rot)[None, :]            # [T, n/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :n // 2], x[..., n // 2:n]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., n:]], -1)


def retention(h: torch.Tensor, W: dict, p: str, m: dict, eps: float, positions=None) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T) if positions is None else positions
    q = rotate((h @ W[p + "q"].T).reshape(T, H, D), pos, m["rot"])
    k = rotate((h @ W[p + "k"].T).reshape(T, H, D), pos, m["rot"]) * D ** -0.5
    v = (h @ W[p + "v"].T).reshape(T, H, Dv)
    out = torch.zeros(T, H, Dv)
    for hd in range(H):
        S = torch.zeros(D, Dv)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = rms_scale(out, eps).reshape(T, H * Dv)
    g = h @ W[p + "g"].T
    return (out * g * torch.sigmoid(g)) @ W[p + "o"].T


def chunked_attention(h: torch.Tensor, W: dict, p: str, m: dict, eps: float, positions=None) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T) if positions is None else positions
    q = rms_scale(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    k = rms_scale(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    q = rotate(q.reshape(T, H, D), pos, m["rot"])
    k = rotate(k.reshape(T, G, D), pos, m["rot"])
    v = (h @ W[p + "v"].T).reshape(T, G, Dv)
    size = m["mask"]["size"]
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros(T, H, Dv)
    for hd in range(H):
        kv = hd // (H // G)
        score = (q[:, hd] @ k[:, kv].T) * m["scale"] * W[p + "temp"][hd]
        score = score.masked_fill(~seen, float("-inf"))
        out[:, hd] = torch.softmax(score, -1) @ v[:, kv]
    gate = torch.sigmoid(h @ W[p + "g"].T)
    return (out.reshape(T, H * Dv) * gate) @ W[p + "o"].T


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K] with the last column on the current token, zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1]), x], 0)
    out = bias.expand(T, -1).clone()
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def gated_recurrence(h: torch.Tensor, W: dict, p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    C, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
    u = causal_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    ub = u.reshape(T, B, C // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ra"], ub) + W[p + "ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ri"], ub) + W[p + "ri.b"]).reshape(T, C)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(W[p + "lam"]))
    inp = torch.sqrt(1.0 - a * a) * (i * u)
    s, out = torch.zeros(C), torch.zeros(T, C)
    for t in range(T):
        s = a[t] * s + inp[t]
        out[t] = s
    return (out * y) @ W[p + "o"].T


def parallel_mixer(h: torch.Tensor, W: dict, p: str, m: dict, eps: float, positions=None) -> torch.Tensor:
    left = chunked_attention(h, W, p + "left.", m["left"], eps, positions)
    right = gated_recurrence(h, W, p + "right.", m["right"])
    return 0.5 * (rms_scale(left, eps) * W[p + "left.out"] + rms_scale(right, eps) * W[p + "right.out"])


def forward(cfg: dict, W: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of a whole sequence from position 0 (and the stream after every layer)."""
    W = {k: v.float() for k, v in W.items()}
    eps, groups, alpha = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["postln_alpha"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = group_norm(W["embed"][ids], W["embed.norm"], groups, eps)
    streams = []
    for n, layer in enumerate(cfg["layers"]):
        p = f"l{n}."
        if layer["type"] == "retention":
            mix = retention(x, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            mix = parallel_mixer(x, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = group_norm(alpha * x + mix, W[p + "norm1"], groups, eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            x = group_norm(alpha * x + feed_forward(x, W, p + "mlp.", layer["mlp"]["limit"]), W[p + "norm2"], groups, eps)
        streams.append(x)
    logits = group_norm(x, W["final.norm"], groups, eps) @ W["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits

"""Plain, slow restatement of the Fonuvik decoder: one function per mechanism, whole sequences at once,
float64 on the CPU.  It shares no code with the package: it reads a raw configuration (the keys of
config.json) and a dict of tensors under the checkpoint's names.

  stream           x = n_e(embed[token]);  per layer  x += n_1b(mixer(n_1(x)));  x += n_2b(ff(n_2(x)));  logits = embed n_f(x)
                   every n is an rms norm with a weight: y = x / sqrt(mean(x^2) + eps) * w
  mixer parallel   a_left * left(h) + a_right * right(h)
     left          grouped-query softmax attention: interleaved rotation of the first `dims` elements of each head with
                   frequencies rescaled by wavelength, then q and k divided by their root mean square per head, scores
                   times `scale`, a key visible only inside the query's block of `size` positions (and not after it)
     right         linear attention with a decay per key channel: S = diag(a_t) S + k_t v_t^T, o_t = S^T q_t,
                   a = sigmoid(z)^(1/tau); rms norm of o per head with one weight, times silu(Wg h), then Wo
  mixer wkv        every projection reads its own blend of h_t and h_(t-1); w = exp(-exp(.)) per key channel;
                   o_t = (S + diag(u) k_t v_t^T)^T r_t, then S = diag(w_t) S + k_t v_t^T; o / rms(o) per head, times a
                   weight over all heads, times silu(gate), then Wo
  feed-forward     the `top` largest router logits (bias included) choose experts, softmax over the chosen logits weighs
                   them; every expert is Wdown (silu(Wgate h) * (Wup h)); one more expert of the same form runs for all
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------------------- rotation
def rescaled_frequencies(dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i = base^(-2i/dims); with `scaling` {factor, low, high, original}: waves shorter than original/high stay,
    waves longer than original/low turn `factor` times slower, those between are blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave > original / low:
                f = f / factor
            elif not wave < original / high:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, freq: torch.Tensor) -> torch.Tensor:
    """x [T, heads, n]: elements (2i, 2i+1), i < dims/2, are turned by position * freq_i; the rest pass."""
    a = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---------------------------------------------------------------------------------------- left: softmax attention in blocks
def visible(T: int, block: Optional[int]) -> torch.Tensor:
    """[T, T] bool: key j is visible to query i when j <= i and, with blocks, both lie in the same block of positions."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if block:
        ok = ok & (i // block == j // block)
    return ok


def block_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, block: Optional[int]) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; query head h reads key/value head h // (H / G).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    rep = H // k.shape[1]
    mask = visible(T, block)
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, h // rep]
    return out


def softmax_mixer(h, positions, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, G, dk)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        freq = rescaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_pairs(q, positions, rot["dims"], freq), rotate_pairs(k, positions, rot["dims"], freq)
    q, k = rms(q, eps), rms(k, eps)
    block = (m.get("mask") or {}).get("size")
    o = block_attention(q, k, v, float(m["scale"]), block).reshape(T, H * dv)
    return o @ w[p + "o"].T


# ---------------------------------------------------------------------------------------- the two recurrences
def decayed_sum(q, k, v, a, state: Optional[torch.Tensor] = None):
    """q, k, a [T, H, dk], v [T, H, dv]:  S = diag(a_t) S + k_t v_t^T;  o_t = S^T q_t.  Returns (o, S)."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, v.shape[-1], dtype=F)
    for t in range(T):
        S = S * a[t][:, :, None] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def bonus_sum(r, k, v, w, u, state: Optional[torch.Tensor] = None):
    """r, k, w [T, H, d], v [T, H, dv], u [H, d]:  o_t = (S + diag(u) k_t v_t^T)^T r_t;  then S = diag(w_t) S + k_t v_t^T."""
    T, H, d = r.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, v.shape[-1], dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = S * w[t][:, :, None] + kv
    return o, S


def decay_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    a = torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).view(T, H, dk)
    o, _ = decayed_sum(q, k, v, a)
    o = (rms(o, eps) * w[p + "norm"]).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def shifted(h: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row t holds h_(t-1); the row in front of the first is `before` (zeros at the start of a sequence)."""
    first = torch.zeros(1, h.shape[1], dtype=h.dtype) if before is None else before.view(1, -1)
    return torch.cat([first, h[:-1]], 0)


def wkv_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    back = shifted(h) - h
    blend = lambda s: h + back * w[p + "mu." + s]
    r = (blend("r") @ w[p + "r"].T).view(T, H, d)
    k = (blend("k") @ w[p + "k"].T).view(T, H, d)
    v = (blend("v") @ w[p + "v"].T).view(T, H, d)
    gate = silu(blend("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(blend("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    o, _ = bonus_sum(r, k, v, decay, w[p + "u"])
    o = rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


# ---------------------------------------------------------------------------------------- feed-forward
def gated_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, top: int):
    """(chosen experts [T, top], their weights [T, top])."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    best, ids = torch.topk(z, top, dim=-1)
    return ids, torch.softmax(best, -1)


def experts_ff(h, w, p: str, mlp: dict) -> torch.Tensor:
    ids, weights = route(h, w, p, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            out[t] += weights[t, j] * gated_ff(h[t:t + 1], w, f"{p}e{int(ids[t, j])}.")[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------------------------------- the model
def mixer(raw_layer: dict, h, positions, w, p: str, eps: float) -> torch.Tensor:
    m = raw_layer["mixer"]
    if raw_layer["type"] == "parallel":
        left = softmax_mixer(h, positions, w, p + "left.", m["left"], eps)
        right = decay_mixer(h, w, p + "right.", m["right"], eps)
        return float(m["left_scale"]) * left + float(m["right_scale"]) * right
    if raw_layer["type"] == "wkv":
        return wkv_mixer(h, w, p, m, eps)
    raise ValueError(raw_layer["type"])


def forward(raw: dict, weights: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; `layers_out` receives the stream after every layer."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = float(raw["norm"]["eps"])
    positions = torch.arange(len(tokens))
    x = rms(w["embed"][torch.tensor(tokens)], eps) * w["embed.norm"]
    for i, layer in enumerate(raw["layers"]):
        p = f"l{i}."
        x = x + rms(mixer(layer, rms(x, eps) * w[p + "norm1"], positions, w, p + "mix.", eps), eps) * w[p + "norm1b"]
        if layer.get("mlp") is not None:
            x = x + rms(experts_ff(rms(x, eps) * w[p + "norm2"], w, p + "mlp.", layer["mlp"]), eps) * w[p + "norm2b"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["embed"].T

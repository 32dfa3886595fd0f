"""Plain, slow restatement of the Lozepel decoder: one function per mechanism, whole sequences at once, float64 on
the CPU.  It shares no code with the package: it reads a raw configuration (the keys of config.json) and a dict of
tensors under the checkpoint's names.

  stream        x_t = E[tok_t] + B[(tok_(t-1) * a + tok_t * b) mod n]   (row n of B for a sequence's first token)
                per layer  x += n_1b(mixer(n_1(x)));  x += n_2b(ff(n_2(x)))      (the second line only with a feed-forward)
                logits = c * tanh(W_head n_f(x) / c);   every n:  y = x / sqrt(mean(x^2) + eps) * (1 + w)
  attention     q = Wq h + bq, k = Wk h + bk, v = k before its rotation; interleaved rotation of the first `dims` elements
                of each head; p_j = exp(s_j) / (1 + sum_i exp(s_i)); each head's output times sigmoid(Wg h)_head; Wo
  parallel      a_l * left(h) + a_r * right(h)
     left       q, k each divided by the root mean square of their WHOLE row, times a weight of that length; no rotation;
                the softmax's denominator also holds exp(sink_head); head gate as above; Wo
     right      q, k, v = silu(W. h); per head S = d_head S + k_t v_t^T, o_t = S^T q_t; the heads side by side are
                normalised together (weight without the one), times sigmoid(Wg h) element by element, then Wo
  attention_2   interleaved rotation, then q and k of each head divided by their root mean square; s = cap * tanh(q.k *
                scale / cap); the denominator also holds exp(sink_head); no gate; a layer with `kv_from` has no key or
                value projections and reads the keys and values of the layer it names
  feed-forward  dense: g = min(Wg h, L), u = clamp(Wu h, -L, L), y = Wd (g * sigmoid(1.702 g) * (u + 1))
                routed: s = softmax(Wr h) over all outputs; the `top` largest s + correction are chosen; each adds
                s_e * expert_e(h), expert_e(h) = Wd_e (silu(Wg_e h) * (Wu_e h)), or s_e * h for the last `identity` outputs
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

F = torch.float64


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rms_quotient(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def stream_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The stream's norms store their weight around zero."""
    return rms_quotient(x, eps) * (1.0 + w.to(F))


# ---------------------------------------------------------------------------------------- embedding
def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embed(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    x = w["embed"].to(F)[torch.tensor(tokens)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + w["bigram"].to(F)[torch.tensor(bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"]))]
    return x


# ---------------------------------------------------------------------------------------- rotation
def rotate_pairs(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, n]: elements (2i, 2i+1), i < dims/2, are turned by t * base^(-2i/dims); the rest pass."""
    T = x.shape[0]
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    a = torch.arange(T, dtype=F)[:, None] * freq[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---------------------------------------------------------------------------------------- softmax attention with a sink
def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: torch.Tensor,
                   cap: Optional[float] = None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv], sink [H]; query head h reads key/value head h // (H / G); a query at t
    sees keys 0..t.  p_j = exp(s_j) / (exp(sink_h) + sum_i exp(s_i)).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=F)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[: t + 1, g] @ q[t, h]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[t, h] = (e[:, None] * v[: t + 1, g]).sum(0) / (e.sum() + torch.exp(sink[h] - m))
    return out


def head_gate(o: torch.Tensor, wg: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """o [T, H, dv] times sigmoid(Wg h) [T, H], one number per head."""
    return o * torch.sigmoid(h @ wg.to(F).T)[:, :, None]


def mixer_attention(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    T, H, G, dk = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].to(F).T + w[p + "q.b"].to(F)).view(T, H, dk)
    k = (h @ w[p + "k"].to(F).T + w[p + "k.b"].to(F)).view(T, G, dk)
    v = k.clone()
    rot = m.get("rot")
    if rot:
        q, k = rotate_pairs(q, rot["dims"], rot["base"]), rotate_pairs(k, rot["dims"], rot["base"])
    o = sink_attention(q, k, v, m["scale"], torch.zeros(H, dtype=F))
    return head_gate(o, w[p + "g"], h).reshape(T, -1) @ w[p + "o"].to(F).T


def mixer_attention_2(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float, shared=None):
    """Returns (result, (k, v)); `shared`: the (k, v) of the layer this one reads instead of projecting its own."""
    T, H, G, dk, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    q = (h @ w[p + "q"].to(F).T).view(T, H, dk)
    if rot:
        q = rotate_pairs(q, rot["dims"], rot["base"])
    q = rms_quotient(q, eps)
    if shared is None:
        k = (h @ w[p + "k"].to(F).T).view(T, G, dk)
        v = (h @ w[p + "v"].to(F).T).view(T, G, dv)
        if rot:
            k = rotate_pairs(k, rot["dims"], rot["base"])
        k = rms_quotient(k, eps)
    else:
        k, v = shared
    o = sink_attention(q, k, v, m["scale"], w[p + "sink"].to(F), m.get("softcap"))
    return o.reshape(T, -1) @ w[p + "o"].to(F).T, (k, v)


def left_attention(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    T, H, G, dk, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_quotient(h @ w[p + "q"].to(F).T, eps) * w[p + "q.norm"].to(F)      # over the whole row, before the heads are split
    k = rms_quotient(h @ w[p + "k"].to(F).T, eps) * w[p + "k.norm"].to(F)
    v = h @ w[p + "v"].to(F).T
    o = sink_attention(q.view(T, H, dk), k.view(T, G, dk), v.view(T, G, dv), m["scale"], w[p + "sink"].to(F))
    return head_gate(o, w[p + "g"], h).reshape(T, -1) @ w[p + "o"].to(F).T


def decayed_state(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """q, k [T, H, dk], v [T, H, dv]; per head S = d S + k_t v_t^T from zero, o_t = S^T q_t."""
    T, H, dk = q.shape
    out = torch.zeros((T, H, v.shape[-1]), dtype=F)
    for h in range(H):
        S = torch.zeros((dk, v.shape[-1]), dtype=F)
        for t in range(T):
            S = float(decay[h]) * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def right_lightning(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    T, H, dk, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].to(F).T).view(T, H, dk)
    k = silu(h @ w[p + "k"].to(F).T).view(T, H, dk)
    v = silu(h @ w[p + "v"].to(F).T).view(T, H, dv)
    o = decayed_state(q, k, v, m["decay"]).reshape(T, H * dv)
    o = rms_quotient(o, eps) * w[p + "norm"].to(F) * torch.sigmoid(h @ w[p + "g"].to(F).T)
    return o @ w[p + "o"].to(F).T


def mixer_parallel(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    return (m["left_scale"] * left_attention(m["left"], w, p + "left.", h, eps)
            + m["right_scale"] * right_lightning(m["right"], w, p + "right.", h, eps))


# ---------------------------------------------------------------------------------------- feed-forward
def dense_ff(mlp: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    L = float(mlp["limit"])
    g = torch.clamp(h @ w[p + "gate"].to(F).T, max=L)
    u = torch.clamp(h @ w[p + "up"].to(F).T, -L, L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].to(F).T


def route(z: torch.Tensor, correction: torch.Tensor, top: int):
    """z [T, N] router outputs -> (chosen [T, top], their weights [T, top]): softmax over all, choice by s + correction
    (ties: the smaller index), weights s without it and not renormalised."""
    s = torch.softmax(z, -1)
    chosen = []
    for t in range(z.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(s[t, e] + correction[e]), e))
        chosen.append(order[:top])
    chosen = torch.tensor(chosen)
    return chosen, torch.gather(s, 1, chosen)


def routed_ff(mlp: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, router_input: Optional[torch.Tensor] = None) -> torch.Tensor:
    E, I, top = mlp["router"]["experts"], int(mlp["router"].get("identity", 0)), mlp["router"]["top"]
    z = (h if router_input is None else router_input) @ w[p + "router"].to(F).T
    chosen, weights = route(z, w[p + "correction"].to(F), top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            if e >= E:
                y = h[t]
            else:
                y = (silu(h[t] @ w[f"{p}e{e}.gate"].to(F).T) * (h[t] @ w[f"{p}e{e}.up"].to(F).T)) @ w[f"{p}e{e}.down"].to(F).T
            out[t] += weights[t, j] * y
    return out


# ---------------------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; `streams` (a list) receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(cfg, w, tokens)
    kv = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = stream_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = mixer_attention(m, w, p + "mix.", h)
        elif layer["type"] == "parallel":
            y = mixer_parallel(m, w, p + "mix.", h, eps)
        elif layer["type"] == "attention_2":
            y, kv[i] = mixer_attention_2(m, w, p + "mix.", h, eps, kv[m["kv_from"]] if m.get("kv_from") is not None else None)
        else:
            raise ValueError(layer["type"])
        x = x + stream_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = stream_norm(x, w[p + "norm2"], eps)
            y = dense_ff(mlp, w, p + "mlp.", h) if mlp["kind"] == "dense" else routed_ff(mlp, w, p + "mlp.", h)
            x = x + stream_norm(y, w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    z = stream_norm(x, w["final.norm"], eps) @ w["head"].to(F).T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z

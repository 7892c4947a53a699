"""A plain, slow implementation of the Zuzelorn decoder, for comparison.

Whole sequences, no cache, one function per mechanism, float32 on the CPU.  It
shares no code with ``janas_b200``: the configuration is a dictionary as
``config.json`` holds it, the weights a dictionary name -> float32 tensor.

The design, in this file's notation.  x is the residual stream [T, W].

    x_t      = E[token_t] + P[t]
    layer:     h = dyt1(x);  x = x + dyt1b(mixer(h) * sigmoid(R1 h + r1))
               h = dyt2(x);  x = x + dyt2b(ff(h)    * sigmoid(R2 h + r2))    (if the layer has a ff)
    dyt(v)   = tanh(alpha v) * w + b                      (no mean, no variance)
    mixer:     q = Wq h + bq, k = Wk h + bk, v = Wv h + bv; head a reads KV head a // (H // G)
               s_ij = (q_i . k_j) * scale * temp_a   for j <= i
               p_ij = exp(s_ij) / (exp(sink_a) + sum_j' exp(s_ij'))
               out  = Wo concat_a(sum_j p_ij v_j) + bo
               a layer with kv_from = j takes k and v as layer j made them
    ff:        Wd polynorm(Wu h),  polynorm(z) = c0 n(z) + c1 n(z^2) + c2 n(z^3) + c3,
               n(u) = u / sqrt(mean(u^2) + eps) over the ff values of one token
    logits   = (H dyt_final(x)) * logit_scale

``rounding="bfloat16"`` rounds activations where a bfloat16 engine stores them
(norm outputs, q/k/v, the attention output, the activated ff); sums stay float32.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def _round(x: torch.Tensor, rounding: Optional[str]) -> torch.Tensor:
    if rounding is None:
        return x
    assert rounding == "bfloat16"
    return x.to(torch.bfloat16).to(torch.float32)


def embed(table: torch.Tensor, pos_table: torch.Tensor, tokens: Sequence[int], pos0: int = 0) -> torch.Tensor:
    t = torch.tensor(list(tokens), dtype=torch.long)
    p = torch.arange(pos0, pos0 + len(tokens), dtype=torch.long)
    return table[t] + pos_table[p]


def dynamic_tanh(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    return torch.tanh(alpha.reshape(()) * x) * w + b


def gate(h: torch.Tensor, W: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.sigmoid(h @ W.T + b)


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, temp: torch.Tensor,
                   sink: torch.Tensor, pos0: int = 0, window: int = 0) -> torch.Tensor:
    """q [T, H, D], k [S, G, D], v [S, G, Dv]; row i of q sits at position pos0 + i and sees
    keys 0 .. pos0 + i (with a window w, only the last w of them).  Returns [T, H, Dv]."""
    T, H, D = q.shape
    S, G, Dv = v.shape
    out = torch.zeros(T, H, Dv)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a, :] @ k[:, g, :].T) * scale * temp[a]                      # [T, S]
        i = torch.arange(T).unsqueeze(1) + pos0
        j = torch.arange(S).unsqueeze(0)
        s = s.masked_fill(j > i, -math.inf)
        if window > 0:
            s = s.masked_fill(j < i + 1 - window, -math.inf)
        m = torch.maximum(s.max(dim=1, keepdim=True).values, sink[a].reshape(1, 1))
        e = torch.exp(s - m)
        den = e.sum(dim=1, keepdim=True) + torch.exp(sink[a] - m)
        out[:, a, :] = (e / den) @ v[:, g, :]
    return out


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    def n(u):
        return u / torch.sqrt((u * u).mean(dim=-1, keepdim=True) + eps)
    return coef[0] * n(z) + coef[1] * n(z * z) + coef[2] * n(z * z * z) + coef[3]


def attention_mixer(w: Dict[str, torch.Tensor], p: str, m: Dict, h: torch.Tensor, kv, rounding) -> tuple:
    """Returns (output [T, W], (k, v)); kv: another layer's (k, v) to read, or None."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _round(h @ w[p + ".q"].T + w[p + ".q.b"], rounding).reshape(T, H, D)
    if kv is None:
        k = _round(h @ w[p + ".k"].T + w[p + ".k.b"], rounding).reshape(T, G, D)
        v = _round(h @ w[p + ".v"].T + w[p + ".v.b"], rounding).reshape(T, G, Dv)
        kv = (k, v)
    o = sink_attention(q, kv[0], kv[1], float(m["scale"]), w[p + ".temp"], w[p + ".sink"])
    o = _round(o, rounding).reshape(T, H * Dv)
    return o @ w[p + ".o"].T + w[p + ".o.b"], kv


def feed_forward(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float, rounding) -> torch.Tensor:
    z = h @ w[p + ".up"].T
    return _round(polynorm(z, w[p + ".act"], eps), rounding) @ w[p + ".down"].T


def forward(c: Dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], rounding: Optional[str] = None,
            trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence; with ``trace`` the residual stream after every layer."""
    eps = float(c["norm"]["eps"])

    def norm(x, name):
        return dynamic_tanh(x, w[name], w[name + ".b"], w[name + ".alpha"])

    x = embed(w["embed"], w["pos"], tokens)
    made = {}
    for i, layer in enumerate(c["layers"]):
        assert layer["type"] == "attention"
        L = f"l{i}"
        m = layer["mixer"]
        h = _round(norm(x, L + ".norm1"), rounding)
        src = m.get("kv_from")
        y, made[i] = attention_mixer(w, L + ".mix", m, h, made[src] if src is not None else None, rounding)
        x = x + norm(y * gate(h, w[L + ".rg1"], w[L + ".rg1.b"]), L + ".norm1b")
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            h = _round(norm(x, L + ".norm2"), rounding)
            y = feed_forward(w, L + ".mlp", h, eps, rounding)
            x = x + norm(y * gate(h, w[L + ".rg2"], w[L + ".rg2.b"]), L + ".norm2b")
        if trace is not None:
            trace.append(x.clone())
    h = _round(norm(x, "final.norm"), rounding)
    return (h @ w["head"].T) * float(c["logit_scale"])

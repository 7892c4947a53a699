"""A plain, slow implementation of the Dunavik decoder, for comparison.

Whole sequences, no cache, one function per mechanism, float32 on the CPU.  It
shares no code with ``janas_b200``: the configuration is a dictionary as
``config.json`` holds it, the weights a dictionary name -> float32 tensor.

The design, in this file's notation.  x is the residual stream [T, W].

    e        = LN_embed(E[token])                      layer norm with weight and bias
    x        = e
    run:       layers 0 .. start-1 once, layers start .. stop-1 `times` times (every pass a
               cache of its own; before every pass but the first x = x + e), the rest once
    layer:     h = LN_1(x);  x = x + m * (mixer(h) + ff(h))       (ff(h) = 0 for a layer without one)
    LN(v)    = (v - mean v) / sqrt(var v + eps) * w + b

    mixer "latent_attention" (H heads; per head D plain and R rotated key dims, Dv value dims):
               cq = rms(Wdq h) * wq;  q = Wuq cq, per head [D plain | R rotated]
               z  = Wdkv h;  c = rms(z[:C]) * wc;  kr = z[C:]          (one rotated key for all heads)
               rotate(q_rot, p), rotate(kr, p): pairs (2i, 2i+1) by the angle p * base^(-2i/R)
               s_ij = (q_plain_i . (Wuk c_j)_head + q_rot_i . kr_j) * scale,  j <= i, softmax
               out  = Wo (concat_heads(sum_j p_ij (Wuv c_j)_head) * sigmoid(Wg h))

    mixer "attention" (H heads, G key/value heads, head a reads a // (H / G)):
               q_i = (Wq h_i) * (1 + coef * ln(floor((i + 1) / every) + 1))
               s_ij = cap * tanh((q_i . k_j) * scale / cap) - 2^(-8 (a + 1) / H) * (i - j)
               for 0 <= i - j < window, softmax;  out = Wo concat_heads(sum_j p_ij v_j)

    ff:        Wd relu(Wu h)^2
    logits   = Head LN_final(x)

rms(u) = u / sqrt(mean(u^2) + eps).
``rounding="bfloat16"`` rounds activations where a bfloat16 engine stores them.
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


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w + b


def rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, ..., >= dims]: the first `dims` values of the last axis are rotated pair by pair
    (2i, 2i+1) by pos * base^(-2i/dims); the rest pass unchanged."""
    out = x.clone()
    shape = [x.shape[0]] + [1] * (x.dim() - 2)
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        a = pos.to(torch.float32) * torch.tensor(f, dtype=torch.float32)      # the angle is a float32
        c = torch.cos(a.to(torch.float64)).to(torch.float32).reshape(shape)
        s = torch.sin(a.to(torch.float64)).to(torch.float32).reshape(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def softmax_rows(s: torch.Tensor) -> torch.Tensor:
    m = s.max(dim=1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(dim=1, keepdim=True)


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, pos0: int = 0,
                   window: int = 0, cap: float = 0.0, slope_exponent: Optional[float] = None) -> torch.Tensor:
    """q [T, H, D] at positions pos0 .. pos0 + T - 1; k [S, G, D], v [S, G, Dv] at positions
    0 .. S - 1.  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    S, G, Dv = v.shape
    i = torch.arange(T).unsqueeze(1) + pos0
    j = torch.arange(S).unsqueeze(0)
    out = torch.zeros(T, H, Dv)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if slope_exponent is not None:
            s = s - 2.0 ** (-slope_exponent * (a + 1) / H) * (i - j).to(torch.float32)
        s = s.masked_fill(j > i, -math.inf)
        if window:
            s = s.masked_fill(i - j >= window, -math.inf)
        out[:, a] = softmax_rows(s) @ v[:, g]
    return out


def latent_core(q_plain: torch.Tensor, q_rot: torch.Tensor, c: torch.Tensor, kr: torch.Tensor,
                w_uk: torch.Tensor, w_uv: torch.Tensor, scale: float, pos0: int = 0) -> torch.Tensor:
    """q_plain [T, H, D], q_rot [T, H, R] (rotated already) at positions pos0 ..; c [S, C] latents
    and kr [S, R] rotated shared key parts at positions 0 .. S - 1; w_uk [H D, C], w_uv [H Dv, C].
    Keys and values per head are formed here, plainly.  Returns [T, H, Dv]."""
    T, H, D = q_plain.shape
    S = c.shape[0]
    Dv = w_uv.shape[0] // H
    k_plain = (c @ w_uk.T).reshape(S, H, D)
    v = (c @ w_uv.T).reshape(S, H, Dv)
    i = torch.arange(T).unsqueeze(1) + pos0
    j = torch.arange(S).unsqueeze(0)
    out = torch.zeros(T, H, Dv)
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ kr.T) * scale
        s = s.masked_fill(j > i, -math.inf)
        out[:, a] = softmax_rows(s) @ v[:, a]
    return out


def query_temperature(pos: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    return 1.0 + coef * torch.log(torch.floor((pos + 1).to(torch.float32) / every) + 1.0)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float,
                     rounding: Optional[str] = None) -> torch.Tensor:
    """h [T, W] at positions 0 .. T-1 -> the mixer's output [T, W]."""
    T = h.shape[0]
    H, D, R, Dv, C = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    pos = torch.arange(T)
    cq = _round(rms(h @ w[p + "dq"].T, w[p + "dq.norm"], eps), rounding)
    q = (cq @ w[p + "uq"].T).reshape(T, H, D + R)
    z = h @ w[p + "dkv"].T
    c = _round(rms(z[:, :C], w[p + "dkv.norm"], eps), rounding)
    kr = _round(rotate_pairs(z[:, C:], pos, mx["rot"]["base"], mx["rot"]["dims"]), rounding)
    q_plain = _round(q[:, :, :D], rounding)
    q_rot = _round(rotate_pairs(q[:, :, D:], pos, mx["rot"]["base"], mx["rot"]["dims"]), rounding)
    out = latent_core(q_plain, q_rot, c, kr, w[p + "uk"], w[p + "uv"], mx["scale"])
    g = torch.sigmoid(h @ w[p + "g"].T)
    return _round(out.reshape(T, H * Dv) * g, rounding) @ w[p + "o"].T


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict,
                     rounding: Optional[str] = None) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    qt = mx.get("q_temp")
    if qt:
        q = q * query_temperature(torch.arange(T), qt["coef"], qt["every"]).reshape(T, 1, 1)
    q = _round(q, rounding)
    k = _round((h @ w[p + "k"].T).reshape(T, G, D), rounding)
    v = _round((h @ w[p + "v"].T).reshape(T, G, Dv), rounding)
    out = attention_core(q, k, v, mx["scale"], 0, (mx.get("mask") or {}).get("size", 0),
                         mx.get("softcap") or 0.0, 8.0)
    return _round(out.reshape(T, H * Dv), rounding) @ w[p + "o"].T


def relu2_ff(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, rounding: Optional[str] = None) -> torch.Tensor:
    z = torch.relu(h @ up.T)
    return _round(z * z, rounding) @ down.T


def run_order(config: dict) -> List[int]:
    n = len(config["layers"])
    lp = config.get("loop")
    if not lp:
        return list(range(n))
    a, b, times = lp["start"], lp["stop"], lp["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], rounding: Optional[str] = None,
            trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; with `trace`, x after every layer run is appended."""
    eps = config["norm"]["eps"]
    m = config["residual_mult"]
    t = torch.tensor(list(tokens), dtype=torch.long)
    e = layer_norm(w["embed"][t], w["embed.norm"], w["embed.norm.b"], eps)
    x = e.clone()
    lp = config.get("loop")
    order = run_order(config)
    seen_first = False
    for at, li in enumerate(order):
        if lp and li == lp["start"] and lp["stop"] > lp["start"]:
            if seen_first:
                x = x + e
            seen_first = True
        L = config["layers"][li]
        p = "l%d." % li
        h = _round(layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps), rounding)
        if L["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", L["mixer"], eps, rounding)
        elif L["type"] == "attention":
            y = window_attention(h, w, p + "mix.", L["mixer"], rounding)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            assert L["mlp"]["kind"] == "dense"
            y = y + relu2_ff(h, w[p + "mlp.up"], w[p + "mlp.down"], rounding)
        x = x + m * y
        if trace is not None:
            trace.append(x.clone())
    hf = _round(layer_norm(x, w["final.norm"], w["final.norm.b"], eps), rounding)
    return hf @ w["head"].T

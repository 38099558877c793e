"""Plain implementation of the Kinanex design: float64, whole sequences, no cache, one function per mechanism.

It shares no code with the product path (`qspec_b200/kinanex.py` and its kernels) and is the reference of the tests.
`cfg` is the dictionary of a config.json, `w` maps tensor names to torch tensors (any float type; read as float64).

    start:      x = N(embed[token]; embed.norm)                                       N(v; g) = v / sqrt(mean(v^2) + eps) * g
    layer:      x <- x + ls1 * mixer(N(x; norm1));   x <- x + ls2 * ff(N(x; norm2))   (ls: one factor per column)
    attention:  q, k, v with biases; q, k <- N(per head; shared weight), rotated; v <- unit_rms per head, blended with the first
                blending layer's v; p_g = softmax over the causal keys and one extra logit 0; P_h = sum_g talk[h, g] p_g;
                head h = P_h applied to the values of its key/value head; W_o
    delta:      q, k, v = silu(conv(W h)); q, k unit vectors (q / sqrt(dim)); S <- g S; u = beta (v - S^T k); S <- S + k u^T;
                o = S^T q; W_o (N(o per head; norm) * silu(W_g h))
    mamba1:     [x | z] = W_in h; x = silu(conv(x) + b); [dt | B | C] = W_x x; dt = softplus(W_dt dt + b_dt);
                S <- exp(-dt exp(A_log)) S + dt x B^T; y = S C + D x; W_o (y * silu(z))
    ff:         g = min(W_gate h, limit); u = clamp(W_up h, +-limit); W_down (g sigmoid(1.702 g) (u + 1))
    end:        logits = logit_scale * embed N(x; final.norm)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def _t(w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return w[name].to(F64)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x: torch.Tensor, taps_w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], taps_w [C, K]: y_t = bias + sum_j taps_w[:, j] * x_(t - K + 1 + j), zeros before the start."""
    T, C = x.shape
    K = taps_w.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(K):
            s = t - (K - 1) + j
            if s >= 0:
                y[t] += taps_w[:, j] * x[s]
    return y if bias is None else y + bias


def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]) -> List[float]:
    """One frequency per rotated pair; long wavelengths are slowed down by `factor`, short ones kept, a linear ramp between."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            wl = 2.0 * math.pi / f
            short, long_ = scaling["original"] / scaling["high"], scaling["original"] / scaling["low"]
            if wl > long_:
                f = f / scaling["factor"]
            elif wl >= short:
                s = (scaling["original"] / wl - scaling["low"]) / (scaling["high"] - scaling["low"])
                f = (1.0 - s) * f / scaling["factor"] + s * f
        out.append(f)
    return out


def rotate_halves(x: torch.Tensor, pos: torch.Tensor, freqs: List[float]) -> torch.Tensor:
    """x [T, heads, n]: entry i and entry i + len(freqs) turn by pos * freqs[i]; entries from 2 len(freqs) on pass."""
    out = x.clone()
    half = len(freqs)
    for i, f in enumerate(freqs):
        a = pos.to(F64) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def sink_softmax_rows(scores: torch.Tensor) -> torch.Tensor:
    """scores [n]: exp(s_j) / (1 + sum exp(s_j))."""
    m = max(float(scores.max()), 0.0)
    e = torch.exp(scores - m)
    return e / (math.exp(-m) + e.sum())


def talking_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, talk: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, DV]. Every head's causal weights with the extra unit in the denominator; the weights of
    all heads are mixed by talk [H, H]; head h applies its mixed weights to the values of key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        p = torch.stack([sink_softmax_rows((k[:t + 1, h // rep] @ q[t, h]) * scale) for h in range(H)])      # [H, t + 1]
        mixed = talk @ p
        for h in range(H):
            out[t, h] = mixed[h] @ v[:t + 1, h // rep]
    return out


def attention_values(h: torch.Tensor, w, p: str, m: dict, eps: float, ctx: dict) -> torch.Tensor:
    """Values of an attention layer as they are kept: [T, G, DV], normed, blended if the layer is a later blending layer."""
    T = h.shape[0]
    v = (h @ _t(w, p + "v").T + _t(w, p + "v.b")).view(T, m["kv_heads"], m["vdim"])
    v = unit_rms(v, eps)
    if m.get("v_mix"):
        if "first" in ctx:
            lam = _t(w, p + "vmix")
            v = (1.0 - lam) * v + lam * ctx["first"]
        else:
            ctx["first"] = v
    return v


def attention_mixer(h: torch.Tensor, w, p: str, m: dict, eps: float, ctx: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    q = (h @ _t(w, p + "q").T + _t(w, p + "q.b")).view(T, H, D)
    k = (h @ _t(w, p + "k").T + _t(w, p + "k.b")).view(T, G, D)
    q = unit_rms(q, eps) * _t(w, p + "q.norm")
    k = unit_rms(k, eps) * _t(w, p + "k.norm")
    rot = m.get("rot") or {}
    if rot.get("dims"):
        fr = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_halves(q, pos, fr), rotate_halves(k, pos, fr)
    v = attention_values(h, w, p, m, eps, ctx)
    o = talking_attention(q, k, v, _t(w, p + "talk"), m["scale"])
    return o.reshape(T, -1) @ _t(w, p + "o").T


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, g: torch.Tensor,
               state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q, k [T, G, D] (already unit vectors), v [T, H, DV], beta, g [T, H]: per head the state decays, is corrected towards v
    along k, and is read with q after the write. Returns o [T, H, DV]; `state` [H, D, DV], if given, is updated in place."""
    T, H, DV = v.shape
    G, D = k.shape[1], k.shape[2]
    rep = H // G
    S = torch.zeros(H, D, DV, dtype=F64) if state is None else state
    o = torch.zeros(T, H, DV, dtype=F64)
    for t in range(T):
        for h in range(H):
            kk, qq = k[t, h // rep], q[t, h // rep]
            S[h] = g[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ kk)
            S[h] = S[h] + torch.outer(kk, u)
            o[t, h] = S[h].T @ qq
    return o


def delta_mixer(h: torch.Tensor, w, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ _t(w, p + "q").T, _t(w, p + "q.conv"))).view(T, G, D)
    k = silu(causal_conv(h @ _t(w, p + "k").T, _t(w, p + "k.conv"))).view(T, G, D)
    v = silu(causal_conv(h @ _t(w, p + "v").T, _t(w, p + "v.conv"))).view(T, H, DV)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(D)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ _t(w, p + "b").T)
    g = torch.exp(-torch.exp(_t(w, p + "A_log")) * softplus(h @ _t(w, p + "a").T + _t(w, p + "dt_bias")))
    o = delta_rule(q, k, v, beta, g)
    o = unit_rms(o, eps) * _t(w, p + "norm") * silu(h @ _t(w, p + "g").T).view(T, H, DV)
    return o.reshape(T, H * DV) @ _t(w, p + "o").T


def selective_scan(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, D: torch.Tensor) -> torch.Tensor:
    """x, dt [T, I], A [I, N], B, C [T, N], D [I]: S <- exp(dt A) S + dt x B^T; y = S C + D x."""
    T, I = x.shape
    S = torch.zeros(I, A.shape[1], dtype=F64)
    y = torch.zeros(T, I, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y


def mamba_mixer(h: torch.Tensor, w, p: str, m: dict) -> torch.Tensor:
    I, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ _t(w, p + "in").T
    x, z = xz[:, :I], xz[:, I:]
    x = silu(causal_conv(x, _t(w, p + "conv"), _t(w, p + "conv.b")))
    dbc = x @ _t(w, p + "x").T
    dt = softplus(dbc[:, :R] @ _t(w, p + "dt").T + _t(w, p + "dt.b"))
    y = selective_scan(x, dt, -torch.exp(_t(w, p + "A_log")), dbc[:, R:R + N], dbc[:, R + N:], _t(w, p + "D"))
    return (y * silu(z)) @ _t(w, p + "o").T


def clamped_glu(h: torch.Tensor, w, p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ _t(w, p + "gate").T, max=limit)
    u = torch.clamp(h @ _t(w, p + "up").T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _t(w, p + "down").T


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence; layers_out, if a list, receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = unit_rms(_t(w, "embed")[torch.as_tensor(tokens, dtype=torch.long)], eps) * _t(w, "embed.norm")
    ctx: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = unit_rms(x, eps) * _t(w, p + "norm1")
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", m, eps, ctx)
        elif layer["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "mamba1":
            y = mamba_mixer(h, w, p + "mix.", m)
        else:
            raise ValueError(layer["type"])
        x = x + _t(w, p + "ls1") * y
        if layer.get("mlp") is not None:
            x = x + _t(w, p + "ls2") * clamped_glu(unit_rms(x, eps) * _t(w, p + "norm2"), w, p + "mlp.", layer["mlp"]["limit"])
        if layers_out is not None:
            layers_out.append(x.clone())
    x = unit_rms(x, eps) * _t(w, "final.norm")
    return x @ _t(w, "embed").T * cfg.get("logit_scale", 1.0)

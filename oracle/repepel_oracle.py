"""Plain implementation of the Repepel design: float64, whole sequences, no cache, one function per mechanism.

It shares no code with the product path (`qspec_b200/repepel.py` and its kernels) and is the reference of the tests.
`cfg` is the dictionary of a config.json, `w` maps tensor names to torch tensors (any float type; read as float64).

    layer:      x <- x + m * mixer(N(x; norm1));   x <- x + m * ff(N(x; norm2))        N(v; g) = v / sqrt(mean(v^2) + eps) * (1 + g)
    loop:       layers start .. stop-1 run `times` times in a row (same weights, separate state), then the rest
    lightning:  q, k, v = silu(W h);  S_t = a_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;  out = W_o (rms(o over all heads) * g_n * sigmoid(W_g h))
    latent:     q = W_q h = per head [plain | rotary];  W_dkv h = [c' | r'];  c = rms(c') * g_c;  key_h = [W_uk c | rot(r')],  value_h = W_uv c
                causal softmax of scale * q.k;  head output * sigmoid(W_g h)_head;  out = W_o (heads)
    dense ff:   W_down gelu(W_up h)          (erf form)
    moe ff:     s = sigmoid(W_r h);  choice = s + correction, limited to the best groups;  sum over the top choices of
                scale * s_e * expert_e(h)  +  sigmoid(W_sg h) * shared(h);   expert(h) = W_down (silu(W_gate h) * W_up h)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def _t(w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return w[name].to(F64)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_centered(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + g)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotate_interleaved(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, ..., n]: entries (2i, 2i+1), i < dims/2, turn by pos * base^(-2i/dims); the rest pass."""
    out = x.clone()
    shape = [x.shape[0]] + [1] * (x.dim() - 2)
    for i in range(dims // 2):
        a = pos.to(F64) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay) -> torch.Tensor:
    """q, k [T, H, D], v [T, H, DV]: per head S_t = decay_h S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t."""
    T, H, D = q.shape
    o = torch.zeros(T, H, v.shape[2], dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, v.shape[2], dtype=F64)
        a = float(decay[hd])
        for t in range(T):
            S = a * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    return o


def lightning_mixer(h: torch.Tensor, w, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ _t(w, p + "q").T).view(T, H, D)
    k = silu(h @ _t(w, p + "k").T).view(T, H, D)
    v = silu(h @ _t(w, p + "v").T).view(T, H, DV)
    o = linear_attention(q, k, v, m["decay"])
    o = unit_rms(o.reshape(T, H * DV), eps) * _t(w, p + "norm")
    o = o * torch.sigmoid(h @ _t(w, p + "g").T)
    return o @ _t(w, p + "o").T


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q, k [T, H, DK], v [T, H, DV]: position i sees every j <= i; ordinary softmax of scale * q.k."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * float(scale)
    s = s.masked_fill(~torch.ones(T, T).tril().bool(), float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v)


def latent_mixer(h: torch.Tensor, w, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, DV, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims", R)), float(rot.get("base", 10000.0))
    pos = torch.arange(T)
    q = (h @ _t(w, p + "q").T).view(T, H, D + R)
    q = torch.cat([q[..., :D], rotate_interleaved(q[..., D:], pos, dims, base)], -1)
    d = h @ _t(w, p + "dkv").T
    c = unit_rms(d[:, :r], eps) * _t(w, p + "dkv.norm")
    k_rot = rotate_interleaved(d[:, r:], pos, dims, base)                       # [T, R], one part shared by the heads
    k = torch.cat([(c @ _t(w, p + "uk").T).view(T, H, D), k_rot.unsqueeze(1).expand(T, H, R)], -1)
    val = (c @ _t(w, p + "uv").T).view(T, H, DV)
    o = causal_attention(q, k, val, m["scale"])
    o = o * torch.sigmoid(h @ _t(w, p + "g").T).unsqueeze(-1)                   # one gate per head
    return o.reshape(T, H * DV) @ _t(w, p + "o").T


def gated_expert(h: torch.Tensor, w, p: str) -> torch.Tensor:
    return (silu(h @ _t(w, p + "gate").T) * (h @ _t(w, p + "up").T)) @ _t(w, p + "down").T


def choose_experts(s: torch.Tensor, correction: torch.Tensor, top: int, count: int, keep: int, scale: float):
    """s [T, E] scores. Returns idx [T, top] (descending choice score, lowest index among equals) and weights [T, top]."""
    T, E = s.shape
    choice = s + correction
    size = E // count
    idx = torch.zeros(T, top, dtype=torch.long)
    wt = torch.zeros(T, top, dtype=F64)
    for t in range(T):
        ch = choice[t].clone()
        if count > 1:
            gs = [sum(sorted(ch[gi * size:(gi + 1) * size].tolist(), reverse=True)[:2]) for gi in range(count)]
            best = sorted(range(count), key=lambda gi: (-gs[gi], gi))[:keep]
            for gi in range(count):
                if gi not in best:
                    ch[gi * size:(gi + 1) * size] = float("-inf")
        for k in range(top):
            e = max(range(E), key=lambda j: (ch[j].item(), -j))
            idx[t, k] = e
            wt[t, k] = s[t, e] * float(scale)
            ch[e] = float("-inf")
    return idx, wt


def route(h: torch.Tensor, w, p: str, r: dict) -> Tuple[torch.Tensor, torch.Tensor]:
    g = r.get("groups") or {}
    count = int(g.get("count", 1))
    s = torch.sigmoid(h @ _t(w, p + "router").T)
    return choose_experts(s, _t(w, p + "correction"), r["top"], count, int(g.get("keep", count)), r.get("scale", 1.0))


def moe_ff(h: torch.Tensor, w, p: str, f: dict) -> torch.Tensor:
    idx, wt = route(h, w, p, f["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            out[t] += wt[t, k] * gated_expert(h[t:t + 1], w, p + f"e{int(idx[t, k])}.")[0]
    if f.get("shared"):
        out = out + torch.sigmoid(h @ _t(w, p + "shared.sg").T) * gated_expert(h, w, p + "shared.")
    return out


def dense_ff(h: torch.Tensor, w, p: str) -> torch.Tensor:
    return gelu_erf(h @ _t(w, p + "up").T) @ _t(w, p + "down").T


def layer_runs(cfg: dict) -> List[int]:
    """Indices of the layers in the order they run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; `trace` receives the residual stream after every layer run."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = _t(w, "embed")[torch.as_tensor(tokens, dtype=torch.long)]
    for i in layer_runs(cfg):
        spec, p = cfg["layers"][i], f"l{i}."
        h = norm_centered(x, _t(w, p + "norm1"), eps)
        if spec["type"] == "lightning":
            y = lightning_mixer(h, w, p + "mix.", spec["mixer"], eps)
        elif spec["type"] == "latent_attention":
            y = latent_mixer(h, w, p + "mix.", spec["mixer"], eps)
        else:
            raise ValueError(spec["type"])
        x = x + mult * y
        f = spec.get("mlp")
        if f is not None:
            h = norm_centered(x, _t(w, p + "norm2"), eps)
            y = moe_ff(h, w, p + "mlp.", f) if f["kind"] == "moe" else dense_ff(h, w, p + "mlp.")
            x = x + mult * y
        if trace is not None:
            trace.append(x.clone())
    x = norm_centered(x, _t(w, "final.norm"), eps)
    return x @ _t(w, "head").T


def greedy(cfg: dict, w, prompt, n_new: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        t = int(forward(cfg, w, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out

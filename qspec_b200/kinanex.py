"""Kinanex: a pre-norm decoder with a layer scale on every sublayer that mixes three kinds of sequence mixers -- grouped-query
attention whose heads talk to one another after the softmax, the gated delta rule, and the selective scan -- with a clamped
gated feed-forward layer.

With x the float32 residual stream and N(v; w) = v / sqrt(mean(v^2) + eps) * w:

    x = N(embed[token]; embed.norm)
    x <- x + ls1 * mixer(N(x; norm1));      x <- x + ls2 * ff(N(x; norm2))        (a layer may have no feed-forward)
    logits = logit_scale * embed N(x; final.norm)                                  (the embedding table is the output matrix)

mixers (`layers[i].type`):
    attention   q, k, v with biases; q and k normed per head (N over `dim` with a shared weight), then the first `rot.dims`
                entries of every head rotated (entry i with i + dims/2, angle = position * f_i, the frequencies stretched per
                wavelength band as `rot.scaling` says); v normed per head without a weight and, in every `v_mix` layer after the
                first, blended with the first such layer's values of the same token. Causal over the whole sequence; the
                softmax denominator carries one extra term exp(0). The finished weights of all heads are mixed by `talk`
                [H, H] before each head applies them to the values of its own key/value head.
    delta       q, k (kv_heads x dim) and v (heads x vdim) through a short causal convolution and silu; q, k unit vectors per
                head (q times dim^-1/2); per head S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q with
                beta = sigmoid(W_b h), g = exp(-exp(A_log) softplus(W_a h + dt_bias)); o normed per head, times silu(W_g h).
    mamba1      [x | z] = W_in h; x through a convolution with bias and silu; [dt | B | C] = W_x x; dt = softplus(W_dt dt + b);
                S <- exp(-dt exp(A_log)) S + dt x B, y = S C + D x; y * silu(z).
feed-forward (`mlp.kind` = dense): g = min(W_gate h, limit), u = clamp(W_up h, +-limit); W_down (g sigmoid(1.702 g) (u + 1)).

Wiring follows `repepel.RepepelModel`: a flat token batch with per-token slot and position (`state.BatchMeta`), state held by
the model and indexed by slot, a scratch arena allocated once, dense products in the vendor library, everything else in the
sequence-mixer kernel library (`ops.seq_*`). Every residual sum is fused with the layer scale and with the norm that follows it
(`ops.seq_residual_norm`). Per-slot state: key / value rows of every attention layer (row = position), the float32 matrices of
the delta and scan layers, and the last `conv - 1` inputs of every convolution (double-buffered by the step's phase). Nothing
is cleared when a slot is released: cache rows are valid by position, and the recurrences start from zero at position 0.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import ops
from .state import BatchMeta

GLU_ALPHA = 1.702                   # the gate's sigmoid slope of the feed-forward activation
UNIT_EPS = 1e-6                     # under the root of the delta rule's unit vectors
FULL_WINDOW = 1 << 30               # the attention sees the whole sequence: a window no sequence reaches


@dataclass
class KinanexMixer:
    kind: str                       # "attention" | "delta" | "mamba1"
    heads: int = 0                  # attention, delta
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 1.0              # attention ...
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: Optional[Dict[str, float]] = None      # factor, low, high, original
    v_mix: bool = False
    conv: int = 1                   # delta, mamba1: taps of the convolution
    inner: int = 0                  # mamba1 ...
    state: int = 0
    dt_rank: int = 0


@dataclass
class KinanexFF:
    ff: int
    limit: float


@dataclass
class KinanexLayer:
    mixer: KinanexMixer
    mlp: Optional[KinanexFF]


def rotary_frequencies(dims: int, base: float, scaling: Optional[Dict[str, float]] = None) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2 (float64). With `scaling` = {factor, low, high, original}: a frequency whose
    wavelength l = 2 pi / f is shorter than original / high stays; one longer than original / low is divided by factor; between
    the two, with s = (original / l - low) / (high - low), it becomes (1 - s) f / factor + s f."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / max(dims, 1))
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wl = 2.0 * math.pi / f
        s = (orig / wl - low) / (high - low)
        f = torch.where(wl < orig / high, f, torch.where(wl > orig / low, f / factor, (1.0 - s) * f / factor + s * f))
    return f


@dataclass
class KinanexConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float = 1.0
    layers: List[KinanexLayer] = field(default_factory=list)
    name: str = "kinanex"

    @staticmethod
    def from_dict(d: dict) -> "KinanexConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            kind, m = e.get("type"), e["mixer"]
            if kind == "attention":
                rot = m.get("rot") or {}
                mixer = KinanexMixer(kind=kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                     vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), rot_dims=int(rot.get("dims", 0)),
                                     rot_base=float(rot.get("base", 10000.0)), rot_scaling=dict(rot["scaling"]) if rot.get("scaling") else None,
                                     v_mix=bool(m.get("v_mix", False)))
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                    raise ValueError(f"layer {i}: {mixer.rot_dims} rotated dimensions of {mixer.dim}")
            elif kind == "delta":
                mixer = KinanexMixer(kind=kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                     vdim=int(m.get("vdim", m["dim"])), conv=int(m["conv"]))
            elif kind == "mamba1":
                mixer = KinanexMixer(kind=kind, conv=int(m["conv"]), inner=int(m["inner"]), state=int(m["state"]), dt_rank=int(m["dt_rank"]))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            if kind != "mamba1" and (mixer.kv_heads < 1 or mixer.heads % mixer.kv_heads):
                raise ValueError(f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key heads")
            if mixer.conv < 1:
                raise ValueError(f"layer {i}: a convolution of {mixer.conv} taps")
            f = e.get("mlp")
            if f is None:
                mlp = None
            elif f.get("kind", "dense") == "dense":
                mlp = KinanexFF(ff=int(f["ff"]), limit=float(f["limit"]))
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            layers.append(KinanexLayer(mixer=mixer, mlp=mlp))
        cfg = KinanexConfig(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                            logit_scale=float(d.get("logit_scale", 1.0)), layers=layers)
        mixed = [l.mixer for l in layers if l.mixer.kind == "attention" and l.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (mixed[0].kv_heads, mixed[0].vdim) for m in mixed):
            raise ValueError("the layers that blend their values must agree in key/value heads and value size")
        return cfg

    def to_dict(self) -> dict:
        out = {"architecture": "Kinanex", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "logit_scale": self.logit_scale, "layers": []}
        for l in self.layers:
            m, f = l.mixer, l.mlp
            if m.kind == "attention":
                rot = {"base": m.rot_base, "dims": m.rot_dims}
                if m.rot_scaling:
                    rot["scaling"] = dict(m.rot_scaling)
                mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "v_mix": m.v_mix, "rot": rot}
            elif m.kind == "delta":
                mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            else:
                mx = {"conv": m.conv, "inner": m.inner, "state": m.state, "dt_rank": m.dt_rank}
            out["layers"].append({"type": m.kind, "mixer": mx,
                                  "mlp": None if f is None else {"kind": "dense", "ff": f.ff, "limit": f.limit}})
        return out

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every tensor a checkpoint of this configuration must hold."""
        W = self.width
        out = {"embed": (self.vocab, W), "embed.norm": (W,)}
        for i, l in enumerate(self.layers):
            m, f, p = l.mixer, l.mlp, f"l{i}."
            out[p + "norm1"] = (W,)
            out[p + "ls1"] = (W,)
            x = p + "mix."
            if m.kind == "attention":
                out.update({x + "q": (m.heads * m.dim, W), x + "q.b": (m.heads * m.dim,), x + "k": (m.kv_heads * m.dim, W),
                            x + "k.b": (m.kv_heads * m.dim,), x + "v": (m.kv_heads * m.vdim, W), x + "v.b": (m.kv_heads * m.vdim,),
                            x + "q.norm": (m.dim,), x + "k.norm": (m.dim,), x + "talk": (m.heads, m.heads),
                            x + "o": (W, m.heads * m.vdim)})
                if m.v_mix:
                    out[x + "vmix"] = ()
            elif m.kind == "delta":
                out.update({x + "q": (m.kv_heads * m.dim, W), x + "q.conv": (m.kv_heads * m.dim, m.conv), x + "k": (m.kv_heads * m.dim, W),
                            x + "k.conv": (m.kv_heads * m.dim, m.conv), x + "v": (m.heads * m.vdim, W),
                            x + "v.conv": (m.heads * m.vdim, m.conv), x + "b": (m.heads, W), x + "a": (m.heads, W),
                            x + "A_log": (m.heads,), x + "dt_bias": (m.heads,), x + "norm": (m.vdim,), x + "g": (m.heads * m.vdim, W),
                            x + "o": (W, m.heads * m.vdim)})
            else:
                out.update({x + "in": (2 * m.inner, W), x + "conv": (m.inner, m.conv), x + "conv.b": (m.inner,),
                            x + "x": (m.dt_rank + 2 * m.state, m.inner), x + "dt": (m.inner, m.dt_rank), x + "dt.b": (m.inner,),
                            x + "A_log": (m.inner, m.state), x + "D": (m.inner,), x + "o": (W, m.inner)})
            if f is not None:
                out.update({p + "norm2": (W,), p + "ls2": (W,), p + "mlp.gate": (f.ff, W), p + "mlp.up": (f.ff, W),
                            p + "mlp.down": (W, f.ff)})
        out["final.norm"] = (W,)
        return out


def random_weights(cfg: KinanexConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bfloat16 tensors of a configuration (CPU): matrices ~ N(0, 1/fan_in), norm weights and layer scales near 1, the
    head mix near the identity, decays and step sizes in the range where the state neither dies nor saturates."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        if name.endswith(".talk"):
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g) / shape[0] ** 0.5
        elif name.endswith("mix.A_log"):
            t = torch.log(0.5 + 3.5 * torch.rand(shape, generator=g)) if len(shape) == 2 else 0.5 * torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif name.endswith(("norm1", "norm2", "mix.norm", "q.norm", "k.norm", "embed.norm", "final.norm", "ls1", "ls2", "mix.D")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("vmix"):
            t = 0.2 + 0.5 * torch.rand(shape, generator=g)
        elif name.endswith(("dt_bias", "dt.b")):
            t = -1.0 + 0.5 * torch.randn(shape, generator=g)
        else:
            t = 0.1 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


class _LayerWeights:
    """Device tensors of one layer: large matrices in the activation type (fused where one product serves several), vectors,
    convolutions and everything a recurrence reads in float32."""

    def __init__(self, cfg: KinanexConfig, i: int, sd: Dict[str, torch.Tensor], dtype, device):
        spec, p = cfg.layers[i], f"l{i}."
        m, f = spec.mixer, spec.mlp

        def big(*names):
            t = torch.cat([sd[p + n] for n in names], 0) if len(names) > 1 else sd[p + names[0]]
            return t.to(device=device, dtype=dtype).contiguous()

        def small(*names):
            t = torch.cat([sd[p + n].to(torch.float32) for n in names], 0) if len(names) > 1 else sd[p + names[0]]
            return t.to(device=device, dtype=torch.float32).contiguous()

        self.norm1, self.ls1 = small("norm1"), small("ls1")
        if m.kind == "attention":
            self.qkv = big("mix.q", "mix.k", "mix.v")                                             # rows [q ; k ; v]
            self.qkv_b = big("mix.q.b", "mix.k.b", "mix.v.b")
            self.q_norm, self.k_norm = small("mix.q.norm"), small("mix.k.norm")
            self.talk = small("mix.talk")
            self.sink = torch.zeros(m.heads, dtype=torch.float32, device=device)                  # the extra term of the denominator: exp(0)
            self.vmix = sd[p + "mix.vmix"].to(device=device, dtype=torch.float32).reshape(1).contiguous() if m.v_mix else None
            self.inv_freq = rotary_frequencies(m.rot_dims, m.rot_base, m.rot_scaling).to(device=device, dtype=torch.float32) \
                if m.rot_dims else None
        elif m.kind == "delta":
            self.qkvg = big("mix.q", "mix.k", "mix.v", "mix.g")                                   # rows [q ; k ; v ; g]
            self.ba = big("mix.b", "mix.a")                                                       # rows [b ; a], float32 results
            self.conv = small("mix.q.conv", "mix.k.conv", "mix.v.conv")
            self.A_log, self.dt_bias, self.o_norm = small("mix.A_log"), small("mix.dt_bias"), small("mix.norm")
        else:
            self.w_in, self.w_x, self.w_dt = big("mix.in"), big("mix.x"), big("mix.dt")
            self.conv, self.conv_b = small("mix.conv"), small("mix.conv.b")
            self.dt_b, self.A_log, self.D = small("mix.dt.b"), small("mix.A_log"), small("mix.D")
        self.o = big("mix.o")
        if f is not None:
            self.norm2, self.ls2 = small("norm2"), small("ls2")
            self.gate_up, self.down = big("mlp.gate", "mlp.up"), big("mlp.down")                  # rows [gate ; up]


class KinanexModel(torch.nn.Module):
    """Weights, per-slot state and the forward pass over a flat token batch (`state.BatchMeta`).

    dtype: torch.bfloat16 (serving: bfloat16 matrix products with float32 accumulation) or torch.float32 (everything in true
    float32). n_slots sequences can be live at once; a step carries at most max_step_tokens tokens; a sequence holds at most
    max_seq_tokens tokens (the attention caches have that many rows per slot and layer)."""

    architecture = "Kinanex"
    DEFAULT_SEQ_TOKENS = 8192

    def __init__(self, cfg: KinanexConfig, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16, device="cuda",
                 n_slots: int = 8, max_step_tokens: int = 2048, max_seq_tokens: Optional[int] = None):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("KinanexModel: dtype must be torch.bfloat16 or torch.float32")
        for name, shape in cfg.tensor_shapes().items():
            if name not in weights:
                raise KeyError(f"tensor {name} is missing from the checkpoint")
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"tensor {name}: shape {tuple(weights[name].shape)}, the configuration says {tuple(shape)}")
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.n_slots, self.max_step_tokens = n_slots, max_step_tokens
        has_attention = any(l.mixer.kind == "attention" for l in cfg.layers)
        self.max_seq_len = max(int(max_seq_tokens or self.DEFAULT_SEQ_TOKENS), 1) if has_attention else None   # checked by the scheduler
        # true float32 products in float32 mode; no reduced-precision accumulation of bfloat16 products
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        dev, W, T = self.device, cfg.width, max_step_tokens
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=dtype, device=dev)
        self.embed = weights["embed"].to(**act).contiguous()
        self.embed_norm = weights["embed.norm"].to(**f32).contiguous()
        self.final_norm = weights["final.norm"].to(**f32).contiguous()
        self.weights = [_LayerWeights(cfg, i, weights, dtype, dev) for i in range(len(cfg.layers))]
        # ---- per-slot state ----
        self.cache_k: Dict[int, torch.Tensor] = {}                                             # layer -> [slots, cap, G, D]
        self.cache_v: Dict[int, torch.Tensor] = {}                                             # layer -> [slots, cap, G, DV]
        self.rec_state: Dict[int, torch.Tensor] = {}                                           # layer -> float32 [slots, H, D, DV] | [slots, inner, N]
        self.conv_tail: Dict[int, torch.Tensor] = {}                                           # layer -> float32 [2, slots, taps - 1, C]
        for i, l in enumerate(cfg.layers):
            m = l.mixer
            if m.kind == "attention":
                self.cache_k[i] = torch.zeros(n_slots, self.max_seq_len, m.kv_heads, m.dim, **act)
                self.cache_v[i] = torch.zeros(n_slots, self.max_seq_len, m.kv_heads, m.vdim, **act)
            elif m.kind == "delta":
                self.rec_state[i] = torch.zeros(n_slots, m.heads, m.dim, m.vdim, **f32)
                self.conv_tail[i] = torch.zeros(2, n_slots, m.conv - 1, 2 * m.kv_heads * m.dim + m.heads * m.vdim, **f32)
            else:
                self.rec_state[i] = torch.zeros(n_slots, m.inner, m.state, **f32)
                self.conv_tail[i] = torch.zeros(2, n_slots, m.conv - 1, m.inner, **f32)
        # ---- scratch arena, allocated once ----
        mx = lambda vals: max(list(vals) + [1])
        mix = [l.mixer for l in cfg.layers]
        att = [m for m in mix if m.kind == "attention"]
        dlt = [m for m in mix if m.kind == "delta"]
        mam = [m for m in mix if m.kind == "mamba1"]
        ffs = [l.mlp for l in cfg.layers if l.mlp]
        self.buf_x = torch.empty(T * W, **f32)                                                 # residual stream (updated in place)
        self.buf_h = torch.empty(T * W, **act)                                                 # sublayer input
        self.buf_y = torch.empty(T * W, **act)                                                 # sublayer output
        self.buf_proj = torch.empty(T * mx([(m.heads + m.kv_heads) * m.dim + m.kv_heads * m.vdim for m in att] +
                                           [2 * m.kv_heads * m.dim + 2 * m.heads * m.vdim for m in dlt] +
                                           [2 * m.inner for m in mam]), **act)
        self.buf_q = torch.empty(T * mx([m.heads * m.dim for m in att] +                        # float32 queries | convolved q, k, v | dt
                                        [2 * m.kv_heads * m.dim + m.heads * m.vdim for m in dlt] + [m.inner for m in mam]), **f32)
        self.buf_att = torch.empty(T * mx([m.heads * m.vdim for m in att + dlt] + [m.inner for m in mam]), **act)
        self.buf_vfirst = torch.empty(T * mx(m.kv_heads * m.vdim for m in att if m.v_mix), **f32)
        self.buf_ba = torch.empty(T * mx(2 * m.heads for m in dlt), **f32)
        self.buf_gates = torch.empty(T * mx(2 * m.heads + m.kv_heads for m in dlt), **f32)
        self.buf_o = torch.empty(T * mx(m.heads * m.vdim for m in dlt), **f32)                  # un-normalised read-outs
        self.buf_xc = torch.empty(T * mx(m.inner for m in mam), **act)                          # convolved scan input
        self.buf_dbc = torch.empty(T * mx(m.dt_rank + 2 * m.state for m in mam), **act)
        self.buf_ff = torch.empty(T * mx(3 * f.ff for f in ffs), **act)
        self._mm_f32_out = None                        # whether torch.mm takes bfloat16 operands with a float32 out (probed once)

    # ------------------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path: str, dtype=torch.bfloat16, device="cuda", **kw) -> "KinanexModel":
        from .checkpoint import read_safetensors_file
        with open(os.path.join(path, "config.json")) as f:
            cfg = KinanexConfig.from_dict(json.load(f))
        return cls(cfg, read_safetensors_file(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @property
    def vocab_size(self) -> int:
        return self.cfg.vocab

    def state_bytes_per_slot(self) -> int:
        ts = list(self.cache_k.values()) + list(self.cache_v.values()) + list(self.rec_state.values())
        tails = sum(t.numel() * t.element_size() // self.n_slots for t in self.conv_tail.values())
        return sum(t.numel() * t.element_size() // self.n_slots for t in ts) + tails

    def _mm_to_f32(self, a: torch.Tensor, b_t: torch.Tensor, out: torch.Tensor) -> None:
        """out (float32) = a @ b_t^T, accumulated in float32 whatever the operands' type."""
        if a.dtype == torch.float32:
            torch.matmul(a, b_t.t(), out=out)
            return
        if self._mm_f32_out is None:
            try:
                torch.mm(a, b_t.t(), out_dtype=torch.float32, out=out)
                self._mm_f32_out = True
                return
            except (TypeError, RuntimeError):
                self._mm_f32_out = False
        if self._mm_f32_out:
            torch.mm(a, b_t.t(), out_dtype=torch.float32, out=out)
        else:
            out.copy_(torch.mm(a, b_t.t(), out_dtype=torch.float32))

    # ------------------------------------------------------------------------------------------
    def _attention(self, i, m, p, h, meta, T, first_mixed):
        tab = meta.table
        H, G, D, DV = m.heads, m.kv_heads, m.dim, m.vdim
        ld = (H + G) * D + G * DV
        proj = self.buf_proj[:T * ld].view(T, ld)
        torch.addmm(p.qkv_b, h, p.qkv.t(), out=proj)                                            # biases added in the projection
        qf = self.buf_q[:T * H * D].view(T, H, D)
        vf = self.buf_vfirst[:T * G * DV] if m.v_mix else None
        ops.seq_gqa_prep(proj, p.q_norm, p.k_norm, p.inv_freq, m.rot_dims, qf, self.cache_k[i], self.cache_v[i], tab, H, self.cfg.eps,
                         v_norm=True, v_first_in=vf if (m.v_mix and i != first_mixed) else None,
                         v_first_out=vf if (m.v_mix and i == first_mixed) else None, mix=p.vmix)
        att = self.buf_att[:T * H * DV].view(T, H, DV)
        # prompt portions: four consecutive rows per CTA share the key and value rows they read; decode-shaped steps: a CTA per row
        rows = 4 if T >= 4 * len(meta.segments) else 1
        ops.seq_talking_attention(qf, self.cache_k[i], self.cache_v[i], p.talk, att, tab, FULL_WINDOW, m.scale, sink=p.sink,
                                  rows_per_cta=rows)
        return att.view(T, H * DV)

    def _delta(self, i, m, p, h, meta, T):
        H, G, D, DV = m.heads, m.kv_heads, m.dim, m.vdim
        C = 2 * G * D + H * DV
        ld = C + H * DV
        proj = self.buf_proj[:T * ld].view(T, ld)
        torch.matmul(h, p.qkvg.t(), out=proj)
        ba = self.buf_ba[:T * 2 * H].view(T, 2 * H)
        self._mm_to_f32(h, p.ba, ba)                                                            # what feeds an exponential stays float32
        cs = self.buf_q[:T * C].view(T, C)
        ops.seq_conv_act(proj[:, :C], p.conv, None, self.conv_tail[i], cs, meta.table, act="silu")
        att = self.buf_att[:T * H * DV].view(T, H * DV)
        ops.seq_delta_rule(cs, ba, p.A_log, p.dt_bias, p.o_norm, proj[:, C:], self.rec_state[i], self.buf_gates, self.buf_o, att,
                           meta.table, meta.seg_starts, H, G, D, DV, self.cfg.eps, unit_eps=UNIT_EPS)
        return att

    def _mamba(self, i, m, p, h, meta, T):
        I, N, R = m.inner, m.state, m.dt_rank
        xz = self.buf_proj[:T * 2 * I].view(T, 2 * I)
        torch.matmul(h, p.w_in.t(), out=xz)
        xc = self.buf_xc[:T * I].view(T, I)
        ops.seq_conv_act(xz[:, :I], p.conv, p.conv_b, self.conv_tail[i], xc, meta.table, act="silu")
        dbc = self.buf_dbc[:T * (R + 2 * N)].view(T, R + 2 * N)
        torch.matmul(xc, p.w_x.t(), out=dbc)
        dt = self.buf_q[:T * I].view(T, I)
        self._mm_to_f32(dbc[:, :R], p.w_dt, dt)                                                 # the step size before its bias and softplus
        att = self.buf_att[:T * I].view(T, I)
        ops.seq_selective_scan(xc, dt, p.dt_b, dbc[:, R:], xz[:, I:], p.A_log, p.D, self.rec_state[i], att, meta.table, meta.seg_starts)
        return att

    @torch.no_grad()
    def forward_batch(self, input_ids: torch.Tensor, meta: BatchMeta, trace: Optional[list] = None) -> torch.Tensor:
        """input_ids: int32 [ntok] on the device. Returns the final-norm hidden state [ntok, W] (activation type), a view of
        the arena. `trace`, if a list, receives a copy of the residual stream after every layer (debugging)."""
        cfg, T, W = self.cfg, meta.ntok, self.cfg.width
        if T > self.max_step_tokens or input_ids.numel() != T:
            raise ValueError(f"forward_batch: {T} tokens (at most {self.max_step_tokens})")
        eps = cfg.eps
        x = self.buf_x[:T * W].view(T, W)
        h = self.buf_h[:T * W].view(T, W)
        y = self.buf_y[:T * W].view(T, W)
        ops.seq_embed(self.embed, input_ids, x)
        ops.seq_add_norm(x, self.embed_norm, None, eps, kind="rms", x_out=x)                    # the embedding's own norm, float32
        n = len(cfg.layers)
        ops.seq_residual_norm(x, self.weights[0].norm1 if n else self.final_norm, eps, w_offset=0.0, out=h)
        mixed = [k for k, l in enumerate(cfg.layers) if l.mixer.kind == "attention" and l.mixer.v_mix]
        first_mixed = mixed[0] if mixed else -1
        for i in range(n):
            p, m, f = self.weights[i], cfg.layers[i].mixer, cfg.layers[i].mlp
            after = self.weights[i + 1].norm1 if i + 1 < n else self.final_norm                 # the norm that reads this layer's result
            if m.kind == "attention":
                att = self._attention(i, m, p, h, meta, T, first_mixed)
            elif m.kind == "delta":
                att = self._delta(i, m, p, h, meta, T)
            else:
                att = self._mamba(i, m, p, h, meta, T)
            torch.matmul(att, p.o.t(), out=y)
            ops.seq_residual_norm(x, p.norm2 if f is not None else after, eps, y=y, y_scale=p.ls1, w_offset=0.0, x_out=x, out=h)
            if f is not None:
                gu = self.buf_ff[:T * 2 * f.ff].view(T, 2 * f.ff)
                a = self.buf_ff[T * 2 * f.ff:T * 3 * f.ff].view(T, f.ff)
                torch.matmul(h, p.gate_up.t(), out=gu)
                ops.seq_glu_clamp(gu, a, f.limit, GLU_ALPHA)
                torch.matmul(a, p.down.t(), out=y)
                ops.seq_residual_norm(x, after, eps, y=y, y_scale=p.ls2, w_offset=0.0, x_out=x, out=h)
            if trace is not None:
                trace.append(x.clone())
        return h

    @torch.no_grad()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [n, vocab] of final-norm hidden rows [n, W]: the embedding table is the output matrix."""
        if self.dtype == torch.float32:
            out = torch.matmul(hidden_rows, self.embed.t())
        else:
            out = torch.mm(hidden_rows, self.embed.t(), out_dtype=torch.float32)
        if self.cfg.logit_scale != 1.0:
            ops.seq_scale(out, self.cfg.logit_scale)
        return out

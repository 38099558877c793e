"""Repepel: a pre-norm decoder with a scaled residual that mixes full-length latent attention with scalar-decay linear
attention ("lightning") layers, dense or mixture-of-experts feed-forward layers, and a block of layers that runs several
times with the same weights.

With x the float32 residual stream, m = `residual_mult` and N(v; g) = v / sqrt(mean(v^2) + eps) * (1 + g):

    x <- x + m * mixer(N(x; norm1));      x <- x + m * ff(N(x; norm2))          (a layer may have no feed-forward)
    loop: layers start .. stop-1 run `times` times in a row with the same weights; every run has its own cache / state

mixers (`layers[i].type`):
    latent_attention  q = W_q h = per head [plain | rotary];  W_dkv h = [c' | r'];  c = unit_rms(c') * g_c;  only [c | rot(r')] is
                      cached. key_h = [W_uk c | rot(r')], value_h = W_uv c, causal softmax of scale * q.k over the whole
                      sequence, head output * sigmoid(W_g h)_head (one gate per head), then W_o. The rotation pairs entries
                      (2i, 2i + 1). Decode-shaped steps run the absorbed form (the query moves into the latent space, the cache
                      rows serve as keys and values); prompt portions expand keys and values of the sequence's rows.
    lightning         q, k, v = silu(W h);  per head S <- a_h S + k v^T,  o = S^T q;  all heads normed together, times a plain
                      weight and sigmoid(W_g h), then W_o. The state is float32 per slot and run.
feed-forward (`mlp.kind`):
    dense             W_down gelu(W_up h), the erf form
    moe               s = sigmoid(W_r h) in float32; choice = s + correction; the experts form groups of neighbours, a group
                      scores the sum of its two largest choices, only the best groups stay; the `top` largest choices get
                      weight scale * s; expert(h) = W_down (silu(W_gate h) * W_up h); a shared expert of the same form runs
                      for every token, times sigmoid(W_sg h).

Wiring follows `pitudra.PitudraModel`: a flat token batch with per-token slot and position (`state.BatchMeta`), state held by
the model and indexed by slot, a scratch arena allocated once, dense products in the vendor library, everything else in the
sequence-mixer kernel library (`ops.seq_*`, `ops.moe_*`). Every residual sum is fused with the norm that follows it
(`ops.seq_residual_norm`), the last one with the model's final norm. Nothing is cleared when a slot is released: cache rows are
valid by position, and the recurrence starts from zero at position 0.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from . import ops
from .state import BatchMeta

GROUP_TOP = 2                       # a group's score is the sum of this many of its largest choice scores
FULL_WINDOW = 1 << 30               # the latent layers see the whole sequence: a window no sequence reaches


@dataclass
class RepepelMixer:
    kind: str                       # "latent_attention" | "lightning"
    heads: int
    dim: int
    vdim: int
    kv_rank: int = 0                # latent attention ...
    rot_dim: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    scale: float = 1.0
    decay: Tuple[float, ...] = ()   # lightning: one per head


@dataclass
class RepepelFF:
    kind: str                       # "dense" | "moe"
    ff: int                         # hidden size (of one expert for "moe")
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    scale: float = 1.0
    shared_ff: int = 0              # 0: no shared expert


@dataclass
class RepepelLayer:
    mixer: RepepelMixer
    mlp: Optional[RepepelFF]


@dataclass
class RepepelConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float = 1.0
    layers: List[RepepelLayer] = field(default_factory=list)
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)
    name: str = "repepel"

    @staticmethod
    def from_dict(d: dict) -> "RepepelConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            kind, m = e.get("type"), e["mixer"]
            if kind == "latent_attention":
                rot = m.get("rot") or {}
                mixer = RepepelMixer(kind=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                                     kv_rank=int(m["kv_rank"]), rot_dim=int(m["rot_dim"]), rot_dims=int(rot.get("dims", m["rot_dim"])),
                                     rot_base=float(rot.get("base", 10000.0)), scale=float(m["scale"]))
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ValueError(f"layer {i}: {mixer.rot_dims} rotated dimensions of {mixer.rot_dim}")
            elif kind == "lightning":
                mixer = RepepelMixer(kind=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                                     decay=tuple(float(a) for a in m["decay"]))
                if len(mixer.decay) != mixer.heads:
                    raise ValueError(f"layer {i}: {len(mixer.decay)} decays for {mixer.heads} heads")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = e.get("mlp")
            if f is None:
                mlp = None
            elif f.get("kind") == "dense":
                mlp = RepepelFF(kind="dense", ff=int(f["ff"]))
            elif f.get("kind") == "moe":
                r = f["router"]
                g = r.get("groups") or {}
                count = int(g.get("count", 1))
                shared = f.get("shared") or {}
                mlp = RepepelFF(kind="moe", ff=int(f["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]), groups=count,
                                keep=int(g.get("keep", count)), scale=float(r.get("scale", 1.0)), shared_ff=int(shared.get("ff") or 0))
                if mlp.groups < 1 or mlp.experts % mlp.groups or not 1 <= mlp.keep <= mlp.groups:
                    raise ValueError(f"layer {i}: {mlp.experts} experts in {mlp.groups} groups, keep {mlp.keep}")
                if not 1 <= mlp.top <= mlp.keep * (mlp.experts // mlp.groups):
                    raise ValueError(f"layer {i}: top {mlp.top} of {mlp.keep} groups of {mlp.experts // mlp.groups} experts")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            layers.append(RepepelLayer(mixer=mixer, mlp=mlp))
        loop = None
        lp = d.get("loop")
        if lp:
            loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"]))
            if not (0 <= loop[0] <= loop[1] <= len(layers)) or loop[2] < 0:
                raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        return RepepelConfig(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                             residual_mult=float(d.get("residual_mult", 1.0)), layers=layers, loop=loop)

    def to_dict(self) -> dict:
        out = {"architecture": "Repepel", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "residual_mult": self.residual_mult, "layers": []}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        for l in self.layers:
            m, f = l.mixer, l.mlp
            if m.kind == "latent_attention":
                mx = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "rot_dim": m.rot_dim, "kv_rank": m.kv_rank, "scale": m.scale,
                      "rot": {"base": m.rot_base, "dims": m.rot_dims}}
            else:
                mx = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            if f is None:
                ff = None
            elif f.kind == "dense":
                ff = {"kind": "dense", "ff": f.ff}
            else:
                ff = {"kind": "moe", "expert": {"ff": f.ff},
                      "router": {"experts": f.experts, "top": f.top, "scale": f.scale, "groups": {"count": f.groups, "keep": f.keep}}}
                if f.shared_ff:
                    ff["shared"] = {"ff": f.shared_ff}
            out["layers"].append({"type": m.kind, "mixer": mx, "mlp": ff})
        return out

    def runs(self) -> List[int]:
        """Layer index of every layer run, in order: the looped block repeats, the rest runs once."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every tensor a checkpoint of this configuration must hold."""
        W = self.width
        out = {"embed": (self.vocab, W)}
        for i, l in enumerate(self.layers):
            m, f, p = l.mixer, l.mlp, f"l{i}."
            out[p + "norm1"] = (W,)
            x = p + "mix."
            if m.kind == "latent_attention":
                out.update({x + "q": (m.heads * (m.dim + m.rot_dim), W), x + "dkv": (m.kv_rank + m.rot_dim, W), x + "dkv.norm": (m.kv_rank,),
                            x + "uk": (m.heads * m.dim, m.kv_rank), x + "uv": (m.heads * m.vdim, m.kv_rank), x + "g": (m.heads, W),
                            x + "o": (W, m.heads * m.vdim)})
            else:
                out.update({x + "q": (m.heads * m.dim, W), x + "k": (m.heads * m.dim, W), x + "v": (m.heads * m.vdim, W),
                            x + "g": (m.heads * m.vdim, W), x + "norm": (m.heads * m.vdim,), x + "o": (W, m.heads * m.vdim)})
            if f is None:
                continue
            out[p + "norm2"] = (W,)
            y = p + "mlp."
            if f.kind == "dense":
                out.update({y + "up": (f.ff, W), y + "down": (W, f.ff)})
                continue
            out.update({y + "router": (f.experts, W), y + "correction": (f.experts,)})
            for e in range(f.experts):
                out.update({y + f"e{e}.gate": (f.ff, W), y + f"e{e}.up": (f.ff, W), y + f"e{e}.down": (W, f.ff)})
            if f.shared_ff:
                out.update({y + "shared.gate": (f.shared_ff, W), y + "shared.up": (f.shared_ff, W), y + "shared.down": (W, f.shared_ff),
                            y + "shared.sg": (1, W)})
        out.update({"final.norm": (W,), "head": (self.vocab, W)})
        return out


def random_weights(cfg: RepepelConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bfloat16 tensors of a configuration (CPU): matrices ~ N(0, 1/fan_in), the plain norm weights near 1, the
    zero-centred ones and the corrections small."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        if len(shape) == 2:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif name.endswith(("mix.norm", "dkv.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            t = 0.1 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


class _LayerWeights:
    """Device tensors of one layer: large matrices in the activation type (fused where one product serves several), vectors
    and the router float32."""

    def __init__(self, cfg: RepepelConfig, i: int, sd: Dict[str, torch.Tensor], dtype, device):
        spec, p = cfg.layers[i], f"l{i}."
        m, f = spec.mixer, spec.mlp

        def big(*names):
            t = torch.cat([sd[p + n] for n in names], 0) if len(names) > 1 else sd[p + names[0]]
            return t.to(device=device, dtype=dtype).contiguous()

        def small(*names):
            t = torch.cat([sd[p + n].to(torch.float32) for n in names], 0) if len(names) > 1 else sd[p + names[0]]
            return t.to(device=device, dtype=torch.float32).contiguous()

        self.norm1 = small("norm1")
        if m.kind == "latent_attention":
            self.q = big("mix.q")
            self.dkvg = big("mix.dkv", "mix.g")                                                   # rows [c' | r' | one gate per head]
            self.dkv_norm = small("mix.dkv.norm")
            self.uk_flat, self.uv_flat = big("mix.uk"), big("mix.uv")                             # latent rows -> per-head keys / values
            self.uk = self.uk_flat.view(m.heads, m.dim, m.kv_rank)                                # q_plain[h] @ uk[h] -> latent space
            self.uv_t = self.uv_flat.view(m.heads, m.vdim, m.kv_rank).transpose(1, 2)             # latent[h] @ uv_t[h] -> value space
            half = m.rot_dims // 2
            fr = torch.tensor(m.rot_base, dtype=torch.float64) ** (-2.0 * torch.arange(half, dtype=torch.float64) / max(m.rot_dims, 1))
            self.inv_freq = fr.to(device=device, dtype=torch.float32)
        else:
            self.qkvg = big("mix.q", "mix.k", "mix.v", "mix.g")                                   # rows [q ; k ; v ; g]
            self.o_norm = small("mix.norm")
            self.decay = torch.tensor(m.decay, dtype=torch.float64).to(device=device, dtype=torch.float32)
        self.o = big("mix.o")
        if f is None:
            return
        self.norm2 = small("norm2")
        if f.kind == "dense":
            self.up, self.down = big("mlp.up"), big("mlp.down")
            return
        # the shared expert's gate row rides behind the router's rows: one float32 product serves both
        self.router = small("mlp.router", "mlp.shared.sg") if f.shared_ff else small("mlp.router")
        self.correction = small("mlp.correction")
        self.gate_up = torch.stack([torch.cat([sd[p + f"mlp.e{e}.gate"], sd[p + f"mlp.e{e}.up"]], 0) for e in range(f.experts)]) \
            .to(device=device, dtype=dtype).contiguous()                                          # [E, 2 F, W], gate rows first
        self.edown = torch.stack([sd[p + f"mlp.e{e}.down"] for e in range(f.experts)]).to(device=device, dtype=dtype).contiguous()
        if f.shared_ff:
            self.shared_gu, self.shared_down = big("mlp.shared.gate", "mlp.shared.up"), big("mlp.shared.down")


class RepepelModel(torch.nn.Module):
    """Weights, per-slot state and the forward pass over a flat token batch (`state.BatchMeta`).

    dtype: torch.bfloat16 (serving: bfloat16 matrix products with float32 accumulation) or torch.float32 (everything in true
    float32). n_slots sequences can be live at once; a step carries at most max_step_tokens tokens; a sequence holds at most
    max_seq_tokens tokens (the latent caches have that many rows per slot and layer run)."""

    architecture = "Repepel"
    DEFAULT_SEQ_TOKENS = 8192

    def __init__(self, cfg: RepepelConfig, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16, device="cuda",
                 n_slots: int = 8, max_step_tokens: int = 2048, max_seq_tokens: Optional[int] = None):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("RepepelModel: dtype must be torch.bfloat16 or torch.float32")
        for name, shape in cfg.tensor_shapes().items():
            if name not in weights:
                raise KeyError(f"tensor {name} is missing from the checkpoint")
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"tensor {name}: shape {tuple(weights[name].shape)}, the configuration says {tuple(shape)}")
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.n_slots, self.max_step_tokens = n_slots, max_step_tokens
        self.max_seq_len = max(int(max_seq_tokens or self.DEFAULT_SEQ_TOKENS), 1)      # checked by the scheduler
        # true float32 products in float32 mode; no reduced-precision accumulation of bfloat16 products
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        dev, W, T = self.device, cfg.width, max_step_tokens
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=dtype, device=dev)
        self.embed = weights["embed"].to(**act).contiguous()
        self.head = weights["head"].to(**act).contiguous()
        self.final_norm = weights["final.norm"].to(**f32).contiguous()
        self.weights = [_LayerWeights(cfg, i, weights, dtype, dev) for i in range(len(cfg.layers))]
        self.runs = cfg.runs()
        # ---- per-slot state, one per layer RUN (a looped layer has one per pass) ----
        self.latent_cache: Dict[int, torch.Tensor] = {}                                        # run -> [slots, cap, kv_rank + rot_dim]
        self.rec_state: Dict[int, torch.Tensor] = {}                                           # run -> [slots, H, D, DV] float32
        for r, i in enumerate(self.runs):
            m = cfg.layers[i].mixer
            if m.kind == "latent_attention":
                self.latent_cache[r] = torch.zeros(n_slots, self.max_seq_len, m.kv_rank + m.rot_dim, **act)
            else:
                self.rec_state[r] = torch.zeros(n_slots, m.heads, m.dim, m.vdim, **f32)
        # ---- scratch arena, allocated once ----
        mx = lambda vals: max(list(vals) + [1])
        mix = [l.mixer for l in cfg.layers]
        lat = [m for m in mix if m.kind == "latent_attention"]
        lin = [m for m in mix if m.kind == "lightning"]
        ffs = [l.mlp for l in cfg.layers if l.mlp]
        moes = [f for f in ffs if f.kind == "moe"]
        self.buf_x = torch.empty(T * W, **f32)                                                 # residual stream (updated in place)
        self.buf_h = torch.empty(T * W, **act)                                                 # sublayer input
        self.buf_y = torch.empty(T * W, **act)                                                 # sublayer output
        self.buf_y2 = torch.empty(T * W, **act)                                                # shared expert's output
        self.buf_proj = torch.empty(T * mx([m.kv_rank + m.rot_dim + m.heads for m in lat] +
                                           [2 * m.heads * (m.dim + m.vdim) for m in lin]), **act)
        self.buf_q = torch.empty(T * mx(m.heads * (m.dim + m.rot_dim) for m in lat), **act)
        self.buf_qa = torch.empty(T * mx(m.heads * (max(m.kv_rank, m.dim) + m.rot_dim) for m in lat), **f32)
        self.buf_att = torch.empty(T * mx([m.heads * m.kv_rank for m in lat] + [m.heads * m.vdim for m in lin]), **act)
        self.buf_att2 = torch.empty(T * mx(m.heads * m.vdim for m in lat), **act)
        self.buf_rec = torch.empty(T * mx(m.heads * (m.vdim + 2 * m.dim) for m in lin), **f32)   # un-normalised outputs, silu(q), silu(k)
        self.buf_ff = torch.empty(T * mx([f.ff for f in ffs if f.kind == "dense"] + [3 * f.shared_ff for f in moes]), **act)
        tops = mx(f.top for f in moes)
        self.buf_idx = torch.empty(T * tops, dtype=torch.int32, device=dev)
        self.buf_rw = torch.empty(T * (tops + 1), **f32)                                       # expert weights, then the shared expert's gate
        self.buf_pair = torch.empty(T * tops * W if moes else 1, **act)
        # bfloat16 takes the tensor-core forms where the sizes allow: grouped experts once an expert sees several rows, latent
        # attention per 16 tokens (prompt portions) or per 16 heads (decoding). QSPEC_SEQ_TILES=0 keeps the plain forms.
        self.use_tiles = dtype == torch.bfloat16 and os.environ.get("QSPEC_SEQ_TILES", "1") != "0"
        self.tiles_min_tokens = 64           # a step with fewer tokens, or fewer than 16 per sequence, is decode-shaped
        self.prompt_tiles_min_ctas = 256     # (64-token blocks x heads) from which a prompt portion takes the tile form of its attention
        lat_tiles = [m for m in lat if self.use_tiles and m.kv_rank % 8 == 0 and m.rot_dim % 8 == 0 and
                     ops.seq_window_attention_mma_supported(dtype, m.dim, m.rot_dim, m.vdim, m.heads, m.heads, True)]
        self._lat_tiles = {id(m) for m in lat_tiles}
        self.buf_kmat = torch.empty(mx(self.max_seq_len * m.heads * m.dim for m in lat_tiles), **act)
        self.buf_vmat = torch.empty(mx(self.max_seq_len * m.heads * m.vdim for m in lat_tiles), **act)
        self._bmm_f32_out = None                       # whether torch.bmm takes bfloat16 operands with a float32 out (probed once)

    # ------------------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path: str, dtype=torch.bfloat16, device="cuda", **kw) -> "RepepelModel":
        from .checkpoint import read_safetensors_file
        with open(os.path.join(path, "config.json")) as f:
            cfg = RepepelConfig.from_dict(json.load(f))
        return cls(cfg, read_safetensors_file(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @property
    def vocab_size(self) -> int:
        return self.cfg.vocab

    def state_bytes_per_slot(self) -> int:
        ts = list(self.latent_cache.values()) + list(self.rec_state.values())
        return sum(t.numel() * t.element_size() // self.n_slots for t in ts)

    def _bmm_to_f32(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
        """out (float32) = a @ b per batch entry, accumulated in float32 whatever the operands' type."""
        if a.dtype == torch.float32:
            torch.bmm(a, b, out=out)
            return
        if self._bmm_f32_out is None:
            try:
                torch.bmm(a, b, out_dtype=torch.float32, out=out)
                self._bmm_f32_out = True
                return
            except (TypeError, RuntimeError):
                self._bmm_f32_out = False
        if self._bmm_f32_out:
            torch.bmm(a, b, out_dtype=torch.float32, out=out)
        else:
            out.copy_(torch.bmm(a, b))

    # ------------------------------------------------------------------------------------------
    def _latent_attention(self, run, m, p, h, meta, T, prompt_shaped):
        tab = meta.table
        H, DQ, r, R = m.heads, m.dim + m.rot_dim, m.kv_rank, m.rot_dim
        q = self.buf_q[:T * H * DQ].view(T, H, DQ)
        torch.matmul(h, p.q.t(), out=q.view(T, H * DQ))
        ld = r + R + H
        d = self.buf_proj[:T * ld].view(T, ld)
        torch.matmul(h, p.dkvg.t(), out=d)
        gate = d[:, r + R:]                                                         # one logit per head
        cache = self.latent_cache[run]
        ops.seq_latent_prep(d, 0, r, R, None, p.dkv_norm, p.inv_freq, m.rot_dims, None, cache, tab, self.cfg.eps, pairing="interleaved")
        if prompt_shaped and len(meta.segments) == 1 and id(m) in self._lat_tiles:
            # expanded form on the tensor cores: per-head keys and values of the rows this sequence holds after the step
            slot, rows, cap = meta.segments[0][1], meta.max_length, cache.shape[1]
            ring = cache[slot, :rows]
            kmat = self.buf_kmat[:rows * H * m.dim].view(rows, H * m.dim)
            vmat = self.buf_vmat[:rows * H * m.vdim].view(rows, H * m.vdim)
            torch.matmul(ring[:, :r], p.uk_flat.t(), out=kmat)
            torch.matmul(ring[:, :r], p.uv_flat.t(), out=vmat)
            qf = self.buf_qa[:T * H * DQ].view(T, H, DQ)
            qf[:, :, :m.dim].copy_(q[:, :, :m.dim])
            ops.seq_rotary(q, m.dim, qf[:, :, m.dim:], m.rot_dims, p.inv_freq, tab, pairing="interleaved")
            att = self.buf_att2[:T * H * m.vdim].view(T, H, m.vdim)
            # the products cover `rows` rows only; positions below `rows` never wrap, so any ring size >= rows addresses them
            kview = kmat.view(1, rows, H, m.dim).expand(self.n_slots, rows, H, m.dim)
            vview = vmat.view(1, rows, H, m.vdim).expand(self.n_slots, rows, H, m.vdim)
            # 64 tokens per CTA with the keys through shared memory, once the portion fills the GPU with such CTAs; shorter
            # portions keep 16 tokens per CTA, whose four warps share a block's keys
            if ((T + 63) // 64) * H >= self.prompt_tiles_min_ctas and ops.seq_prompt_attention_mma_supported(self.dtype, m.dim, R, m.vdim):
                ops.seq_prompt_attention_mma(qf, kview, cache[:, :rows, r:], vview, att, slot, meta.segments[0][2], FULL_WINDOW, m.scale,
                                             gate=gate, gate_per_head=True)
            else:
                ops.seq_window_attention_mma(qf, kview, cache[:, :rows, r:], vview, att, tab, FULL_WINDOW, m.scale, True, gate=gate,
                                             gate_per_head=True)
            return att.view(T, H * m.vdim)
        # absorbed form: the query moves into the latent space (W_uk^T q_plain per head, float32) and the cache rows serve as
        # keys and as values; the up-projection of the values follows the attention. The per-head gate is a scalar, so it may
        # multiply the latent output before that projection.
        qf = self.buf_qa[:T * H * (r + R)].view(T, H, r + R)
        self._bmm_to_f32(q[:, :, :m.dim].transpose(0, 1), p.uk, qf[:, :, :r].transpose(0, 1))
        ops.seq_rotary(q, m.dim, qf[:, :, r:], m.rot_dims, p.inv_freq, tab, pairing="interleaved")
        olat = self.buf_att[:T * H * r].view(T, H, r)
        groups = 1 if H <= 16 else (H // 16 if H % 16 == 0 else 0)                 # the heads share one key row: 16 of them per CTA
        if self.use_tiles and groups and r % 8 == 0 and R % 8 == 0 and \
                ops.seq_window_attention_mma_supported(self.dtype, r, R, r, H, groups, False):
            ck = cache[:, :, :r].unsqueeze(2).expand(cache.shape[0], cache.shape[1], groups, r)
            ops.seq_window_attention_mma(qf, ck, cache[:, :, r:], ck, olat, tab, FULL_WINDOW, m.scale, False, gate=gate, gate_per_head=True)
        else:
            ck = cache.unsqueeze(2)                                                 # one key/value head: [slots, cap, 1, kv_rank + rot_dim]
            ops.seq_window_attention(qf[:, :, :r], qf[:, :, r:], ck, ck[..., :r], olat, tab, FULL_WINDOW, m.scale, gate=gate,
                                     gate_per_head=True)
        att = self.buf_att2[:T * H * m.vdim].view(T, H, m.vdim)
        torch.bmm(olat.transpose(0, 1), p.uv_t, out=att.transpose(0, 1))
        return att.view(T, H * m.vdim)

    def _lightning(self, run, m, p, h, meta, T):
        ld = 2 * m.heads * (m.dim + m.vdim)
        proj = self.buf_proj[:T * ld].view(T, ld)
        torch.matmul(h, p.qkvg.t(), out=proj)
        att = self.buf_att[:T * m.heads * m.vdim].view(T, m.heads * m.vdim)
        ops.seq_lightning(proj, p.decay, p.o_norm, self.rec_state[run], self.buf_rec, att, meta.table, m.heads, m.dim, m.vdim,
                          self.cfg.eps, seg_starts=meta.seg_starts)
        return att

    @torch.no_grad()
    def forward_batch(self, input_ids: torch.Tensor, meta: BatchMeta, trace: Optional[list] = None) -> torch.Tensor:
        """input_ids: int32 [ntok] on the device. Returns the final-norm hidden state [ntok, W] (activation type), a view of
        the arena. `trace`, if a list, receives a copy of the residual stream after every layer run (debugging)."""
        cfg, T, W = self.cfg, meta.ntok, self.cfg.width
        if T > self.max_step_tokens or input_ids.numel() != T:
            raise ValueError(f"forward_batch: {T} tokens (at most {self.max_step_tokens})")
        eps, mult = cfg.eps, cfg.residual_mult
        x = self.buf_x[:T * W].view(T, W)
        h = self.buf_h[:T * W].view(T, W)
        y = self.buf_y[:T * W].view(T, W)
        ops.seq_embed(self.embed, input_ids, x)
        prompt_shaped = self.use_tiles and T >= self.tiles_min_tokens and T >= 16 * len(meta.segments)
        runs = self.runs
        first = self.weights[runs[0]].norm1 if runs else self.final_norm
        ops.seq_residual_norm(x, first, eps, out=h)
        for r, i in enumerate(runs):
            p, m, f = self.weights[i], cfg.layers[i].mixer, cfg.layers[i].mlp
            after = self.weights[runs[r + 1]].norm1 if r + 1 < len(runs) else self.final_norm      # the norm that reads this layer's result
            if m.kind == "latent_attention":
                att = self._latent_attention(r, m, p, h, meta, T, prompt_shaped)
            else:
                att = self._lightning(r, m, p, h, meta, T)
            torch.matmul(att, p.o.t(), out=y)
            ops.seq_residual_norm(x, p.norm2 if f is not None else after, eps, y=y, mult=mult, x_out=x, out=h)
            if f is not None and f.kind == "dense":
                u = self.buf_ff[:T * f.ff].view(T, f.ff)
                torch.matmul(h, p.up.t(), out=u)
                ops.seq_act(u, "gelu_erf")
                torch.matmul(u, p.down.t(), out=y)
                ops.seq_residual_norm(x, after, eps, y=y, mult=mult, x_out=x, out=h)
            elif f is not None:
                idx = self.buf_idx[:T * f.top].view(T, f.top)
                pair = self.buf_pair[:T * f.top * W].view(T, f.top, W)
                wts = self._route(f, p, h, idx, T)
                # grouped tiles once an expert sees several rows on average; a handful of tokens stay with the row-per-CTA form
                if self.use_tiles and T * f.top >= 4 * f.experts and ops.moe_expert_grouped_supported(h, f.ff):
                    ops.moe_expert_grouped(h, p.gate_up, p.edown, idx, pair, f.experts, f.ff, 0.0, act="silu")
                else:
                    ops.moe_expert_tokens(h, p.gate_up, p.edown, idx, pair, f.experts, f.ff, 0.0, act="silu")
                y2 = y2w = None
                if f.shared_ff:
                    F = f.shared_ff
                    gu = self.buf_ff[:T * 2 * F].view(T, 2 * F)
                    a = self.buf_ff[T * 2 * F:T * 3 * F].view(T, F)
                    torch.matmul(h, p.shared_gu.t(), out=gu)
                    ops.seq_silu_mul(gu, a)
                    y2 = self.buf_y2[:T * W].view(T, W)
                    torch.matmul(a, p.shared_down.t(), out=y2)
                    y2w = wts[1]
                ops.seq_residual_norm(x, after, eps, y=pair, y_w=wts[0], y2=y2, y2_w=y2w, mult=mult, x_out=x, out=h)
            if trace is not None:
                trace.append(x.clone())
        return h

    def _route(self, f, p, h, idx, T):
        """Expert choice and weights of a mixture layer: (weights [T, top], the shared expert's gate [T] or None)."""
        rw = self.buf_rw[:T * f.top].view(T, f.top)
        extra = self.buf_rw[T * f.top:T * (f.top + 1)].view(T, 1) if f.shared_ff else None
        ops.moe_route_grouped(h, p.router, p.correction, idx, rw, score="sigmoid", groups=f.groups, keep=f.keep, group_top=GROUP_TOP,
                              scale=f.scale, extra=extra)
        return rw, (extra.view(T) if extra is not None else None)

    @torch.no_grad()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [n, vocab] of final-norm hidden rows [n, W]."""
        if self.dtype == torch.float32:
            return torch.matmul(hidden_rows, self.head.t())
        return torch.mm(hidden_rows, self.head.t(), out_dtype=torch.float32)

"""Kinanex on the GPU against the plain CPU restatement (oracle/kinanex_oracle.py): every mechanism alone, then whole models
through the scheduler's step function -- whole prompts, token-by-token decoding, portions down to two tokens, mixed batches,
reused slots, keys far back in the cache, the first tokens of a sequence, other sizes, long decoding and greedy generation."""
import json
import math
import os

import pytest
import torch

from oracle import kinanex_oracle as O

pytestmark = pytest.mark.gpu

F32, BF16, F64 = torch.float32, torch.bfloat16, torch.float64
FULL = 1 << 30


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from qspec_b200.build import build_seq_library
    build_seq_library()


def meta_table(segments):
    """segments: (slot, first position, count, phase) -> (int32 [5, ntok], int32 [segments] first rows) on the device."""
    rows = [[], [], [], [], []]
    at, starts = 0, []
    for slot, p0, n, phase in segments:
        starts.append(at)
        for k in range(n):
            for r, v in zip(rows, (slot, p0 + k, at, at + n, phase)):
                r.append(v)
        at += n
    return torch.tensor(rows, dtype=torch.int32, device="cuda"), torch.tensor(starts, dtype=torch.int32, device="cuda")


def rnd(g, *shape, dtype=F32, scale=1.0):
    """Random values that the element type represents exactly, as float64."""
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(F64)


def tol(dtype):
    return 2e-5 if dtype == F32 else 2.5e-2


def close(got, want, dtype, scale=None):
    want = want.to(F64)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got.detach().cpu().to(F64) - want).abs().max())
    assert err <= tol(dtype) * max(s, 1e-6), f"max error {err:.3g} against scale {s:.3g}"


def dev(t, dtype=F32):
    return t.to(dtype).cuda().contiguous()


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("W", [96, 257, 40])
def test_residual_sum_with_a_layer_scale_and_plain_norm_weight(dtype, W):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W)
    T = 7
    x, y, ls, w = rnd(g, T, W), rnd(g, T, W, dtype=dtype), rnd(g, W) + 1.0, rnd(g, W) + 1.0
    r = x + ls * y
    want = O.unit_rms(r, 1e-5) * w
    xo = torch.empty(T, W, dtype=F32, device="cuda")
    out = torch.empty(T, W, dtype=dtype, device="cuda")
    ops.seq_residual_norm(dev(x), dev(w), 1e-5, y=dev(y, dtype), y_scale=dev(ls), w_offset=0.0, x_out=xo, out=out)
    close(xo, r, F32)
    close(out, want, dtype)


def _feed_conv(ops, x, w, b, tail, cuts, slot, dtype, out_dtype, phase0=0):
    """Runs x [T, C] through the convolution kernel in portions; returns the outputs and the phase after the last step."""
    outs, at, phase = [], 0, phase0
    for n in cuts:
        tab, _ = meta_table([(slot, at, n, phase)])
        o = torch.empty(n, x.shape[1], dtype=out_dtype, device="cuda")
        ops.seq_conv_act(dev(x[at:at + n], dtype), w, b, tail, o, tab, act="silu")
        outs.append(o.float().cpu())
        at += n
        phase ^= 1
    return torch.cat(outs), phase


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("C,taps,bias", [(40, 4, True), (300, 2, False), (17, 5, True), (8, 1, False), (64, 3, False)])
def test_short_convolution_carries_its_last_inputs_over_portions(dtype, C, taps, bias):
    """Portions shorter than the convolution, single tokens, a long one; the tail of a slot survives another slot's steps and a
    new sequence in a used slot starts from zeros."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(C + taps)
    T = 41
    x, w = rnd(g, T, C, dtype=dtype), rnd(g, C, taps)
    b = rnd(g, C) if bias else None
    want = O.silu(O.causal_conv(x, w, b))
    tail = torch.full((2, 3, taps - 1, C), 7.0, dtype=F32, device="cuda")                        # stale numbers everywhere
    wd, bd = dev(w), dev(b) if bias else None
    for out_dtype in {dtype, F32}:
        cuts = [1, 1, 2, 1, 9, 2, 3, 1, 1, 20]
        got, phase = _feed_conv(ops, x, wd, bd, tail, cuts, 1, dtype, out_dtype)
        close(got, want, out_dtype if out_dtype == BF16 else F32)
        # another sequence in another slot in between, then the first one again from its start in the slot it used
        _feed_conv(ops, x.flip(0), wd, bd, tail, [5, 36], 2, dtype, out_dtype)
        got, _ = _feed_conv(ops, x, wd, bd, tail, [T], 1, dtype, out_dtype, phase0=phase)
        close(got, want, out_dtype if out_dtype == BF16 else F32)
    # two sequences in one step, one of them continuing
    xa, xb = x[:19], x[19:]
    tab, _ = meta_table([(0, 0, 6, 0)])
    o = torch.empty(6, C, dtype=F32, device="cuda")
    ops.seq_conv_act(dev(xa[:6], dtype), wd, bd, tail, o, tab, act="silu")
    tab, _ = meta_table([(0, 6, 13, 1), (2, 0, 22, 0)])
    o = torch.empty(35, C, dtype=F32, device="cuda")
    ops.seq_conv_act(dev(torch.cat([xa[6:], xb]), dtype), wd, bd, tail, o, tab, act="silu")
    close(o[:13], O.silu(O.causal_conv(xa, w, b))[6:], F32)
    close(o[13:], O.silu(O.causal_conv(xb, w, b)), F32)


def _delta_inputs(g, T, H, G, D, DV):
    q, k, v = rnd(g, T, G, D), rnd(g, T, G, D), rnd(g, T, H, DV)
    b, a = rnd(g, T, H), rnd(g, T, H)
    A_log, dt_bias, norm_w = rnd(g, H, scale=0.5), rnd(g, H, scale=0.5) - 1.0, rnd(g, DV, scale=0.1) + 1.0
    return q, k, v, b, a, A_log, dt_bias, norm_w


def _delta_want(q, k, v, b, a, A_log, dt_bias, norm_w, gate, eps):
    D = q.shape[-1]
    qn = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(D)
    kn = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(b)
    dec = torch.exp(-torch.exp(A_log) * O.softplus(a + dt_bias))
    o = O.delta_rule(qn, kn, v, beta, dec)
    o = O.unit_rms(o, eps) * norm_w
    return o * O.silu(gate) if gate is not None else o


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,G,D,DV", [(2, 2, 16, 24), (4, 2, 33, 7), (3, 1, 130, 40), (2, 2, 64, 64), (6, 3, 5, 17), (1, 1, 200, 16)])
def test_delta_rule_state_over_portions_and_slots(dtype, H, G, D, DV):
    """The whole sequence at once, then in portions down to one token with another sequence stepping through a neighbouring
    slot, then again from position 0 in the used slot (the old state must not leak)."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(H * 1000 + D)
    T, eps = 45, 1e-5
    q, k, v, b, a, A_log, dt_bias, norm_w = _delta_inputs(g, T, H, G, D, DV)
    gate = rnd(g, T, H * DV, dtype=dtype)
    want = _delta_want(q, k, v, b, a, A_log, dt_bias, norm_w, gate.view(T, H, DV), eps).reshape(T, H * DV)
    q2, k2, v2, b2, a2 = rnd(g, T, G, D), rnd(g, T, G, D), rnd(g, T, H, DV), rnd(g, T, H), rnd(g, T, H)
    want2 = _delta_want(q2, k2, v2, b2, a2, A_log, dt_bias, norm_w, None, eps).reshape(T, H * DV)
    state = torch.full((3, H, D, DV), 3.0, dtype=F32, device="cuda")
    C = 2 * G * D + H * DV
    scratch_g = torch.empty(2 * T * (2 * H + G), dtype=F32, device="cuda")
    scratch_o = torch.empty(2 * T * H * DV, dtype=F32, device="cuda")

    def step(segs):
        """segs: (slot, first position, count, which sequence)."""
        rows, bas, gates = [], [], []
        for slot, p0, n, which in segs:
            qq, kk, vv, bb, aa = (q, k, v, b, a) if which == 0 else (q2, k2, v2, b2, a2)
            rows.append(torch.cat([qq[p0:p0 + n].reshape(n, -1), kk[p0:p0 + n].reshape(n, -1), vv[p0:p0 + n].reshape(n, -1)], 1))
            bas.append(torch.cat([bb[p0:p0 + n], aa[p0:p0 + n]], 1))
            gates.append(gate[p0:p0 + n] if which == 0 else torch.full((n, H * DV), 30.0, dtype=F64))     # silu(30) = 30
        tab, starts = meta_table([(s, p0, n, 0) for s, p0, n, _ in segs])
        n = tab.shape[1]
        out = torch.empty(n, H * DV, dtype=dtype, device="cuda")
        ops.seq_delta_rule(dev(torch.cat(rows)), dev(torch.cat(bas)), dev(A_log), dev(dt_bias), dev(norm_w), dev(torch.cat(gates), dtype),
                           state, scratch_g, scratch_o, out, tab, starts, H, G, D, DV, eps)
        return out.float().cpu()

    close(step([(1, 0, T, 0)]), want, dtype)
    at, got, got2 = 0, [], []
    for n in [1, 2, 1, 17, 2, 3, 19]:
        o = step([(1, at, n, 0), (0, at, n, 1)])
        got.append(o[:n]); got2.append(o[n:] / 30.0)
        at += n
    close(torch.cat(got), want, dtype)
    close(torch.cat(got2), want2, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("inner,N", [(40, 16), (130, 3), (256, 40), (33, 1), (64, 130), (20, 8), (12, 500)])
def test_selective_scan_state_over_portions_and_slots(dtype, inner, N):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(inner + N)
    T = 50
    x, z, bc = rnd(g, T, inner, dtype=dtype), rnd(g, T, inner, dtype=dtype), rnd(g, T, 2 * N, dtype=dtype)
    dt_pre, dt_b = rnd(g, T, inner), rnd(g, inner) - 1.0
    A_log, Dk = torch.log(0.5 + 3.0 * torch.rand(inner, N, generator=g)).to(F32).to(F64), rnd(g, inner)
    dt = O.softplus(dt_pre + dt_b)
    want = O.selective_scan(x, dt, -torch.exp(A_log), bc[:, :N], bc[:, N:], Dk) * O.silu(z)
    state = torch.full((3, inner, N), 5.0, dtype=F32, device="cuda")

    def step(slot, p0, n, other=None):
        segs = [(slot, p0, n, 0)] + ([other] if other else [])
        tab, starts = meta_table(segs)
        idx = list(range(p0, p0 + n)) + (list(range(other[1], other[1] + other[2])) if other else [])
        out = torch.empty(len(idx), inner, dtype=dtype, device="cuda")
        ops.seq_selective_scan(dev(x[idx], dtype), dev(dt_pre[idx]), dev(dt_b), dev(bc[idx], dtype), dev(z[idx], dtype), dev(A_log), dev(Dk),
                               state, out, tab, starts)
        return out.float().cpu()

    close(step(2, 0, T), want, dtype)
    at, got = 0, []
    for n in [1, 1, 2, 16, 1, 17, 2, 10]:
        o = step(2, at, n, other=(0, 0, 5, 0))                      # a second sequence restarts in slot 0 in every step
        got.append(o[:n])
        close(o[n:], want[:5], dtype)
        at += n
    close(torch.cat(got), want, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,G,D,DV,dims,scaling", [(4, 2, 16, 24, 16, True), (3, 3, 10, 6, 4, False), (2, 1, 40, 33, 0, False),
                                                   (6, 2, 12, 8, 12, True)])
def test_head_norms_rotation_value_norm_and_value_blend(dtype, H, G, D, DV, dims, scaling):
    _cuda()
    from qspec_b200 import ops
    from qspec_b200.kinanex import rotary_frequencies
    g = torch.Generator().manual_seed(H + D)
    eps, cap, T = 1e-5, 64, 9
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64} if scaling else None
    pos0 = 31
    p = rnd(g, T, (H + G) * D + G * DV + 3, dtype=dtype)                          # three more columns: the leading dimension is free
    qw, kw = rnd(g, D) + 1.0, rnd(g, D) + 1.0
    pos = torch.arange(pos0, pos0 + T)
    fr = O.stretched_frequencies(dims, 50.0, sc) if dims else []
    q = O.unit_rms(p[:, :H * D].view(T, H, D), eps) * qw
    k = O.unit_rms(p[:, H * D:(H + G) * D].view(T, G, D), eps) * kw
    if dims:
        q, k = O.rotate_halves(q, pos, fr), O.rotate_halves(k, pos, fr)
        assert torch.allclose(rotary_frequencies(dims, 50.0, sc), torch.tensor(fr, dtype=F64), rtol=1e-12)
        if scaling:                                                                # the bands differ: kept, ramp, divided
            plain = O.stretched_frequencies(dims, 50.0, None)
            ratios = sorted({round(a / b, 6) for a, b in zip(fr, plain)})
            assert ratios[0] == 0.25 and ratios[-1] == 1.0 and len(ratios) >= 3
    v = O.unit_rms(p[:, (H + G) * D:(H + G) * D + G * DV].view(T, G, DV), eps)
    first = rnd(g, T, G, DV)
    lam = 0.3125
    tab, _ = meta_table([(1, pos0, T, 0)])
    inv = dev(torch.tensor(fr, dtype=F64)) if dims else None
    for blend in (False, True):
        ck = torch.zeros(2, cap, G, D, dtype=dtype, device="cuda")
        cv = torch.zeros(2, cap, G, DV, dtype=dtype, device="cuda")
        qo = torch.empty(T, H, D, dtype=F32, device="cuda")
        keep = torch.zeros(T * G * DV, dtype=F32, device="cuda")
        ops.seq_gqa_prep(dev(p, dtype), dev(qw), dev(kw), inv, dims, qo, ck, cv, tab, H, eps, v_norm=True,
                         v_first_in=dev(first.reshape(-1)) if blend else None, v_first_out=None if blend else keep,
                         mix=dev(torch.tensor([lam], dtype=F64)))
        close(qo, q, F32)
        close(ck[1, pos0:pos0 + T], k, dtype)
        close(cv[1, pos0:pos0 + T], (1 - lam) * v + lam * first if blend else v, dtype)
        if not blend:
            close(keep.view(T, G, DV), v, F32)
        assert float(ck[0].abs().max()) == 0.0 and float(ck[1, :pos0].abs().max()) == 0.0   # nothing but the step's rows is written


def _fill_cache(k, v, slot, slots, cap, dtype):
    n, G, D = k.shape
    ck = torch.full((slots, cap, G, D), 9.0, dtype=dtype, device="cuda")
    cv = torch.full((slots, cap, G, v.shape[2]), 9.0, dtype=dtype, device="cuda")
    ck[slot, :n] = dev(k, dtype)
    cv[slot, :n] = dev(v, dtype)
    return ck, cv


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("rows", [1, 4])
@pytest.mark.parametrize("H,G,D,DV,n", [(4, 2, 16, 24, 70), (3, 3, 10, 6, 33), (8, 1, 40, 130, 50), (1, 1, 7, 5, 3), (6, 2, 48, 64, 97),
                                        (20, 2, 8, 3, 150), (12, 4, 128, 128, 140)])
def test_attention_with_mixed_heads_and_the_extra_unit_in_the_denominator(dtype, H, G, D, DV, n, rows):
    """A prompt portion (the last rows of the sequence) and single tokens against the plain form; rows of other slots and rows
    behind the sequence hold other numbers."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + n)
    q, k, v = rnd(g, n, H, D), rnd(g, n, G, D, dtype=dtype), rnd(g, n, G, DV, dtype=dtype)
    talk = torch.eye(H, dtype=F64) + rnd(g, H, H, scale=0.3)
    scale = 0.8 / math.sqrt(D)
    want = O.talking_attention(q, k, v, talk, scale)
    ck, cv = _fill_cache(k, v, 1, 3, n + 9, dtype)
    sink = torch.zeros(H, dtype=F32, device="cuda")
    first = n // 2
    tab, _ = meta_table([(1, first, n - first, 0)])
    out = torch.empty(n - first, H, DV, dtype=dtype, device="cuda")
    ops.seq_talking_attention(dev(q[first:]), ck, cv, dev(talk), out, tab, FULL, scale, sink=sink, rows_per_cta=rows)
    close(out, want[first:], dtype, scale=float(want.abs().max()))
    # rows of two sequences in one step: the second sequence's first rows sit in the CTA that holds the first one's last rows
    q2, k2, v2 = rnd(g, 9, H, D), rnd(g, 9, G, D, dtype=dtype), rnd(g, 9, G, DV, dtype=dtype)
    ck[2, :9], cv[2, :9] = dev(k2, dtype), dev(v2, dtype)
    want2 = O.talking_attention(q2, k2, v2, talk, scale)
    a = min(n, 6)
    tab, _ = meta_table([(1, n - a, a, 0), (2, 0, 9, 0)])
    out2 = torch.empty(a + 9, H, DV, dtype=dtype, device="cuda")
    ops.seq_talking_attention(dev(torch.cat([q[n - a:], q2])), ck, cv, dev(talk), out2, tab, FULL, scale, sink=sink, rows_per_cta=rows)
    close(out2[:a], want[n - a:], dtype, scale=float(want.abs().max()))
    close(out2[a:], want2, dtype, scale=float(want2.abs().max()))
    for t in (0, 1, n - 1):                                                      # the first tokens see almost nothing but the extra unit
        tab, _ = meta_table([(1, t, 1, 0)])
        out = torch.empty(1, H, DV, dtype=dtype, device="cuda")
        ops.seq_talking_attention(dev(q[t:t + 1]), ck, cv, dev(talk), out, tab, FULL, scale, sink=sink)
        close(out, want[t:t + 1], dtype, scale=float(want.abs().max()))
    # without the extra unit the weights of one token sum to one: with an identity mix the first token returns its own value
    tab, _ = meta_table([(1, 0, 1, 0)])
    out = torch.empty(1, H, DV, dtype=dtype, device="cuda")
    ops.seq_talking_attention(dev(q[:1]), ck, cv, dev(torch.eye(H, dtype=F64)), out, tab, FULL, scale, sink=None)
    close(out[0], v[0].repeat_interleave(H // G, 0), dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("decoded,rows", [(False, 4), (False, 1), (True, 1)])
def test_a_far_key_among_hundreds_is_found(dtype, decoded, rows):
    """One early key matches the last queries of one head far better than all others, and its value stands out: the output of the
    heads that listen to that head must carry it. A window argument one short of the key's distance must lose it."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(5)
    H, G, D, DV, n, far = 4, 2, 32, 16, 700, 3
    q, k, v = rnd(g, n, H, D, scale=0.3), rnd(g, n, G, D, dtype=dtype, scale=0.3), rnd(g, n, G, DV, dtype=dtype, scale=0.1)
    k[far, 1] = q[n - 1, 2].to(dtype).to(F64) * 6.0                               # head 2 reads key/value head 1
    v[far, 1] = 5.0
    talk = torch.eye(H, dtype=F64)
    talk[0, 2] = 0.5                                                             # head 0 (key/value head 0) listens to head 2
    v[far, 0] = -4.0
    want = O.talking_attention(q, k, v, talk, 1.0)
    assert float(want[n - 1, 2].mean()) > 2.0 and float(want[n - 1, 0].mean()) < -0.5
    ck, cv = _fill_cache(k, v, 0, 1, n, dtype)
    sink = torch.zeros(H, dtype=F32, device="cuda")
    toks = [n - 1] if decoded else list(range(n - 40, n))
    tab, _ = meta_table([(0, toks[0], len(toks), 0)])
    out = torch.empty(len(toks), H, DV, dtype=dtype, device="cuda")
    ops.seq_talking_attention(dev(q[toks]), ck, cv, dev(talk), out, tab, FULL, 1.0, sink=sink, rows_per_cta=rows)
    close(out, want[toks], dtype, scale=float(want[toks].abs().max()))
    ops.seq_talking_attention(dev(q[toks]), ck, cv, dev(talk), out, tab, n - 1 - far, 1.0, sink=sink, rows_per_cta=rows)   # sees far + 1 .. only
    assert float(out[-1, 2].float().mean()) < 1.0
    ops.seq_talking_attention(dev(q[toks]), ck, cv, dev(talk), out, tab, n - far, 1.0, sink=sink, rows_per_cta=rows)       # the key is the window's first
    inside = O.talking_attention(q[far:], k[far:], v[far:], talk, 1.0)                                    # the same keys, counted from the window's start
    close(out[-1], inside[-1], dtype, scale=float(want[toks].abs().max()))


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_clamped_gated_activation(dtype):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(3)
    for T, F, limit in ((5, 24, 1.5), (3, 7, 0.75), (2, 130, 7.0)):
        gu = rnd(g, T, 2 * F, dtype=dtype, scale=2.0)
        a, u = torch.clamp(gu[:, :F], max=limit), torch.clamp(gu[:, F:], -limit, limit)
        out = torch.empty(T, F, dtype=dtype, device="cuda")
        ops.seq_glu_clamp(dev(gu, dtype), out, limit)
        close(out, a * torch.sigmoid(1.702 * a) * (u + 1.0), dtype)


# ---------------------------------------------------------------------------------------------------------------------
# whole models through the scheduler
# ---------------------------------------------------------------------------------------------------------------------
def attention(heads=4, kv_heads=2, dim=16, vdim=12, scale=0.3, dims=None, base=500.0, scaling=None, v_mix=True):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix,
                                           "rot": rot}}


def delta(heads=2, kv_heads=2, dim=12, vdim=10, conv=4):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def mamba(inner=48, state=8, dt_rank=4, conv=4):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff=40, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(layers, width=64, vocab=97, eps=1e-5, logit_scale=1.5):
    return {"architecture": "Kinanex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "layers": [dict(l, mlp=l.get("mlp")) for l in layers]}


STRETCH = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
CONFIGS = {
    # all three mixers; three blending attention layers of which the first only lends its values
    "mixed": config([dict(attention(scaling=STRETCH), mlp=dense()), dict(delta(), mlp=None), dict(attention(heads=6, dim=8, dims=4), mlp=dense(ff=24)),
                     dict(mamba(), mlp=dense(ff=32, limit=0.5)), dict(delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=3), mlp=dense()),
                     dict(attention(heads=2, kv_heads=2), mlp=None)]),
    # nothing divisible by anything: one head, one key/value head for all, a convolution of one or two taps, a scan with a
    # single state, layers that open with a recurrence, an attention layer outside the blend before the blending ones, no
    # rotation at all, a unit logit scale
    "odd": config([dict(mamba(inner=50, state=1, dt_rank=3, conv=2), mlp=None),
                   dict(attention(heads=3, kv_heads=3, dim=10, vdim=6, dims=0, v_mix=False), mlp=dense(ff=13, limit=1.0)),
                   dict(delta(heads=1, kv_heads=1, dim=33, vdim=7, conv=1), mlp=None),
                   dict(attention(heads=5, kv_heads=1, dim=6, vdim=9, dims=2, base=37.0), mlp=None),
                   dict(mamba(inner=24, state=20, dt_rank=1, conv=5), mlp=dense(ff=9)),
                   dict(attention(heads=1, kv_heads=1, dim=6, vdim=9, dims=6), mlp=dense(ff=11))],
                  width=50, vocab=33, eps=1e-6, logit_scale=1.0),
    # sizes of the wide register forms: key size above 128, states spread over several lanes, values wider than one CTA's columns
    "wide": config([dict(delta(heads=2, kv_heads=1, dim=130, vdim=40, conv=2), mlp=dense(ff=64)),
                    dict(mamba(inner=136, state=40, dt_rank=8, conv=3), mlp=None),
                    dict(attention(heads=8, kv_heads=4, dim=32, vdim=32, dims=16, scaling=STRETCH, scale=0.2), mlp=None)], width=96,
                   logit_scale=0.5),
}


def build(name, dtype, seed=0, n_slots=3, max_step_tokens=64, max_seq_tokens=256):
    _cuda()
    from qspec_b200.kinanex import KinanexConfig, KinanexModel, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = KinanexConfig.from_dict(CONFIGS[name])
    w = random_weights(cfg, seed)
    model = KinanexModel(cfg, w, dtype=dtype, device="cuda", n_slots=n_slots, max_step_tokens=max_step_tokens, max_seq_tokens=max_seq_tokens)
    return CONFIGS[name], w, model, Scheduler(model)


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close_logits(got, ref, dtype, same_format=False):
    """Per position: root mean square over the vocabulary of the difference (mean taken off), relative to the spread of the
    logits. float32 against the plain implementation: rounding level. bfloat16 against the plain implementation: what an 8-bit
    mantissa leaves after six layers at this width (a wrong cache row or a lost state puts the median near 1). same_format:
    bfloat16 against bfloat16 logits of the same model fed another way."""
    ref = ref.to(F64)
    d = got.detach().cpu().to(F64) - ref
    d = d - d.mean(-1, keepdim=True)
    spread = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    rows = d.pow(2).mean(-1).sqrt() / spread
    if dtype == F32:
        assert float(rows.median()) <= 1e-5, f"median position: {float(rows.median()):.3g} of the logits' spread"
        assert float(rows.max()) <= 3e-4, f"worst position: {float(rows.max()):.3g} of the logits' spread"
        return
    bound = 1.5e-2 if same_format else 3e-2
    assert float(rows.median()) <= bound, f"median position: {float(rows.median()):.3g} of the logits' spread"
    over = float((rows > 0.1).float().mean())
    assert over <= 0.1, f"{over:.1%} of the positions are off by more than 10% of the logits' spread"


def reference_logits(name, cfg, w, toks, dtype):
    """float32: the plain implementation. bfloat16: the same weights in a second model that takes the prompt whole, after that
    has been held against the plain implementation."""
    ref = O.forward(cfg, w, toks)
    if dtype == F32:
        return ref
    _, _, _, s = build(name, dtype, max_step_tokens=256)
    whole = s.feed([("whole", toks, list(range(len(toks))))]).float().cpu()
    close_logits(whole, ref, dtype)
    return whole


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_the_plain_implementation(name, dtype):
    cfg, w, model, s = build(name, dtype, max_step_tokens=128)
    toks = tokens(70, cfg["vocab"], 1)
    lay = []
    ref = O.forward(cfg, w, toks, lay)
    got = s.feed([("a", toks, list(range(len(toks))))])
    close_logits(got, ref, dtype)
    if dtype == F32:                                       # residual stream after every layer
        meta = s.table.plan([("b", len(toks))])
        tr = []
        model.forward_batch(torch.tensor(toks, dtype=torch.int32, device="cuda"), meta, trace=tr)
        assert len(tr) == len(lay) == len(cfg["layers"])
        for a, b in zip(tr, lay):
            close(a, b, F32)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_decoding_and_portions_equal_the_whole_prompt(name, dtype):
    """Token by token from the first token on; a prompt then 40 single tokens; portions of 2, 3, 1, 7, ... tokens; a step
    longer than the model's step size (cut inside the step function)."""
    cfg, w, model, s = build(name, dtype, max_step_tokens=16)
    toks = tokens(75, cfg["vocab"], 2)
    ref = reference_logits(name, cfg, w, toks, dtype)
    schedules = {"single": [1] * len(toks), "prompt+decode": [16, 16, 3] + [1] * 40, "portions": [2, 3, 1, 7, 2, 2, 13, 5, 2, 16, 14, 8],
                 "one step": [len(toks)]}
    for label, cuts in schedules.items():
        assert sum(cuts) == len(toks)
        at, rows = 0, []
        for n in cuts:
            rows.append(s.feed([(label, toks[at:at + n], list(range(n)))]))
            at += n
        s.release(label)
        close_logits(torch.cat(rows), ref, dtype, same_format=True)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_mixed_batches_equal_each_request_alone_and_slots_are_reused(dtype):
    """Three requests of unequal length advance together -- a prompt portion next to single tokens next to a request that
    starts late in a slot another request has just given back -- and each must see what it sees alone."""
    cfg, w, model, s = build("mixed", dtype, n_slots=2, max_step_tokens=48)
    seqs = {"a": tokens(50, cfg["vocab"], 11), "b": tokens(23, cfg["vocab"], 12), "c": tokens(31, cfg["vocab"], 13)}
    alone = {}
    for rid, toks in seqs.items():
        alone[rid] = s.feed([(rid, toks, list(range(len(toks))))]).float().cpu()
        s.release(rid)
        if dtype == F32:
            close_logits(alone[rid], O.forward(cfg, w, toks), dtype)
    plan = [{"a": 7, "b": 20}, {"a": 1, "b": 1}, {"a": 30, "b": 2}, {"a": 1}, {"a": 1, "c": 9}, {"a": 2, "c": 1}, {"a": 8, "c": 21}]
    at = {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    for stepn, st in enumerate(plan):
        entries = [(rid, seqs[rid][at[rid]:at[rid] + n], list(range(n))) for rid, n in st.items()]
        out = s.feed(entries)
        o = 0
        for rid, n in st.items():
            got[rid].append(out[o:o + n].float().cpu())
            o += n
            at[rid] += n
        if stepn == 2:
            assert at["b"] == len(seqs["b"])
            s.release("b")                                  # request c takes this slot in the step after next
    for rid in seqs:
        assert at[rid] == len(seqs[rid])
        close_logits(torch.cat(got[rid]), alone[rid], dtype, same_format=True)


def test_batch_composition_changes_nothing_in_float32():
    """The same token of the same request, once alone in its step and once between two other requests: every kernel assigns work
    by position and size alone, so the logits agree to the last rounding of the vendor's matrix products."""
    cfg, w, model, s = build("odd", F32, n_slots=3, max_step_tokens=64)
    a, b, c = tokens(20, cfg["vocab"], 21), tokens(9, cfg["vocab"], 22), tokens(14, cfg["vocab"], 23)
    x = s.feed([("a", a[:19], []), ("b", b[:8], []), ("c", c[:13], [])])
    assert x.shape[0] == 0
    mixed = s.feed([("b", b[8:], [0]), ("a", a[19:], [0]), ("c", c[13:], [0])])[1].float().cpu()
    for rid in "abc":
        s.release(rid)
    s.feed([("a", a[:19], [])])
    alone = s.feed([("a", a[19:], [0])])[0].float().cpu()
    assert float((mixed - alone).abs().max()) <= 2e-5 * float(alone.abs().max())


def test_the_blend_reads_the_first_blending_layers_values_of_the_same_step():
    """With the blend weight set to one, every later blending layer attends over the first one's values only: its own value
    projection must not matter."""
    cfg, w, _, _ = build("mixed", F32)
    from qspec_b200.kinanex import KinanexConfig, KinanexModel
    from qspec_b200.scheduler import Scheduler
    w = dict(w)
    for i in (2, 5):
        w[f"l{i}.mix.vmix"] = torch.tensor(1.0, dtype=BF16)
    toks = tokens(30, cfg["vocab"], 4)

    def run(weights):
        m = KinanexModel(KinanexConfig.from_dict(cfg), weights, dtype=F32, device="cuda", n_slots=1, max_step_tokens=8, max_seq_tokens=64)
        return Scheduler(m).feed([("a", toks, list(range(30)))]).float().cpu()

    base = run(w)
    close_logits(base, O.forward(cfg, w, toks), F32)
    w2 = dict(w)
    w2["l5.mix.v"] = w["l5.mix.v"] * 3.0
    assert float((run(w2) - base).abs().max()) <= 1e-4 * float(base.abs().max())
    w3 = dict(w)
    w3["l0.mix.v"] = w["l0.mix.v"].flip(0)
    assert float((run(w3) - base).abs().max()) > 1e-2 * float(base.abs().max())


def test_the_cache_bounds_the_sequence_and_the_scheduler_refuses_more():
    cfg, w, model, s = build("mixed", BF16, max_seq_tokens=40)
    s.feed([("a", tokens(40, cfg["vocab"], 5), [39])])
    with pytest.raises(RuntimeError):
        s.feed([("a", [1], [0])])


def test_long_decoding():
    """A short prompt, then 400 single tokens: the recurrences' states and the growing cache against the plain implementation."""
    cfg, w, model, s = build("mixed", F32, max_step_tokens=8, max_seq_tokens=512)
    toks = tokens(420, cfg["vocab"], 6)
    ref = O.forward(cfg, w, toks)
    rows = [s.feed([("a", toks[:20], [19])])]
    for t in range(20, 420):
        rows.append(s.feed([("a", toks[t:t + 1], [0])]))
    close_logits(torch.cat(rows), ref[19:], F32)


def test_greedy_generation_through_the_scheduler():
    cfg, w, model, s = build("mixed", F32, n_slots=2, max_step_tokens=16)
    prompts = [tokens(9, cfg["vocab"], 31), tokens(21, cfg["vocab"], 32), tokens(3, cfg["vocab"], 33)]
    outs = s.generate(prompts, 6)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in o:
            lg = O.forward(cfg, w, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(lg.abs().max()):     # a near tie may fall either way
                assert int(torch.argmax(lg)) == t
            seq.append(t)


def test_checkpoint_folder_through_the_registry_and_the_trace_replay(tmp_path):
    """config.json + model.safetensors -> registry -> the replay program's main(): logits of a recorded schedule on disk."""
    _cuda()
    import io
    import sys
    import numpy as np
    from qspec_b200 import registry
    from qspec_b200.checkpoint import write_safetensors_file
    from qspec_b200.kinanex import KinanexConfig, random_weights
    from qspec_b200.trace import main
    cfg = CONFIGS["odd"]
    w = random_weights(KinanexConfig.from_dict(cfg), 3)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors_file(str(tmp_path / "model.safetensors"), w)
    assert type(registry.load_model(str(tmp_path), dtype="float32", n_slots=1, max_step_tokens=8, max_seq_tokens=32)).__name__ == "KinanexModel"
    toks = tokens(24, cfg["vocab"], 8)
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:11], "want": [0, 10]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[11:13], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": toks[13:], "want": [10]}], "end": ["r"]},
             {"step": 3, "entries": [{"id": "s", "tokens": toks[:2], "want": [1]}], "end": ["s"]}]
    stdin, stdout = sys.stdin, sys.stdout
    sys.stdin, sys.stdout = io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), io.StringIO()
    try:
        rc = main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "out"), "--max-tokens", "32"])
        printed = sys.stdout.getvalue()
    finally:
        sys.stdin, sys.stdout = stdin, stdout
    assert rc == 0 and [l for l in printed.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    ref = O.forward(cfg, w, toks)
    assert not os.path.exists(tmp_path / "out" / "1.f32")
    for step, rows in ((0, [0, 10]), (2, [23]), (3, [1])):
        got = torch.from_numpy(np.fromfile(tmp_path / "out" / f"{step}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"]))
        close_logits(got, ref[rows], F32)

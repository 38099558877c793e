"""Repepel on the GPU against the plain CPU restatement (oracle/repepel_oracle.py): every mechanism alone, then whole models
through the scheduler's step function -- whole prompts, token-by-token decoding, portions down to two tokens, mixed batches,
reused slots, keys far back in the cache, other sizes, long decoding and greedy generation."""
import json
import math
import os

import pytest
import torch

from oracle import repepel_oracle as O

pytestmark = pytest.mark.gpu

F32, BF16, F64 = torch.float32, torch.bfloat16, torch.float64
FULL = 1 << 30


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from qspec_b200.build import build_seq_library
    build_seq_library()


def meta_table(segments):
    """segments: (slot, first position, count, phase) -> int32 [5, ntok] on the device."""
    rows = [[], [], [], [], []]
    at = 0
    for slot, p0, n, phase in segments:
        for k in range(n):
            for r, v in zip(rows, (slot, p0 + k, at, at + n, phase)):
                r.append(v)
        at += n
    return torch.tensor(rows, dtype=torch.int32, device="cuda")


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


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("W,parts,shared,mult,offset", [(96, 1, False, 0.5, 1.0), (257, 3, True, 0.25, 1.0), (40, 2, False, 1.0, 0.0),
                                                         (1030, 1, True, 2.0, 1.0), (64, 0, False, 1.0, 1.0)])
def test_scaled_residual_sum_and_input_norm(dtype, W, parts, shared, mult, offset):
    """r = x + mult * (weighted parts + weighted extra part), then the norm of r with a weight stored around `offset`."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W + parts)
    T, eps = 9, 1e-5
    x = rnd(g, T, W, scale=3.0)
    y = rnd(g, T, max(parts, 1), W, dtype=dtype)
    yw = rnd(g, T, max(parts, 1)).abs()
    y2, y2w = rnd(g, T, W, dtype=dtype), rnd(g, T, 3).abs()              # the extra part's weights: a strided column
    w = rnd(g, W, scale=0.2)
    v = torch.zeros(T, W, dtype=F64)
    if parts == 1:
        v = v + y[:, 0]
    elif parts > 1:
        v = v + (y * yw[:, :, None]).sum(1)
    if shared:
        v = v + y2 * y2w[:, 1:2]
    r = x + mult * v
    want = O.unit_rms(r, eps) * (offset + w)
    xo = x.float().cuda()
    out = torch.empty(T, W, dtype=dtype, device="cuda")
    ya = None if parts == 0 else (y.to(dtype).cuda() if parts > 1 else y[:, 0].to(dtype).cuda().contiguous())
    y2wd = y2w.float().cuda()
    ops.seq_residual_norm(xo, w.float().cuda(), eps, y=ya, y_w=yw.float().cuda() if parts > 1 else None,
                          y2=y2.to(dtype).cuda() if shared else None, y2_w=y2wd[:, 1] if shared else None, mult=mult, w_offset=offset,
                          x_out=xo, out=out)
    close(xo, r, F32)
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("kv_rank,rot_dim,rot_dims,extra", [(16, 8, 8, 0), (10, 6, 2, 3), (130, 4, 4, 1), (24, 12, 12, 5)])
def test_latent_rows_with_interleaved_pairs(dtype, kv_rank, rot_dim, rot_dims, extra):
    """Rows [latent | rotary part | columns that do not belong to the cache]: the latent is normed, neighbours (2i, 2i + 1) of
    the rotary part turn together by far positions' angles, entries past rot_dims pass, and the query rotates alike."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(kv_rank)
    T, cap, eps, base, p0 = 11, 2000, 1e-6, 1000.0, 1290
    d = rnd(g, T, kv_rank + rot_dim + extra, dtype=dtype, scale=2.0)
    kw = rnd(g, kv_rank) + 1.0
    inv = (torch.tensor(base, dtype=F64) ** (-2.0 * torch.arange(rot_dims // 2, dtype=F64) / rot_dims)).float().cuda()
    cache = torch.full((2, cap, kv_rank + rot_dim), 7.0, dtype=dtype, device="cuda")
    ops.seq_latent_prep(d.to(dtype).cuda(), 0, kv_rank, rot_dim, None, kw.float().cuda(), inv, rot_dims, None, cache,
                        meta_table([(1, p0, T, 0)]), eps, pairing="interleaved")
    pos = torch.arange(p0, p0 + T)
    c = O.unit_rms(d[:, :kv_rank], eps) * kw
    kr = O.rotate_interleaved(d[:, kv_rank:kv_rank + rot_dim], pos, rot_dims, base)
    got = cache[1, p0:p0 + T].float().cpu()
    close(got[:, :kv_rank], c, dtype)
    close(got[:, kv_rank:], kr, dtype, scale=float(kr.abs().max()) * (8 if dtype == F32 else 1))   # float32 angles at position 1300
    assert float((cache[0].float() - 7.0).abs().max()) == 0 and float((cache[1, :p0].float() - 7.0).abs().max()) == 0
    H, D = 3, 5
    q = rnd(g, T, H, D + rot_dim, dtype=dtype)
    dst = torch.zeros(T, H, rot_dim + 2, dtype=F32, device="cuda")
    ops.seq_rotary(q.to(dtype).cuda(), D, dst[:, :, 2:], rot_dims, inv, meta_table([(0, p0, T, 0)]), pairing="interleaved")
    close(dst[:, :, 2:], O.rotate_interleaved(q[..., D:], pos, rot_dims, base), F32, scale=8 * float(q.abs().max()))
    # the halves pairing of the same entry point is another rotation
    dst2 = torch.zeros(T, H, rot_dim, dtype=F32, device="cuda")
    ops.seq_rotary(q.to(dtype).cuda(), D, dst2, rot_dims, inv, meta_table([(0, p0, T, 0)]))
    if rot_dims >= 4:
        assert float((dst2 - dst[:, :, 2:]).abs().max()) > 1e-3


def _latent_case(g, T, H, r, R, dtype):
    q = rnd(g, T, H, r + R, dtype=F32, scale=0.5)
    rows = rnd(g, T, r + R, dtype=dtype)
    gate = rnd(g, T, H + 3, dtype=dtype, scale=2.0)
    return q, rows, gate


def _latent_want(q, rows, gate, H, r, scale):
    T = q.shape[0]
    k = rows.unsqueeze(1).expand(T, H, rows.shape[1])
    o = O.causal_attention(q, k, rows[:, :r].unsqueeze(1).expand(T, H, r), scale)
    return o * torch.sigmoid(gate[:, :H]).unsqueeze(-1)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,r,R,cuts", [(3, 10, 4, [1, 1, 2, 9, 5, 2, 17, 3]), (1, 33, 6, [40]), (4, 16, 8, [2] * 20)])
def test_full_length_attention_over_a_latent_cache_with_one_gate_per_head(dtype, H, r, R, cuts):
    """The cache rows are keys ([latent | rotary part]) and values (the latent) at once; every earlier row is seen; the gate is
    one number per head. Portions write their rows first; the rest of the cache holds 1e4."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + r)
    T, cap, scale = sum(cuts), 64, 0.3
    q, rows, gate = _latent_case(g, T, H, r, R, dtype)
    want = _latent_want(q, rows, gate, H, r, scale)
    for slot in (0, 1):
        cache = torch.full((2, cap, r + R), 1e4, dtype=dtype, device="cuda")
        at, got = 0, []
        for n in cuts:
            cache[slot, at:at + n] = rows[at:at + n].to(dtype).cuda()
            qd = q[at:at + n].float().cuda()
            out = torch.empty(n, H, r, dtype=dtype, device="cuda")
            ck = cache.unsqueeze(2)
            ops.seq_window_attention(qd[:, :, :r], qd[:, :, r:], ck, ck[..., :r], out, meta_table([(slot, at, n, 0)]), FULL, scale,
                                     gate=gate[at:at + n].to(dtype).cuda(), gate_per_head=True)
            got.append(out.float().cpu())
            at += n
        close(torch.cat(got), want, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_far_key_among_hundreds_is_found(dtype, decoded):
    """Position 3 of 700 gets a key aligned with the last query and a value of its own: the last output is that value. One
    row off in the cache (or a lost early row) and the output is noise."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, H, r, R, far = 700, 2, 12, 4, 3
    q, rows, gate = _latent_case(g, T, H, r, R, dtype)
    rows = (rows * 0.1).to(dtype).to(F64)
    rows[far, :r] = 0.0
    rows[far, 0] = 3.0
    rows[far, r:] = torch.tensor([2.0, -2.0, 2.0, 2.0], dtype=F64)
    q[-1] = 0.0
    q[-1, :, 0] = 8.0                                       # 24 from the latent part
    q[-1, :, r:] = torch.tensor([4.0, -4.0, 4.0, 4.0], dtype=F64)          # 32 from the rotary part: the pair stands out by e^56
    want = _latent_want(q, rows, gate, H, r, 1.0)
    assert float((want[-1, 0] - rows[far, :r] * torch.sigmoid(gate[-1, 0])).abs().max()) < 1e-6
    cache = torch.full((1, 1024, r + R), 1e4, dtype=dtype, device="cuda")
    cache[0, :T] = rows.to(dtype).cuda()
    ck = cache.unsqueeze(2)
    first = T - 1 if decoded else T - 40
    qd = q[first:].float().cuda()
    out = torch.empty(T - first, H, r, dtype=dtype, device="cuda")
    ops.seq_window_attention(qd[:, :, :r], qd[:, :, r:], ck, ck[..., :r], out, meta_table([(0, first, T - first, 0)]), FULL, 1.0,
                             gate=gate[first:].to(dtype).cuda(), gate_per_head=True)
    close(out[-1], want[-1], dtype, scale=3.0)


@pytest.mark.parametrize("H,groups,r,n", [(16, 1, 256, 90), (32, 2, 512, 70), (5, 1, 256, 300)])
def test_absorbed_latent_attention_on_the_tensor_cores_with_head_gates(H, groups, r, n):
    """bfloat16 decoding form: 16 heads per CTA share every cache row; the per-head gate multiplies the latent output."""
    _cuda()
    from qspec_b200 import ops
    if not ops.seq_window_attention_mma_supported(BF16, r, 64, r, H, groups, False):
        pytest.skip("shape not taken by the tensor-core form")
    g = torch.Generator().manual_seed(H + r)
    R, scale, T = 64, 0.05, 6
    q, rows, gate = _latent_case(g, n, H, r, R, BF16)
    want = _latent_want(q, rows, gate, H, r, scale)[-T:]
    cache = torch.full((2, 512, r + R), 1e4, dtype=BF16, device="cuda")
    cache[1, :n] = rows.to(BF16).cuda()
    ck = cache[:, :, :r].unsqueeze(2).expand(2, 512, groups, r)
    out = torch.empty(T, H, r, dtype=BF16, device="cuda")
    # the last T positions as T single-token sequences would see them: one segment of T tokens here
    ops.seq_window_attention_mma(q[-T:].float().cuda(), ck, cache[:, :, r:], ck, out, meta_table([(1, n - T, T, 0)]), FULL, scale, False,
                                 gate=gate[-T:].to(BF16).cuda(), gate_per_head=True)
    close(out, want, BF16)


@pytest.mark.parametrize("DA,DB,DV,H,G", [(128, 64, 128, 3, 3), (128, 0, 128, 4, 2), (64, 0, 64, 2, 1)])
@pytest.mark.parametrize("pos0,T,window", [(0, 150, FULL), (37, 200, FULL), (130, 64, FULL), (90, 131, 70), (5, 1, FULL)])
def test_prompt_portion_attention_in_the_tile_form(DA, DB, DV, H, G, pos0, T, window):
    """64 tokens per CTA over key tiles of 64: portions that start anywhere, end inside a tile, a window that cuts tiles on both
    sides, a sink, one gate per head or per element; rows past the portion in the caches hold 1e4."""
    _cuda()
    from qspec_b200 import ops
    if not ops.seq_prompt_attention_mma_supported(BF16, DA, DB, DV):
        pytest.skip("shape not taken by the tile form")
    g = torch.Generator().manual_seed(DA + DB + pos0 + T)
    n, scale, cap = pos0 + T, 0.08, 400
    q = rnd(g, n, H, DA + DB, dtype=BF16, scale=1.0)
    kA, kB, v = rnd(g, n, G, DA, dtype=BF16), rnd(g, n, max(DB, 1), dtype=BF16), rnd(g, n, G, DV, dtype=BF16)
    sink = rnd(g, H)
    rep = H // G
    k = torch.cat([kA.repeat_interleave(rep, 1), kB.unsqueeze(1).expand(n, H, DB)], -1) if DB else kA.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    s = s.masked_fill(~((j <= i) & (i - j < window)), float("-inf"))
    e = torch.exp(s - s.amax(-1, keepdim=True).clamp(min=sink[:, None, None]))
    wts = e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - s.amax(-1, keepdim=True).clamp(min=sink[:, None, None])))
    o = torch.einsum("hij,jhd->ihd", wts, v.repeat_interleave(rep, 1))[pos0:]
    for per_head in (True, False):
        gate = rnd(g, T, H + 5 if per_head else H * DV + 8, dtype=BF16, scale=2.0)
        want = o * (torch.sigmoid(gate[:, :H]).unsqueeze(-1) if per_head else torch.sigmoid(gate[:, :H * DV]).view(T, H, DV))
        ck = torch.full((2, cap, G, DA), 1e4, dtype=BF16, device="cuda")
        cs = torch.full((2, cap, max(DB, 8)), 1e4, dtype=BF16, device="cuda")
        cv = torch.full((2, cap, G, DV), 1e4, dtype=BF16, device="cuda")
        ck[1, :n], cv[1, :n] = kA.to(BF16).cuda(), v.to(BF16).cuda()
        if DB:
            cs[1, :n, :DB] = kB.to(BF16).cuda()
        out = torch.empty(T, H, DV, dtype=BF16, device="cuda")
        ops.seq_prompt_attention_mma(q[pos0:].float().cuda(), ck, cs[:, :, :DB] if DB else None, cv, out, 1, pos0, window, scale,
                                     sink=sink.float().cuda(), gate=gate.to(BF16).cuda(), gate_per_head=per_head)
        close(out, want, BF16)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,D,DV", [(2, 16, 24), (1, 33, 7), (3, 130, 40), (2, 64, 64)])
def test_linear_attention_state_over_portions_and_slots(dtype, H, D, DV):
    """Portions of 1 to 17 tokens in two slots with NaN-filled state; decays from fast to none at all; the grid with one CTA
    per segment and the one per token agree."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(H * 7 + D)
    cuts = [1, 2, 1, 17, 3, 16, 5]
    T, eps = sum(cuts), 1e-5
    decay = [0.5, 1.0, 0.97][:H]
    p = rnd(g, T, 2 * H * (D + DV) + 2, dtype=dtype)
    other = rnd(g, 11, 2 * H * (D + DV) + 2, dtype=dtype)
    nw = rnd(g, H * DV) + 1.0
    HD, HDV = H * D, H * DV
    q, k = O.silu(p[:, :HD]).view(T, H, D), O.silu(p[:, HD:2 * HD]).view(T, H, D)
    v = O.silu(p[:, 2 * HD:2 * HD + HDV]).view(T, H, DV)
    o = O.linear_attention(q, k, v, decay).reshape(T, HDV)
    want = O.unit_rms(o, eps) * nw * torch.sigmoid(p[:, 2 * HD + HDV:2 * HD + 2 * HDV])
    dec = torch.tensor(decay, dtype=F32, device="cuda")
    for with_starts in (True, False):
        state = torch.full((3, H, D, DV), float("nan"), dtype=F32, device="cuda")
        at, got = 0, []
        for j, n in enumerate(cuts):
            # a neighbour sequence in slot 0 shares every other step (it starts over each time: position 0)
            both = j % 2 == 1
            rows = torch.cat([other, p[at:at + n]]) if both else p[at:at + n]
            segs = ([(0, 0, 11, 0)] if both else []) + [(2, at, n, 0)]
            meta = meta_table(segs)
            nt = rows.shape[0]
            out = torch.empty(nt, HDV, dtype=dtype, device="cuda")
            scratch = torch.empty(nt * H * (DV + 2 * D), dtype=F32, device="cuda")
            starts = torch.tensor([0, 11] if both else [0], dtype=torch.int32, device="cuda") if with_starts else None
            ops.seq_lightning(rows.to(dtype).cuda(), dec, nw.float().cuda(), state, scratch, out, meta, H, D, DV, eps, seg_starts=starts)
            got.append(out[-n:].float().cpu())
            at += n
        close(torch.cat(got), want, dtype)


@pytest.mark.parametrize("E,top,count,keep", [(20, 3, 2, 1), (12, 3, 4, 2), (8, 8, 1, 1), (9, 1, 3, 1), (6, 2, 6, 2), (64, 6, 8, 3)])
def test_sigmoid_router_with_expert_groups(E, top, count, keep):
    """Choice = sigmoid score + correction, corrections large and negative enough that choice scores go below zero (a dropped
    group must count as minus infinity, not as zero); weights are the plain scores times the scale; the gate row behind the
    router's rows comes out as its sigmoid."""
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(E + top)
    T, W, scale = 40, 48, 2.5
    h = rnd(g, T, W)
    rw = rnd(g, E + 1, W, scale=0.3)
    corr = rnd(g, E, scale=0.8) - 1.0
    s = torch.sigmoid(h @ rw[:E].T)
    idx_w, wt_w = O.choose_experts(s, corr, top, count, keep, scale)
    for dtype in (F32, BF16):
        hd = h.to(dtype)
        s2 = torch.sigmoid(hd.to(F64) @ rw[:E].T)
        idx_w, wt_w = O.choose_experts(s2, corr, top, count, keep, scale)
        idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
        wt = torch.empty(T, top, dtype=F32, device="cuda")
        buf = torch.zeros(T, 3, dtype=F32, device="cuda")
        ops.moe_route_grouped(hd.cuda(), rw.float().cuda(), corr.float().cuda(), idx, wt, score="sigmoid", groups=count, keep=keep,
                              group_top=2, scale=scale, extra=buf[:, 1:2])
        assert torch.equal(idx.cpu().long(), idx_w)
        close(wt, wt_w, F32)
        close(buf[:, 1], torch.sigmoid(hd.to(F64) @ rw[E]), F32)
        assert float(buf[:, 0].abs().max()) == 0 and float(buf[:, 2].abs().max()) == 0
        size = E // count
        if keep == 1 and count > 1:
            assert all(len({int(e) // size for e in row}) == 1 for row in idx.cpu().tolist())


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("W,F,E,top", [(64, 24, 5, 3), (72, 10, 3, 1), (128, 64, 9, 2)])
def test_silu_gated_experts_in_both_forms(dtype, W, F, E, top):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(W + F)
    T = 70
    h = rnd(g, T, W, dtype=dtype)
    gu, dn = rnd(g, E, 2 * F, W, dtype=dtype, scale=W ** -0.5), rnd(g, E, W, F, dtype=dtype, scale=F ** -0.5)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    want = torch.zeros(T, top, W, dtype=F64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            want[t, k] = dn[e] @ (O.silu(gu[e, :F] @ h[t]) * (gu[e, F:] @ h[t]))
    out = torch.empty(T, top, W, dtype=dtype, device="cuda")
    args = (h.to(dtype).cuda(), gu.to(dtype).cuda(), dn.to(dtype).cuda(), idx.cuda(), out, E, F, 0.0)
    ops.moe_expert_tokens(*args, act="silu")
    close(out, want, dtype)
    if dtype == BF16 and ops.moe_expert_grouped_supported(args[0], F):
        out.zero_()
        ops.moe_expert_grouped(*args, act="silu")
        close(out, want, dtype)
        assert ops.moe_grouped_status() == 0


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_exact_gelu_and_silu_product(dtype):
    _cuda()
    from qspec_b200 import ops
    g = torch.Generator().manual_seed(3)
    a = rnd(g, 37, 50, dtype=dtype, scale=3.0)
    d = a.to(dtype).cuda()
    ops.seq_act(d, "gelu_erf")
    close(d, O.gelu_erf(a), dtype)
    tanh_form = 0.5 * a * (1 + torch.tanh(math.sqrt(2 / math.pi) * (a + 0.044715 * a ** 3)))
    if dtype == F32:                                        # the two forms of the GELU differ by more than the tolerance
        assert float((d.cpu().to(F64) - tanh_form).abs().max()) > 1e-4
    gu = rnd(g, 19, 2 * 23, dtype=dtype, scale=2.0)
    out = torch.empty(19, 23, dtype=dtype, device="cuda")
    ops.seq_silu_mul(gu.to(dtype).cuda(), out)
    close(out, O.silu(gu[:, :23]) * gu[:, 23:], dtype)


# ---------------------------------------------------------------------------------------------------------------------
# whole models through the scheduler
# ---------------------------------------------------------------------------------------------------------------------
def latent(heads=2, dim=8, vdim=12, rot_dim=4, rot_dims=None, kv_rank=10, scale=0.3, base=500.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "rot_dim": rot_dim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}}


def lightning(heads=2, dim=12, vdim=10, decay=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                          "decay": decay or [math.exp(-1.0 / (1 + 3 * i)) for i in range(heads)]}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=6, top=2, count=3, keep=2, scale=1.25, shared=16):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def config(layers, width=64, vocab=97, eps=1e-5, mult=0.6, loop=None):
    out = {"architecture": "Repepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": [dict(l, mlp=l.get("mlp")) for l in layers]}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CONFIGS = {
    # both mixers and both feed-forwards; the first two layers run three times, each pass with its own cache and state
    "mixed": config([dict(latent(), mlp=dense()), dict(lightning(), mlp=moe()), dict(latent(heads=3, dim=6, vdim=5), mlp=moe(shared=0)),
                     dict(lightning(heads=3, dim=8, vdim=8), mlp=None)], loop=(0, 2, 3)),
    # nothing divisible by anything, one head, top 1, one group, fewer rotated dimensions than the rotary part, no loop, a
    # multiplier of one, a looped block in the middle that runs once, a decay of exactly one
    "odd": config([dict(lightning(heads=1, dim=33, vdim=7, decay=[1.0]), mlp=moe(ff=10, experts=3, top=1, count=1, keep=1, scale=0.7, shared=5)),
                   dict(latent(heads=1, dim=6, vdim=6, rot_dim=6, rot_dims=2, kv_rank=9, base=37.0), mlp=None),
                   dict(latent(heads=5, dim=3, vdim=9, rot_dim=2, kv_rank=7), mlp=dense(ff=13))],
                  width=50, vocab=33, eps=1e-6, mult=1.0, loop=(1, 2, 1)),
    # the loop covers everything and runs twice; every expert chosen; shared expert as wide as the others
    "looped": config([dict(lightning(heads=4, dim=16, vdim=16), mlp=moe(ff=32, experts=2, top=2, count=1, keep=1, shared=32)),
                      dict(latent(heads=4, dim=16, vdim=16, rot_dim=8, kv_rank=24), mlp=moe(ff=32, experts=4, top=2, count=2, keep=1, shared=8))],
                     width=64, mult=0.7, loop=(0, 2, 2)),
    # a latent cache wide enough for the tensor-core absorbed form in bfloat16 decoding, and head sizes that take the expanded
    # form for prompt portions
    "tiles": config([dict(latent(heads=2, dim=128, vdim=128, rot_dim=64, kv_rank=256, scale=0.06), mlp=moe(ff=32, experts=4, top=2, count=2, keep=2)),
                     dict(lightning(heads=2, dim=64, vdim=64), mlp=dense(ff=64)),
                     dict(latent(heads=16, dim=8, vdim=8, rot_dim=64, kv_rank=256, scale=0.1), mlp=None)], width=64, loop=(0, 1, 2)),
}


def build(name, dtype, seed=0, n_slots=3, max_step_tokens=64, max_seq_tokens=256):
    _cuda()
    from qspec_b200.repepel import RepepelConfig, RepepelModel, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = RepepelConfig.from_dict(CONFIGS[name])
    w = random_weights(cfg, seed)
    if dtype == BF16:
        # corrections eight times as wide: the experts' choice scores lie far apart, so that bfloat16 rounding rarely flips a
        # choice (a flip replaces a token's whole feed-forward output and, through the linear-attention state, moves every later
        # position); routing that follows the input closely is what the float32 runs cover
        for k in w:
            if k.endswith("mlp.correction"):
                w[k] = (w[k].float() * 8.0).to(BF16)
    model = RepepelModel(cfg, w, dtype=dtype, device="cuda", n_slots=n_slots, max_step_tokens=max_step_tokens, max_seq_tokens=max_seq_tokens)
    return CONFIGS[name], w, model, Scheduler(model)


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close_logits(got, ref, dtype, same_format=False):
    """Per position: root mean square over the vocabulary of the difference (mean taken off), relative to the spread of the
    logits. float32 against the plain implementation: rounding level. bfloat16 against the plain implementation: what an 8-bit
    mantissa leaves after up to eight layer runs at width 64 (measured: 0.6 to 1.6 % at the median position; a wrong cache row
    or a lost state puts the median near 1), with few positions far off where a router choice still flips. same_format:
    bfloat16 against bfloat16 logits of the same model fed another way -- the same kernels per token agree to float32
    rounding of the logits; where the step's shape selects another kernel form, to bfloat16 rounding."""
    ref = ref.to(F64)
    d = got.detach().cpu().to(F64) - ref
    d = d - d.mean(-1, keepdim=True)
    spread = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    rows = d.pow(2).mean(-1).sqrt() / spread
    if dtype == F32:
        # the worst may be a token whose linear-attention output is tiny before its norm (q.k of the first token cancels to
        # 1e-3 of its terms with some seeds), which multiplies float32 rounding by 1e3
        assert float(rows.median()) <= 1e-5, f"median position: {float(rows.median()):.3g} of the logits' spread"
        assert float(rows.max()) <= 3e-4, f"worst position: {float(rows.max()):.3g} of the logits' spread"
        return
    over = float((rows > 0.1).float().mean())
    bound = 1.5e-2 if same_format else 2.5e-2
    assert float(rows.median()) <= bound, f"median position: {float(rows.median()):.3g} of the logits' spread"
    assert over <= 0.1, f"{over:.1%} of the positions are off by more than 10% of the logits' spread"


def reference_logits(name, cfg, w, toks, dtype):
    """float32: the plain implementation. bfloat16: the same weights in a second model that takes the prompt whole, after that
    has been held against the plain implementation."""
    ref = O.forward(cfg, w, toks)
    if dtype == F32:
        return ref
    _, _, _, s = build(name, dtype, max_step_tokens=256)
    whole = s.feed([("whole", toks, list(range(len(toks))))]).float().cpu()
    if len(toks) >= 8:                                      # a handful of positions has no typical one
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
    if dtype == F32:                                       # residual stream after every layer run
        meta = s.table.plan([("b", len(toks))])
        tr = []
        model.forward_batch(torch.tensor(toks, dtype=torch.int32, device="cuda"), meta, trace=tr)
        assert len(tr) == len(lay) == len(O.layer_runs(cfg))
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
    """Five unequal requests on three slots: prompt portions and single tokens share steps, finished requests give their slot
    to the next one, whose cache rows and state must not show the previous owner's."""
    cfg, w, model, s = build("mixed", dtype, n_slots=3, max_step_tokens=32)
    reqs = {k: tokens(n, cfg["vocab"], 30 + n) for k, n in zip("abcde", (23, 9, 31, 2, 14))}
    got = {k: [] for k in reqs}
    fed = {k: 0 for k in reqs}
    live, waiting = [], list(reqs)
    step = 0
    while live or waiting:
        while waiting and len(live) < 3:
            live.append(waiting.pop(0))
        entries, budget = [], 32
        for k in live:
            n = min(len(reqs[k]) - fed[k], [5, 1, 2, 7][(step + ord(k)) % 4], budget)
            if n > 0:
                entries.append((k, reqs[k][fed[k]:fed[k] + n], list(range(n))))
                budget -= n
        out = s.feed(entries)
        at = 0
        for k, toks, _ in entries:
            got[k].append(out[at:at + len(toks)].clone())
            at += len(toks)
            fed[k] += len(toks)
        for k in [k for k in live if fed[k] == len(reqs[k])]:
            live.remove(k)
            s.release(k)
        step += 1
    refs = {k: reference_logits("mixed", cfg, w, toks, dtype) for k, toks in reqs.items()}
    if dtype == F32:
        for k in reqs:
            close_logits(torch.cat(got[k]), refs[k], dtype)
    else:                                                   # a request of two tokens has no typical position: all rows together
        close_logits(torch.cat([torch.cat(got[k]) for k in reqs]), torch.cat([refs[k] for k in reqs]), dtype, same_format=True)


def test_batch_composition_changes_nothing_in_float32():
    cfg, w, model, s = build("mixed", F32, n_slots=3, max_step_tokens=64)
    a, b = tokens(30, cfg["vocab"], 5), tokens(12, cfg["vocab"], 6)
    alone = s.feed([("x", a, list(range(30)))]).clone()
    s.release("x")
    s.feed([("y", b[:5], [])])
    both = s.feed([("y", b[5:], []), ("x", a, list(range(30)))]).clone()
    # identical kernels per token; only the vendor library's products may sum in another order for another row count
    spread = float((alone - alone.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    assert float((alone - both).abs().max()) <= 1e-4 * spread


def test_prompt_and_decode_forms_on_the_tensor_cores_match_the_plain_implementation():
    """bfloat16 at sizes the tensor-core forms take: a prompt portion of 96 tokens (expanded keys and values, grouped experts), a
    second portion on top of it, then single tokens (absorbed form) next to a neighbour that is still in its prompt."""
    cfg, w, model, s = build("tiles", BF16, n_slots=2, max_step_tokens=128, max_seq_tokens=512)
    toks = tokens(240, cfg["vocab"], 8)
    ref = O.forward(cfg, w, toks)
    rows = [s.feed([("a", toks[:96], list(range(96)))]), s.feed([("a", toks[96:200], list(range(104)))])]
    other = tokens(40, cfg["vocab"], 9)
    s.feed([("n", other[:3], [])])
    for j, t in enumerate(toks[200:]):
        rows.append(s.feed([("n", [other[3 + j % 30]], []), ("a", [t], [0])]))
    close_logits(torch.cat(rows), ref, BF16)
    from qspec_b200 import ops
    assert ops.moe_grouped_status() == 0


def test_prompt_portions_in_the_tile_form_inside_the_model():
    """The same model with the tile form of the prompt attention switched on for short portions: a first portion, a second one
    that starts inside a key tile, then decoding; against the plain implementation and against the 16-token form."""
    cfg, w, model, s = build("tiles", BF16, n_slots=2, max_step_tokens=160, max_seq_tokens=512)
    toks = tokens(230, cfg["vocab"], 11)
    ref = O.forward(cfg, w, toks)
    outs = {}
    for label, ctas in (("tiles", 1), ("rows16", 1 << 30)):
        model.prompt_tiles_min_ctas = ctas
        rows = [s.feed([(label, toks[:130], list(range(130)))]), s.feed([(label, toks[130:210], list(range(80)))])]
        rows += [s.feed([(label, [t], [0])]) for t in toks[210:]]
        s.release(label)
        outs[label] = torch.cat(rows)
        close_logits(outs[label], ref, BF16)
    d = (outs["tiles"] - outs["rows16"]).float()
    spread = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    assert float(d.pow(2).mean(-1).sqrt().median()) <= 1e-2 * spread


def test_the_cache_bounds_the_sequence_and_the_scheduler_refuses_more():
    cfg, w, model, s = build("odd", F32, n_slots=2, max_step_tokens=16, max_seq_tokens=90)
    assert model.max_seq_len == 90 and all(c.shape[1] == 90 for c in model.latent_cache.values())
    toks = tokens(90, cfg["vocab"], 4)
    rows = [s.feed([("a", toks[:50], list(range(50)))])] + [s.feed([("a", [t], [0])]) for t in toks[50:]]
    close_logits(torch.cat(rows), O.forward(cfg, w, toks), F32)
    with pytest.raises(RuntimeError):
        s.feed([("a", [1], [0])])


def test_long_decoding():
    cfg, w, model, s = build("mixed", F32, max_step_tokens=4)
    toks = tokens(170, cfg["vocab"], 7)
    ref = O.forward(cfg, w, toks)
    rows = [s.feed([("a", toks[:3], [0, 1, 2])])]
    for t in toks[3:]:
        rows.append(s.feed([("a", [t], [0])]))
    close_logits(torch.cat(rows), ref, F32)


def test_every_pass_of_the_loop_has_a_state_of_its_own():
    cfg, w, model, s = build("mixed", F32)
    runs = O.layer_runs(cfg)
    assert runs == [0, 1, 0, 1, 0, 1, 2, 3] and model.runs == runs
    assert sorted(model.latent_cache) == [0, 2, 4, 6] and sorted(model.rec_state) == [1, 3, 5, 7]
    assert len({t.data_ptr() for t in list(model.latent_cache.values()) + list(model.rec_state.values())}) == 8


def test_greedy_generation_through_the_scheduler():
    cfg, w, model, s = build("mixed", F32, n_slots=2, max_step_tokens=16)
    prompts = [tokens(n, cfg["vocab"], 20 + n) for n in (5, 19, 2, 11)]
    outs = s.generate(prompts, 6)
    for p, o in zip(prompts, outs):
        assert o == O.greedy(cfg, w, p, 6)


def test_checkpoint_folder_through_the_registry_and_the_trace_replay(tmp_path):
    _cuda()
    from qspec_b200 import registry
    from qspec_b200.checkpoint import write_safetensors_file
    from qspec_b200.repepel import RepepelConfig, random_weights
    from qspec_b200.scheduler import Scheduler
    cfg = CONFIGS["odd"]
    w = random_weights(RepepelConfig.from_dict(cfg), 4)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors_file(str(tmp_path / "model.safetensors"), w)
    model = registry.load_model(str(tmp_path), dtype="float32", n_slots=2, max_step_tokens=32, max_seq_tokens=64)
    assert model.architecture == "Repepel"
    toks = tokens(20, cfg["vocab"], 9)
    close_logits(Scheduler(model).feed([("a", toks, [0, 7, 19])]), O.forward(cfg, w, toks)[[0, 7, 19]], F32)
    # the replay program: two steps of one request, then a second request in the slot the first gave back
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:13], "want": [12]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[13:], "want": [0, 6]}], "end": ["r"]},
             {"step": 2, "entries": [{"id": "s", "tokens": toks[5:9], "want": [3]}], "end": ["s"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "40"],
                       input="\n".join(json.dumps(x) for x in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = O.forward(cfg, w, toks)
    close_logits(torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(1, -1)), ref[[12]], F32)
    close_logits(torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1)), ref[[13, 19]], F32)
    close_logits(torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)), O.forward(cfg, w, toks[5:9])[[3]], F32)

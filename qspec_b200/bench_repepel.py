"""`bench.py --design repepel`: prefill and decode throughput of the Repepel design at sizes that resemble a real model's
layers (random weights), next to Pitudra -- the framework's closest model: latent attention, a linear recurrence, mixture of
experts, float32 residual -- at equal width / heads / latent and expert sizes, both through the same scheduler; plus the
design's kernels one by one against their roofline, with Pitudra's like kernels from `bench_seq`. Prints one JSON line. The
default workload of bench.py is untouched by this option.
"""
from __future__ import annotations

import math

from .bench_seq import PITUDRA_SIZES, SIZES, VOCAB, _pitudra_kernel_table, _throughput, _time_us, pitudra_config

# the sizes of `bench_seq.PITUDRA_SIZES` (width, heads x 128, latent 512 + 64, experts) with a dense feed-forward size and groups
REPEPEL_SIZES = {
    "w2048": dict(PITUDRA_SIZES["w2048"], ff=SIZES["w2048"]["ff"], groups=(4, 2), shared=1024),
    "w4096": dict(PITUDRA_SIZES["w4096"], ff=SIZES["w4096"]["ff"], groups=(4, 2), shared=2048),
}


def repepel_config(s):
    """Four layer runs: a latent layer with a dense feed-forward that runs twice, a latent layer and a linear-attention layer
    with mixtures of experts."""
    H, D = s["heads"], s["dim"]
    _, kvr, rot = s["latent"]
    E, F, top = s["moe"]
    count, keep = s["groups"]
    moe = {"kind": "moe", "expert": {"ff": F}, "shared": {"ff": s["shared"]},
           "router": {"experts": E, "top": top, "scale": 2.0, "groups": {"count": count, "keep": keep}}}
    dense = {"kind": "dense", "ff": s["ff"]}
    lat = {"heads": H, "dim": D, "vdim": D, "rot_dim": rot, "kv_rank": kvr, "scale": (D + rot) ** -0.5, "rot": {"base": 10000.0, "dims": rot}}
    lin = {"heads": H, "dim": D, "vdim": D, "decay": [math.exp(-1.0 / (4.0 * (i + 1))) for i in range(H)]}
    layers = [{"type": "latent_attention", "mixer": lat, "mlp": dense}, {"type": "latent_attention", "mixer": lat, "mlp": moe},
              {"type": "lightning", "mixer": lin, "mlp": moe}]
    return {"architecture": "Repepel", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "residual_mult": 0.7,
            "loop": {"start": 0, "stop": 1, "times": 2}, "layers": layers}


def _kernel_table(torch, s, hbm_gbs, bf16_tflops):
    """Each Repepel kernel at a prompt shape (2 048 tokens of one sequence) and a decode shape (64 sequences x 1 token with
    `window` + 300 rows behind it). frac = achieved / measured peak of the binding resource."""
    from . import ops
    dev = "cuda"
    W, H, D, ctx = s["width"], s["heads"], s["dim"], s["window"] + 300
    _, kvr, rot = s["latent"]
    E, F, top = s["moe"]
    count, keep = s["groups"]
    FS, FF = s["shared"], s["ff"]
    bf, f32 = torch.bfloat16, torch.float32
    full = 1 << 30
    rows = []

    def meta(segs):
        r = [[], [], [], [], []]
        at = 0
        for slot, p0, n in segs:
            r[0] += [slot] * n; r[1] += list(range(p0, p0 + n)); r[2] += [at] * n; r[3] += [at + n] * n; r[4] += [0] * n
            at += n
        return torch.tensor(r, dtype=torch.int32, device=dev)

    def add(name, shape, us, nbytes=None, flops=None, note=None):
        e = {"kernel": name, "shape": shape, "us": round(us, 2)}
        if nbytes is not None:
            e["GBps"] = round(nbytes / us / 1e3, 1); e["frac_hbm"] = round(nbytes / us / 1e3 / hbm_gbs, 3)
        if flops is not None:
            e["TFLOPs"] = round(flops / us / 1e6, 1); e["frac_bf16"] = round(flops / us / 1e6 / bf16_tflops, 3)
        if note:
            e["note"] = note
        rows.append(e)

    nslots, cap = 64, 4096
    shapes = {"prompt": [(0, 0, 2048)], "decode": [(k, ctx - 1 + 3 * k, 1) for k in range(64)]}
    lat_cache = [torch.randn(nslots, cap, kvr + rot, device=dev).to(bf) for _ in range(2)]
    inv = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(dev)
    for label, segs in shapes.items():
        T = sum(n for _, _, n in segs)
        tab = meta(segs)
        nbuf = max(2, min(8, int(200e6 / (T * W * 12)) + 1))
        x = [torch.randn(T, W, device=dev) for _ in range(nbuf)]
        y = [torch.randn(T, W, device=dev).to(bf) for _ in range(nbuf)]
        h = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(nbuf)]
        wv = torch.zeros(W, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_residual_norm(x[i], wv, 1e-5, y=y[i], mult=0.5, x_out=x[i], out=h[i]) for i in range(nbuf)])
        add("seq_residual_norm (scaled residual + next input norm + cast)", f"{label} T={T} W={W}", us, nbytes=T * W * 12)
        pair = [torch.randn(T, top, W, device=dev).to(bf) for _ in range(2)]
        rw = torch.rand(T, top + 1, device=dev)
        rwe, rws = rw[:, :top].contiguous(), rw[:, top]
        us = _time_us(torch, [lambda i=i: ops.seq_residual_norm(x[i], wv, 1e-5, y=pair[i % 2], y_w=rwe, y2=y[i], y2_w=rws,
                                                                mult=0.5, x_out=x[i], out=h[i]) for i in range(nbuf)])
        add("seq_residual_norm (weighted sum of the experts' parts + shared expert)", f"{label} T={T} top={top}+1", us, nbytes=T * W * (12 + 2 * top))
        # latent attention
        ld = kvr + rot + H
        dd = [(torch.randn(T, ld, device=dev)).to(bf) for _ in range(nbuf)]
        kw = torch.ones(kvr, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_latent_prep(dd[i], 0, kvr, rot, None, kw, inv, rot, None, lat_cache[i % 2], tab, 1e-5,
                                                              pairing="interleaved") for i in range(nbuf)])
        add("seq_latent_prep (norm + interleaved rotary + cache rows)", f"{label} T={T}", us, nbytes=T * (ld * 2 + (kvr + rot) * 2))
        q = [(torch.randn(T, H, D + rot, device=dev) * 0.3).to(bf) for _ in range(2)]
        qb = torch.empty(T, H, rot, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_rotary(q[i % 2], D, qb, rot, inv, tab, pairing="interleaved") for i in range(2)])
        add("seq_rotary (query part, interleaved)", f"{label} T={T} H={H}", us, nbytes=T * H * rot * 6)
        gate = dd[0][:, kvr + rot:]
        visible = sum(p + 1 for _, p0, n in segs for p in range(p0, p0 + n))
        if label == "prompt":
            nrows = 2048
            wuk = (torch.randn(H * D, kvr, device=dev) * kvr ** -0.5).to(bf)
            wuv = (torch.randn(H * D, kvr, device=dev) * kvr ** -0.5).to(bf)
            kmat = torch.empty(nrows, H * D, device=dev, dtype=bf)
            vmat = torch.empty(nrows, H * D, device=dev, dtype=bf)

            def expand(i):
                ring = lat_cache[i % 2][0, :nrows]
                torch.matmul(ring[:, :kvr], wuk.t(), out=kmat)
                torch.matmul(ring[:, :kvr], wuv.t(), out=vmat)
            us = _time_us(torch, [lambda i=i: expand(i) for i in range(2)])
            add("latent keys / values of the sequence's rows (2 vendor products)", f"{nrows}x{H * D}x{kvr} x 2", us, flops=4.0 * nrows * H * D * kvr)
            qfull = [torch.randn(T, H, D + rot, device=dev) * 0.3 for _ in range(2)]
            oexp = torch.empty(T, H, D, device=dev, dtype=bf)
            us = _time_us(torch, [lambda i=i: ops.seq_window_attention_mma(
                qfull[i % 2], kmat.view(1, nrows, H, D).expand(nslots, nrows, H, D), lat_cache[i % 2][:, :nrows, kvr:],
                vmat.view(1, nrows, H, D).expand(nslots, nrows, H, D), oexp, tab, full, 0.07, True, gate=gate, gate_per_head=True) for i in range(2)])
            add("seq_window_attention_mma, latent expanded form (16 tokens per CTA), causal over the whole prompt + head gate",
                f"T={T} H={H} key {D}+{rot} value {D}", us, flops=2.0 * visible * H * (2 * D + rot), note="the form before the tile form; kept for other shapes")
            us = _time_us(torch, [lambda i=i: ops.seq_prompt_attention_mma(
                qfull[i % 2], kmat.view(1, nrows, H, D).expand(nslots, nrows, H, D), lat_cache[i % 2][:, :nrows, kvr:],
                vmat.view(1, nrows, H, D).expand(nslots, nrows, H, D), oexp, 0, 0, full, 0.07, gate=gate, gate_per_head=True) for i in range(2)])
            add("seq_prompt_attention_mma, latent expanded form in tiles (64 or 128 tokens per CTA, keys through shared memory) + head gate",
                f"T={T} H={H} key {D}+{rot} value {D}", us, flops=2.0 * visible * H * (2 * D + rot))
        else:
            qabs = [torch.randn(T, H, kvr + rot, device=dev) * 0.05 for _ in range(2)]
            olat = torch.empty(T, H, kvr, device=dev, dtype=bf)
            groups = 1 if H <= 16 else H // 16

            def lat_mma(i):
                c = lat_cache[i % 2]
                k4 = c[:, :, :kvr].unsqueeze(2).expand(nslots, cap, groups, kvr)
                ops.seq_window_attention_mma(qabs[i % 2], k4, c[:, :, kvr:], k4, olat, tab, full, 0.07, False, gate=gate, gate_per_head=True)
            us = _time_us(torch, [lambda i=i: lat_mma(i) for i in range(2)])
            add("seq_window_attention_mma, latent absorbed form + head gate (16 heads per CTA)", f"64 seqs x 1, {visible // 64} keys each", us,
                nbytes=visible * (kvr + rot) * 2)
        # linear attention
        ldr = 2 * H * 2 * D
        pr = [(torch.randn(T, ldr, device=dev)).to(bf) for _ in range(nbuf)]
        state = torch.zeros(nslots, H, D, D, device=dev)
        scr = torch.empty(T * H * 3 * D, device=dev)
        orec = torch.empty(T, H * D, device=dev, dtype=bf)
        dec = torch.full((H,), 0.97, device=dev)
        nw = torch.ones(H * D, device=dev)
        starts = tab[2].unique().to(torch.int32).contiguous()
        us = _time_us(torch, [lambda i=i: ops.seq_lightning(pr[i], dec, nw, state, scr, orec, tab, H, D, D, 1e-5, seg_starts=starts)
                              for i in range(nbuf)])
        nseg = len(segs)
        add("seq_lightning (silu + scan + norm over the heads + gate)", f"{label} T={T} H={H} D={D}", us,
            nbytes=T * (ldr * 2 + H * D * 18) + (2 * nseg * H * D * D * 4 if label == "decode" else 0), flops=4.0 * T * H * D * D,
            note="sequential over a sequence's tokens: H x DV/16 CTAs per sequence" if label == "prompt" else None)
        # feed-forward pieces
        hb = [torch.randn(T, W, device=dev).to(bf) for _ in range(nbuf)]
        rwt = torch.randn(E + 1, W, device=dev) * 0.05
        corr = torch.randn(E, device=dev) * 0.1
        idx = torch.empty(T, top, dtype=torch.int32, device=dev)
        wt = torch.empty(T, top, device=dev)
        ex = torch.empty(T, 1, device=dev)
        us = _time_us(torch, [lambda i=i: ops.moe_route_grouped(hb[i], rwt, corr, idx, wt, groups=count, keep=keep, scale=2.0, extra=ex)
                              for i in range(nbuf)])
        add("moe_route_grouped (sigmoid, groups, shared gate row)", f"{label} T={T} R={E}+1", us, nbytes=T * W * 2)
        gu = [(torch.randn(E, 2 * F, W, device=dev) * W ** -0.5).to(bf) for _ in range(2)]
        dn = [(torch.randn(E, W, F, device=dev) * F ** -0.5).to(bf) for _ in range(2)]
        pr2 = torch.empty(T, top, W, device=dev, dtype=bf)
        us = _time_us(torch, [lambda i=i: ops.moe_expert_grouped(hb[i % nbuf], gu[i % 2], dn[i % 2], idx, pr2, E, F, 0.0, act="silu") for i in range(2)])
        if label == "prompt":
            add("moe_expert_grouped, silu-gated (sort + 2 tile GEMMs)", f"T={T} top={top} E={E} F={F}", us, flops=2.0 * T * top * 3 * W * F)
        else:
            touched = len(set(idx.flatten().tolist()))
            add("moe_expert_grouped, silu-gated (sort + 2 tile GEMMs)", f"T={T} top={top}, {touched} of {E} experts touched", us,
                nbytes=touched * 3 * W * F * 2)
        u = [(torch.randn(T, FF, device=dev)).to(bf) for _ in range(nbuf)]
        us = _time_us(torch, [lambda i=i: ops.seq_act(u[i], "gelu_erf") for i in range(nbuf)])
        add("seq_act (exact GELU, in place)", f"{label} T={T} ff={FF}", us, nbytes=T * FF * 4)
        g2 = [(torch.randn(T, 2 * FS, device=dev)).to(bf) for _ in range(nbuf)]
        a2 = torch.empty(T, FS, device=dev, dtype=bf)
        us = _time_us(torch, [lambda i=i: ops.seq_silu_mul(g2[i], a2) for i in range(nbuf)])
        add("seq_silu_mul (shared expert)", f"{label} T={T} F={FS}", us, nbytes=T * FS * 6)
        del x, y, h, pair, dd, q, pr, hb, gu, dn, u, g2
    return rows


def run_repepel(args, peaks, clock_sampler_cls) -> dict:
    import torch
    from . import ops
    from .build import build_seq_library
    from .pitudra import PitudraConfig, PitudraModel, random_weights as pitudra_weights
    from .repepel import RepepelConfig, RepepelModel, random_weights
    from .scheduler import Scheduler
    build_seq_library()
    torch.cuda.set_device(0)
    hbm_gbs, bf16_tflops, peak_src = peaks
    bf16_tflops = bf16_tflops or 1590.0
    names = [n for n in (args.sizes.split(",") if args.sizes else REPEPEL_SIZES) if n in REPEPEL_SIZES]
    steps, warmup = args.steps, max(3, args.warmup)
    out = {}
    sampler = clock_sampler_cls(0)
    sampler.start()
    l0 = ops.seq_launch_count()
    for name in names:
        s = REPEPEL_SIZES[name]
        ctx = s["window"] + 300
        res = {"layer_runs": 4, "sizes": {k: v for k, v in s.items()}}
        cfg = RepepelConfig.from_dict(repepel_config(s))
        model = RepepelModel(cfg, random_weights(cfg, 0), dtype=torch.bfloat16, device="cuda", n_slots=65, max_step_tokens=2048,
                             max_seq_tokens=4096 + 512)
        res["repepel"] = {p: _throughput(torch, Scheduler(model, prefill_portion=p), VOCAB, 64, ctx, 4096, p, steps, warmup) for p in (2048, 256)}
        res["repepel"]["state_bytes_per_sequence"] = model.state_bytes_per_slot()
        del model
        torch.cuda.empty_cache()
        pcfg = PitudraConfig.from_dict(pitudra_config(PITUDRA_SIZES[name]))
        pit = PitudraModel(pcfg, pitudra_weights(pcfg, 0), dtype=torch.bfloat16, device="cuda", n_slots=65, max_step_tokens=2048)
        res["pitudra"] = {p: _throughput(torch, Scheduler(pit, prefill_portion=p), VOCAB, 64, ctx, 4096, p, steps, warmup) for p in (2048, 256)}
        res["pitudra"]["state_bytes_per_sequence"] = pit.state_bytes_per_slot()
        del pit
        torch.cuda.empty_cache()
        res["kernels"] = _kernel_table(torch, s, hbm_gbs, bf16_tflops)
        res["like_kernels_pitudra"] = _pitudra_kernel_table(torch, PITUDRA_SIZES[name], hbm_gbs, bf16_tflops)
        out[name] = res
    clocks = sampler.stop()
    head = out[names[-1]]["repepel"][2048]
    return {"metric": "repepel_prefill_decode_tokens_per_s", "value": head["decode_tokens_per_s"], "unit": "tokens/s (decode, 64 sequences)",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": head["decode_ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (float32 residual, norms, scores, recurrence)", "data": "synthetic",
            "config": {"design": "repepel", "sizes": names, "weights": "random", "layer_runs": 4,
                       "l2": "kernel timings rotate buffers larger than the L2 where the kernel streams from HBM"},
            "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src},
            "gpu_launches": ops.seq_launch_count() - l0, "clocks": clocks, "results": out}

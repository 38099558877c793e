"""`bench.py --design kinanex`: prefill and decode throughput of the Kinanex design at sizes that resemble a real model's layers
(random weights), next to Pitudra -- the framework's closest model: grouped-query attention with biases and an extra term in the
softmax denominator, a matrix-state recurrence, float32 residual -- at equal width / heads / head sizes, both through the same
scheduler; plus the design's kernels one by one against their roofline, with Pitudra's like kernels from `bench_seq`. Prints one
JSON line. The default workload of bench.py is untouched by this option.
"""
from __future__ import annotations

from .bench_seq import PITUDRA_SIZES, SIZES, VOCAB, _pitudra_kernel_table, _throughput, _time_us, pitudra_config

# the sizes of `bench_seq.PITUDRA_SIZES` (width, heads x 128, key/value heads, context) with a dense feed-forward size, a scan of
# twice the width with 16 states, and delta layers with half as many query / key heads as value heads
KINANEX_SIZES = {
    "w2048": dict(PITUDRA_SIZES["w2048"], ff=SIZES["w2048"]["ff"], scan=(4096, 16, 128), conv=4),
    "w4096": dict(PITUDRA_SIZES["w4096"], ff=SIZES["w4096"]["ff"], scan=(8192, 16, 256), conv=4),
}


def kinanex_config(s):
    """Four layers: two blending attention layers with a dense feed-forward, a delta layer and a scan layer without one."""
    H, G, D = s["heads"], s["kv"], s["dim"]
    inner, N, R = s["scan"]
    dense = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    att = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "v_mix": True,
           "rot": {"base": 500000.0, "dims": D, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    layers = [{"type": "attention", "mixer": att, "mlp": dense},
              {"type": "delta", "mixer": {"heads": H, "kv_heads": H // 2, "dim": D, "vdim": D, "conv": s["conv"]}, "mlp": None},
              {"type": "attention", "mixer": att, "mlp": dense},
              {"type": "mamba1", "mixer": {"inner": inner, "state": N, "dt_rank": R, "conv": s["conv"]}, "mlp": None}]
    return {"architecture": "Kinanex", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "logit_scale": 1.0, "layers": layers}


def _kernel_table(torch, s, hbm_gbs, bf16_tflops):
    """Each Kinanex kernel at a prompt shape (2 048 tokens of one sequence) and a decode shape (64 sequences x 1 token with
    `window` + 300 rows behind it). frac = achieved / measured peak of the binding resource."""
    from . import ops
    dev = "cuda"
    W, H, G, D, ctx = s["width"], s["heads"], s["kv"], s["dim"], s["window"] + 300
    inner, N, R = s["scan"]
    taps, FF = s["conv"], s["ff"]
    GD = H // 2                                             # query / key heads of the delta layer
    bf, f32 = torch.bfloat16, torch.float32
    full = 1 << 30
    rows = []

    def meta(segs):
        r = [[], [], [], [], []]
        at, starts = 0, []
        for slot, p0, n in segs:
            starts.append(at)
            r[0] += [slot] * n; r[1] += list(range(p0, p0 + n)); r[2] += [at] * n; r[3] += [at + n] * n; r[4] += [0] * n
            at += n
        return torch.tensor(r, dtype=torch.int32, device=dev), torch.tensor(starts, dtype=torch.int32, device=dev)

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
    ck = [(torch.randn(nslots, cap, G, D, device=dev) * 0.5).to(bf) for _ in range(2)]
    cv = [(torch.randn(nslots, cap, G, D, device=dev) * 0.5).to(bf) for _ in range(2)]
    fr = (500000.0 ** (-2.0 * torch.arange(D // 2, dtype=torch.float64) / D)).float().to(dev)
    for label, segs in shapes.items():
        T = sum(n for _, _, n in segs)
        nseg = len(segs)
        tab, starts = meta(segs)
        nbuf = max(2, min(8, int(200e6 / (T * W * 12)) + 1))
        x = [torch.randn(T, W, device=dev) for _ in range(nbuf)]
        y = [torch.randn(T, W, device=dev).to(bf) for _ in range(nbuf)]
        h = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(nbuf)]
        wv, ls = torch.ones(W, device=dev), torch.rand(W, device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_residual_norm(x[i], wv, 1e-5, y=y[i], y_scale=ls, w_offset=0.0, x_out=x[i], out=h[i])
                              for i in range(nbuf)])
        add("seq_residual_norm (layer scale + residual + next input norm + cast)", f"{label} T={T} W={W}", us, nbytes=T * W * 12)
        # attention
        ld = (H + G) * D + G * D
        pp = [torch.randn(T, ld, device=dev).to(bf) for _ in range(nbuf)]
        qn = torch.ones(D, device=dev)
        qf = [torch.empty(T, H, D, device=dev) for _ in range(2)]
        vf = torch.randn(T * G * D, device=dev)
        lam = torch.tensor([0.3], device=dev)
        us = _time_us(torch, [lambda i=i: ops.seq_gqa_prep(pp[i], qn, qn, fr, D, qf[i % 2], ck[i % 2], cv[i % 2], tab, H, 1e-5, v_first_in=vf,
                                                           mix=lam) for i in range(nbuf)])
        add("seq_gqa_prep (head norms + rotary + value norm + blend + cache rows)", f"{label} T={T}", us,
            nbytes=T * (ld * 2 + H * D * 4 + 2 * G * D * 2 + G * D * 4))
        talk = (torch.eye(H, device=dev) + 0.05 * torch.randn(H, H, device=dev)).contiguous()
        sink = torch.zeros(H, device=dev)
        qs = [torch.randn(T, H, D, device=dev) * 0.3 for _ in range(2)]
        out = torch.empty(T, H, D, device=dev, dtype=bf)
        visible = sum(p + 1 for _, p0, n in segs for p in range(p0, p0 + n))
        rows_per_cta = 4 if label == "prompt" else 1            # what the model passes for these step shapes
        us = _time_us(torch, [lambda i=i: ops.seq_talking_attention(qs[i % 2], ck[i % 2], cv[i % 2], talk, out, tab, full, D ** -0.5, sink=sink,
                                                                    rows_per_cta=rows_per_cta) for i in range(2)], reps=6 if label == "prompt" else 20)
        if label == "prompt":
            add("seq_talking_attention (two passes, heads mixed after the softmax), causal over the whole prompt",
                f"T={T} H={H} G={G} key {D} value {D}", us, flops=2.0 * visible * H * (2 * D + H))
        else:
            add("seq_talking_attention (two passes, heads mixed after the softmax)", f"64 seqs x 1, {visible // 64} keys each", us,
                nbytes=visible * G * 2 * D * 2)
        # delta rule
        C = 2 * GD * D + H * D
        pr = [torch.randn(T, C + H * D, device=dev).to(bf) for _ in range(nbuf)]
        cw = torch.randn(C, taps, device=dev) * 0.5
        tail = torch.zeros(2, nslots, taps - 1, C, device=dev)
        cs = [torch.empty(T, C, device=dev) for _ in range(nbuf)]
        us = _time_us(torch, [lambda i=i: ops.seq_conv_act(pr[i][:, :C], cw, None, tail, cs[i], tab, act="silu") for i in range(nbuf)])
        add("seq_conv_act (q, k, v of the delta layer: convolution + silu, float32 out)", f"{label} T={T} C={C} taps={taps}", us, nbytes=T * C * 6)
        ba = torch.randn(T, 2 * H, device=dev)
        al, db, nw = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(D, device=dev)
        state = torch.zeros(nslots, H, D, D, device=dev)
        gates = torch.empty(T * (2 * H + GD), device=dev)
        ob = torch.empty(T * H * D, device=dev)
        od = torch.empty(T, H * D, device=dev, dtype=bf)

        def delta(i):
            ops.seq_delta_rule(cs[i], ba, al, db, nw, pr[i][:, C:], state, gates, ob, od, tab, starts, H, GD, D, D, 1e-5)
        us = _time_us(torch, [lambda i=i: delta(i) for i in range(nbuf)])
        add("seq_delta_rule (unit vectors + gates, scan, head norm + gate: 3 launches)", f"{label} T={T} H={H} D={D}", us,
            nbytes=T * (C * 8 + H * D * (4 + 4 + 2 + 2)) + (2 * nseg * H * D * D * 4 if label == "decode" else 0), flops=6.0 * T * H * D * D,
            note="sequential over a sequence's tokens: H x DV/16 CTAs per sequence" if label == "prompt" else None)
        # selective scan
        xz = [torch.randn(T, 2 * inner, device=dev).to(bf) for _ in range(nbuf)]
        cw2, cb2 = torch.randn(inner, taps, device=dev) * 0.5, torch.zeros(inner, device=dev)
        tail2 = torch.zeros(2, nslots, taps - 1, inner, device=dev)
        xc = [torch.empty(T, inner, device=dev, dtype=bf) for _ in range(nbuf)]
        us = _time_us(torch, [lambda i=i: ops.seq_conv_act(xz[i][:, :inner], cw2, cb2, tail2, xc[i], tab, act="silu") for i in range(nbuf)])
        add("seq_conv_act (scan input: convolution + bias + silu)", f"{label} T={T} C={inner} taps={taps}", us, nbytes=T * inner * 4)
        dtp = [torch.randn(T, inner, device=dev) for _ in range(nbuf)]
        bc = torch.randn(T, 2 * N, device=dev).to(bf)
        dtb, alog, dsk = torch.zeros(inner, device=dev), torch.zeros(inner, N, device=dev), torch.ones(inner, device=dev)
        st2 = torch.zeros(nslots, inner, N, device=dev)
        os_ = torch.empty(T, inner, device=dev, dtype=bf)
        us = _time_us(torch, [lambda i=i: ops.seq_selective_scan(xc[i], dtp[i], dtb, bc, xz[i][:, inner:], alog, dsk, st2, os_, tab, starts)
                              for i in range(nbuf)])
        add("seq_selective_scan (softplus, scan, skip, gate)", f"{label} T={T} inner={inner} N={N}", us,
            nbytes=T * inner * (2 + 4 + 2 + 2) + (2 * nseg * inner * N * 4 if label == "decode" else 0), flops=6.0 * T * inner * N,
            note="sequential over a sequence's tokens: inner/128 CTAs per sequence" if label == "prompt" else None)
        gu = [torch.randn(T, 2 * FF, device=dev).to(bf) for _ in range(nbuf)]
        a2 = torch.empty(T, FF, device=dev, dtype=bf)
        us = _time_us(torch, [lambda i=i: ops.seq_glu_clamp(gu[i], a2, 7.0) for i in range(nbuf)])
        add("seq_glu_clamp (clamped gated activation)", f"{label} T={T} ff={FF}", us, nbytes=T * FF * 6)
        del x, y, h, pp, pr, cs, xz, xc, dtp, gu
    return rows


def run_kinanex(args, peaks, clock_sampler_cls) -> dict:
    import torch
    from . import ops
    from .build import build_seq_library
    from .kinanex import KinanexConfig, KinanexModel, random_weights
    from .pitudra import PitudraConfig, PitudraModel, random_weights as pitudra_weights
    from .scheduler import Scheduler
    build_seq_library()
    torch.cuda.set_device(0)
    hbm_gbs, bf16_tflops, peak_src = peaks
    bf16_tflops = bf16_tflops or 1590.0
    names = [n for n in (args.sizes.split(",") if args.sizes else KINANEX_SIZES) if n in KINANEX_SIZES]
    steps, warmup = args.steps, max(3, args.warmup)
    out = {}
    sampler = clock_sampler_cls(0)
    sampler.start()
    l0 = ops.seq_launch_count()
    for name in names:
        s = KINANEX_SIZES[name]
        ctx = s["window"] + 300
        res = {"layers": 4, "sizes": {k: v for k, v in s.items()}}
        cfg = KinanexConfig.from_dict(kinanex_config(s))
        model = KinanexModel(cfg, random_weights(cfg, 0), dtype=torch.bfloat16, device="cuda", n_slots=65, max_step_tokens=2048,
                             max_seq_tokens=4096 + 512)
        res["kinanex"] = {p: _throughput(torch, Scheduler(model, prefill_portion=p), VOCAB, 64, ctx, 4096, p, steps, warmup) for p in (2048, 256)}
        res["kinanex"]["state_bytes_per_sequence"] = model.state_bytes_per_slot()
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
    head = out[names[-1]]["kinanex"][2048]
    return {"metric": "kinanex_prefill_decode_tokens_per_s", "value": head["decode_tokens_per_s"], "unit": "tokens/s (decode, 64 sequences)",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": head["decode_ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (float32 residual, norms, scores, weights, recurrences)", "data": "synthetic",
            "config": {"design": "kinanex", "sizes": names, "weights": "random", "layers": 4,
                       "l2": "kernel timings rotate buffers larger than the L2 where the kernel streams from HBM"},
            "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src},
            "gpu_launches": ops.seq_launch_count() - l0, "clocks": clocks, "results": out}

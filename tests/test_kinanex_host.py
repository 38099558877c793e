"""Host-side logic of the Kinanex design (no GPU): configuration parsing and tensor names, registry entry, the number formats
the replay program accepts, and properties of the plain implementation that the GPU tests lean on."""
import json
import math

import pytest
import torch

from oracle import kinanex_oracle as O
from qspec_b200 import registry
from qspec_b200.kinanex import KinanexConfig, random_weights, rotary_frequencies

F64 = torch.float64

ATT = {"type": "attention", "mlp": {"kind": "dense", "ff": 20, "limit": 1.5},
       "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.4, "v_mix": True,
                 "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}}}}
DEL = {"type": "delta", "mlp": None, "mixer": {"heads": 4, "kv_heads": 2, "dim": 5, "vdim": 7, "conv": 3}}
MAM = {"type": "mamba1", "mlp": None, "mixer": {"inner": 12, "state": 3, "dt_rank": 2, "conv": 2}}


def _cfg(layers, width=32, vocab=41, logit_scale=0.75):
    return {"architecture": "Kinanex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": logit_scale, "layers": layers}


def test_configuration_round_trip_and_tensor_names():
    d = _cfg([ATT, DEL, MAM, dict(ATT, mlp=None)])
    cfg = KinanexConfig.from_dict(d)
    assert KinanexConfig.from_dict(cfg.to_dict()) == cfg
    s = cfg.tensor_shapes()
    assert s["embed"] == (41, 32) and s["embed.norm"] == (32,) and s["final.norm"] == (32,) and "head" not in s
    assert s["l0.mix.q"] == (24, 32) and s["l0.mix.k.b"] == (12,) and s["l0.mix.v"] == (10, 32) and s["l0.mix.talk"] == (4, 4)
    assert s["l0.mix.q.norm"] == (6,) and s["l0.mix.vmix"] == () and s["l0.mix.o"] == (32, 20) and s["l0.ls2"] == (32,)
    assert s["l0.mlp.gate"] == (20, 32) and s["l0.mlp.down"] == (32, 20)
    assert s["l1.mix.q"] == (10, 32) and s["l1.mix.k.conv"] == (10, 3) and s["l1.mix.v.conv"] == (28, 3) and s["l1.mix.b"] == (4, 32)
    assert s["l1.mix.A_log"] == (4,) and s["l1.mix.norm"] == (7,) and s["l1.mix.g"] == (28, 32) and "l1.norm2" not in s
    assert s["l2.mix.in"] == (24, 32) and s["l2.mix.x"] == (8, 12) and s["l2.mix.dt"] == (12, 2) and s["l2.mix.A_log"] == (12, 3)
    assert s["l2.mix.conv.b"] == (12,) and s["l2.mix.D"] == (12,) and "l3.mlp.up" not in s
    assert set(random_weights(cfg)) == set(s)
    # optional keys: no rotation, no scaling, no blend, key heads default to the heads, unit logit scale
    bare = {"type": "attention", "mlp": None, "mixer": {"heads": 3, "dim": 4, "scale": 0.5}}
    c2 = KinanexConfig.from_dict({k: v for k, v in _cfg([bare]).items() if k != "logit_scale"})
    m = c2.layers[0].mixer
    assert (m.kv_heads, m.vdim, m.rot_dims, m.v_mix, m.rot_scaling, c2.logit_scale) == (3, 4, 0, False, None, 1.0)
    assert "l0.mix.vmix" not in c2.tensor_shapes()


def test_configuration_errors():
    with pytest.raises(ValueError):
        KinanexConfig.from_dict(_cfg([dict(DEL, type="conv")]))
    bad = json.loads(json.dumps(ATT))
    bad["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        KinanexConfig.from_dict(_cfg([bad]))
    bad = json.loads(json.dumps(ATT))
    bad["mixer"]["rot"]["dims"] = 8
    with pytest.raises(ValueError):
        KinanexConfig.from_dict(_cfg([bad]))
    bad = json.loads(json.dumps(ATT))
    bad["mixer"]["vdim"] = 9                                           # blending layers must agree in their value rows
    with pytest.raises(ValueError):
        KinanexConfig.from_dict(_cfg([ATT, bad]))
    bad = json.loads(json.dumps(ATT))
    bad["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError):
        KinanexConfig.from_dict(_cfg([bad]))


def test_registry_and_number_formats(tmp_path):
    assert "Kinanex" in registry.architectures()
    assert registry.supports_dtype("Kinanex", "bfloat16") and registry.supports_dtype("Kinanex", "float32")
    assert not registry.supports_dtype("Kinanex", "float16")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(_cfg([DEL]), f)
    from qspec_b200.trace import main
    assert main(["--model", str(tmp_path), "--dtype", "float16", "--out", str(tmp_path / "o")]) == 3


def test_frequency_bands():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    plain = rotary_frequencies(16, 1000.0)
    got = rotary_frequencies(16, 1000.0, sc)
    assert torch.allclose(got, torch.tensor(O.stretched_frequencies(16, 1000.0, sc), dtype=F64), rtol=1e-12)
    wl = 2 * math.pi / plain
    for f, g, l in zip(plain.tolist(), got.tolist(), wl.tolist()):
        if l < 16:
            assert g == f
        elif l > 64:
            assert g == pytest.approx(f / 8.0)
        else:
            assert f / 8.0 < g < f
    assert (wl < 16).any() and (wl > 64).any() and ((wl >= 16) & (wl <= 64)).any()


def test_plain_delta_rule_reads_after_it_writes():
    """With beta = 1, no decay and unit keys, the state returns exactly the value just written for the key just used."""
    g = torch.Generator().manual_seed(0)
    T, H, D, DV = 6, 2, 5, 3
    k = torch.randn(T, H, D, generator=g, dtype=F64)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(T, H, DV, generator=g, dtype=F64)
    o = O.delta_rule(k, k, v, torch.ones(T, H, dtype=F64), torch.ones(T, H, dtype=F64))
    assert torch.allclose(o, v, atol=1e-12)
    # carrying the state over a cut equals the whole sequence
    S = torch.zeros(H, D, DV, dtype=F64)
    q = torch.randn(T, H, D, generator=g, dtype=F64)
    beta, dec = torch.rand(T, H, generator=g, dtype=F64), torch.rand(T, H, generator=g, dtype=F64)
    whole = O.delta_rule(q, k, v, beta, dec)
    parts = torch.cat([O.delta_rule(q[:4], k[:4], v[:4], beta[:4], dec[:4], S), O.delta_rule(q[4:], k[4:], v[4:], beta[4:], dec[4:], S)])
    assert torch.allclose(whole, parts, atol=1e-12)


def test_plain_attention_weights_leave_room_for_the_extra_unit():
    p = O.sink_softmax_rows(torch.tensor([0.0, 0.0, 0.0], dtype=F64))
    assert torch.allclose(p, torch.full((3,), 0.25, dtype=F64))
    p = O.sink_softmax_rows(torch.tensor([-800.0], dtype=F64))
    assert float(p[0]) == 0.0
    p = O.sink_softmax_rows(torch.tensor([800.0, 0.0], dtype=F64))
    assert float(p[0]) == pytest.approx(1.0)


def test_plain_forward_is_causal_and_runs_every_branch():
    d = _cfg([MAM, ATT, DEL, dict(ATT, mlp=None)])
    w = random_weights(KinanexConfig.from_dict(d), 1)
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    lay = []
    full = O.forward(d, w, toks, lay)
    assert full.shape == (8, 41) and len(lay) == 4
    assert torch.allclose(O.forward(d, w, toks[:5]), full[:5], atol=1e-9)

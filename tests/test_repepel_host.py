"""Host-side logic of the Repepel design (no GPU): configuration parsing and tensor names, the order of layer runs, registry
entry, the number formats the replay program accepts, and properties of the plain implementation that the GPU tests lean on."""
import json

import pytest
import torch

from oracle import repepel_oracle as O
from qspec_b200 import registry
from qspec_b200.repepel import RepepelConfig, random_weights

F64 = torch.float64

LAT = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 20},
       "mixer": {"heads": 2, "dim": 6, "vdim": 5, "rot_dim": 4, "kv_rank": 7, "scale": 0.4, "rot": {"base": 100.0, "dims": 4}}}
LIN = {"type": "lightning", "mlp": None, "mixer": {"heads": 3, "dim": 5, "vdim": 7, "decay": [0.5, 0.9, 0.99]}}
MOE = {"kind": "moe", "expert": {"ff": 12}, "shared": {"ff": 9},
       "router": {"experts": 6, "top": 2, "scale": 1.25, "groups": {"count": 3, "keep": 2}}}


def _cfg(layers, loop=None, width=32, vocab=41, mult=0.6):
    out = {"architecture": "Repepel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": mult, "layers": layers}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


def test_configuration_round_trip_and_tensor_names():
    d = _cfg([LAT, dict(LIN, mlp=MOE), LIN], loop=(1, 3, 2))
    cfg = RepepelConfig.from_dict(d)
    assert RepepelConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.runs() == [0, 1, 2, 1, 2] == O.layer_runs(d)
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.q"] == (20, 32) and shapes["l0.mix.dkv"] == (11, 32) and shapes["l0.mix.g"] == (2, 32)
    assert shapes["l0.mix.uk"] == (12, 7) and shapes["l0.mix.uv"] == (10, 7) and shapes["l0.mlp.down"] == (32, 20)
    assert shapes["l1.mix.g"] == (21, 32) and shapes["l1.mix.norm"] == (21,) and shapes["l1.mlp.correction"] == (6,)
    assert shapes["l1.mlp.e5.gate"] == (12, 32) and shapes["l1.mlp.shared.down"] == (32, 9) and shapes["l1.mlp.shared.sg"] == (1, 32)
    assert "l2.norm2" not in shapes and "l2.mlp.up" not in shapes and shapes["final.norm"] == (32,)
    assert set(random_weights(cfg)) == set(shapes)
    # no loop, no groups, no shared expert: all optional
    plain = json.loads(json.dumps(MOE))
    del plain["shared"], plain["router"]["groups"]
    c2 = RepepelConfig.from_dict(_cfg([dict(LIN, mlp=plain)]))
    assert c2.runs() == [0] and c2.layers[0].mlp.groups == 1 and c2.layers[0].mlp.shared_ff == 0
    assert "l0.mlp.shared.sg" not in c2.tensor_shapes()
    assert RepepelConfig.from_dict(_cfg([LAT, LIN], loop=(0, 2, 0))).runs() == []


def test_configuration_errors():
    with pytest.raises(ValueError):
        RepepelConfig.from_dict(_cfg([dict(LIN, type="conv")]))
    bad = json.loads(json.dumps(LIN))
    bad["mixer"]["decay"] = [0.5]
    with pytest.raises(ValueError):
        RepepelConfig.from_dict(_cfg([bad]))
    bad = json.loads(json.dumps(MOE))
    bad["router"]["groups"] = {"count": 4, "keep": 1}                  # six experts do not form four equal groups
    with pytest.raises(ValueError):
        RepepelConfig.from_dict(_cfg([dict(LIN, mlp=bad)]))
    bad = json.loads(json.dumps(MOE))
    bad["router"]["groups"] = {"count": 3, "keep": 1}
    bad["router"]["top"] = 3                                           # more choices than the kept groups hold
    with pytest.raises(ValueError):
        RepepelConfig.from_dict(_cfg([dict(LIN, mlp=bad)]))
    with pytest.raises(ValueError):
        RepepelConfig.from_dict(_cfg([LAT], loop=(0, 2, 2)))
    odd = json.loads(json.dumps(LAT))
    odd["mixer"]["rot"]["dims"] = 3
    with pytest.raises(ValueError):
        RepepelConfig.from_dict(_cfg([odd]))


def test_registry_and_number_formats(tmp_path):
    assert "Repepel" in registry.architectures()
    assert registry.supports_dtype("Repepel", "bfloat16") and registry.supports_dtype("Repepel", "float32")
    assert not registry.supports_dtype("Repepel", "float16")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(_cfg([LIN]), f)
    from qspec_b200.trace import main
    assert main(["--model", str(tmp_path), "--dtype", "float16", "--out", str(tmp_path / "o")]) == 3


def test_plain_implementation_is_causal_and_sees_the_whole_past():
    d = _cfg([dict(LAT, mlp=None)])
    w = random_weights(RepepelConfig.from_dict(d), 3)
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 41, (60,), generator=g).tolist()
    b = list(a)
    b[4] = (b[4] + 1) % 41
    la, lb = O.forward(d, w, a), O.forward(d, w, b)
    assert torch.equal(la[:4], lb[:4])
    assert float((la[59] - lb[59]).abs().max()) > 1e-9                 # token 4 is still seen 55 positions later


def test_plain_recurrence_decays_per_head():
    q = torch.ones(30, 2, 1, dtype=F64)
    k = torch.zeros(30, 2, 1, dtype=F64)
    k[0] = 1.0
    o = O.linear_attention(q, k, torch.ones(30, 2, 1, dtype=F64), [0.5, 1.0])
    assert abs(float(o[10, 0, 0]) - 0.5 ** 10) < 1e-15 and float(o[29, 1, 0]) == 1.0


def test_interleaved_pairs_turn_together():
    x = torch.zeros(3, 6, dtype=F64)
    x[:, 0] = 1.0                                                       # entry 0 leaks into entry 1 only
    r = O.rotate_interleaved(x, torch.tensor([0, 1, 2]), 4, 10.0)
    assert torch.equal(r[0], x[0]) and abs(float(r[1, 1]) - torch.sin(torch.tensor(1.0, dtype=F64)).item()) < 1e-15
    assert float(r[:, 2:].abs().max()) == 0.0
    y = torch.zeros(2, 6, dtype=F64)
    y[:, 4] = 3.0                                                       # past the rotated dimensions: unchanged
    assert torch.equal(O.rotate_interleaved(y, torch.tensor([5, 9]), 4, 10.0), y)


def test_dropped_groups_count_as_minus_infinity():
    """All choice scores negative: the best group still provides the choices; a dropped group's zero would win otherwise."""
    s = torch.tensor([[0.10, 0.20, 0.30, 0.05]], dtype=F64)
    corr = torch.tensor([-1.0, -1.0, -1.0, -1.0], dtype=F64)
    idx, wt = O.choose_experts(s, corr, 2, 2, 1, 2.0)
    assert idx.tolist() == [[2, 3]] and torch.allclose(wt, torch.tensor([[0.6, 0.1]], dtype=F64))
    idx, _ = O.choose_experts(s, corr, 2, 1, 1, 1.0)
    assert idx.tolist() == [[2, 1]]

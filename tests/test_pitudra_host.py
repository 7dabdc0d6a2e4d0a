"""Host-side logic of the Pitudra design (no GPU): configuration parsing and tensor names, registry entry, the number
formats the replay program accepts, and properties of the plain implementation that the GPU tests lean on."""
import json

import pytest
import torch

from oracle import pitudra_oracle as O
from qspec_b200 import registry
from qspec_b200.pitudra import PitudraConfig, random_weights


def _cfg(layers, side=4, width=32, vocab=41):
    out = {"architecture": "Pitudra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": layers}
    if side:
        out["token_side"] = {"dim": side}
    return out


LAT = {"type": "latent_attention", "mlp": None,
       "mixer": {"heads": 2, "dim": 6, "vdim": 5, "rot_dim": 4, "q_rank": 9, "kv_rank": 7, "scale": 0.4, "mask": {"size": 5},
                 "rot": {"base": 100.0, "dims": 4}}}
ATT = {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 3, "top": 2}},
       "mixer": {"heads": 4, "kv_heads": 2, "dim": 4, "vdim": 6, "scale": 0.5, "mask": {"size": 3}}}
REC = {"type": "hgrn2", "mlp": None, "mixer": {"heads": 2, "dim": 5, "vdim": 7}}


def _borrow(window):
    l = json.loads(json.dumps(LAT))
    l["mixer"]["kv_from"] = 0
    l["mixer"]["mask"]["size"] = window
    return l


def test_configuration_round_trip_and_tensor_names():
    d = _cfg([LAT, _borrow(9), REC, ATT])
    cfg = PitudraConfig.from_dict(d)
    assert PitudraConfig.from_dict(cfg.to_dict()) == cfg
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.dkv"] == (11, 32) and "l1.mix.dkv" not in shapes and shapes["l1.mix.uk"] == (12, 7)
    assert shapes["l2.mix.lower"] == (10,) and shapes["l3.mix.q.norm"] == (16,) and shapes["l3.mix.k.b"] == (8,)
    assert "l2.norm2" not in shapes and shapes["l3.mlp.e2.down"] == (32, 12) and shapes["side.embed"] == (41, 16)
    assert set(random_weights(cfg)) == set(shapes)
    assert "side.embed" not in PitudraConfig.from_dict(_cfg([REC], side=0)).tensor_shapes()


def test_configuration_errors():
    bad = _borrow(5)
    bad["mixer"]["kv_rank"] = 8
    with pytest.raises(ValueError):
        PitudraConfig.from_dict(_cfg([LAT, bad]))
    with pytest.raises(ValueError):
        PitudraConfig.from_dict(_cfg([_borrow(5), LAT]))                 # borrows from itself / a later layer
    with pytest.raises(ValueError):
        PitudraConfig.from_dict(_cfg([REC, _borrow(5)]))                 # the named layer has no latent cache
    with pytest.raises(ValueError):
        PitudraConfig.from_dict(_cfg([dict(ATT, type="conv")]))
    odd = json.loads(json.dumps(ATT))
    odd["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        PitudraConfig.from_dict(_cfg([odd]))


def test_registry_and_number_formats(tmp_path):
    assert "Pitudra" in registry.architectures()
    assert registry.supports_dtype("Pitudra", "bfloat16") and registry.supports_dtype("Pitudra", "float32")
    assert not registry.supports_dtype("Pitudra", "float16")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(_cfg([REC]), f)
    from qspec_b200.trace import main
    assert main(["--model", str(tmp_path), "--dtype", "float16", "--out", str(tmp_path / "o")]) == 3


def test_plain_implementation_is_causal_and_window_local():
    """One attention layer: token j reaches position i through key j or, by the token shift, key j + 1; so it is felt up
    to i = j + window and not beyond. Later tokens never change earlier logits."""
    att = json.loads(json.dumps(ATT))
    att["mlp"] = None
    d = _cfg([att], side=0)
    w = random_weights(PitudraConfig.from_dict(d), 3)
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 41, (14,), generator=g).tolist()
    b = list(a)
    b[4] = (b[4] + 1) % 41
    la, lb = O.forward(d, w, a), O.forward(d, w, b)
    window = att["mixer"]["mask"]["size"]
    assert torch.equal(la[:4], lb[:4])
    assert float((la[4 + window] - lb[4 + window]).abs().max()) > 1e-6
    assert torch.equal(la[4 + window + 1:], lb[4 + window + 1:])


def test_plain_recurrence_carries_the_first_token_to_the_end():
    d = _cfg([REC], side=0)
    w = random_weights(PitudraConfig.from_dict(d), 1)
    a = [3] * 30
    b = [4] + [3] * 29
    assert float((O.forward(d, w, a)[-1] - O.forward(d, w, b)[-1]).abs().max()) > 1e-9


def test_sink_softmax_weights():
    s = torch.zeros(1, 4, 4, dtype=torch.float64)
    w = O.windowed_sink_softmax(s, torch.tensor([0.0], dtype=torch.float64), 2)
    assert torch.allclose(w[0, 0], torch.tensor([0.5, 0, 0, 0], dtype=torch.float64))
    assert torch.allclose(w[0, 3], torch.tensor([0, 0, 1 / 3, 1 / 3], dtype=torch.float64))


def test_step_table_lists_the_segments_first_rows():
    from qspec_b200.state import SequenceTable
    t = SequenceTable(4, "cpu", 64)
    m = t.plan([("a", 5), ("b", 1), ("c", 7)], list(range(13)))
    assert m.seg_starts.tolist() == [0, 5, 6] and m.table[2].tolist() == [0] * 5 + [5] + [6] * 7
    t.commit(m)
    m = t.plan([("b", 3)])
    assert m.seg_starts.tolist() == [0] and m.pos.tolist() == [1, 2, 3]

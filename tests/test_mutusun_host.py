"""Host-side logic of the sequence models (no GPU): configuration, checkpoint files, registry, slot table, the step
function's cutting of long steps, and the plain implementation's own invariants."""
import json

import pytest
import torch

from oracle import mutusun_oracle as O
from qspec_b200 import registry
from qspec_b200.checkpoint import read_safetensors_file, write_safetensors_file
from qspec_b200.mutusun import MutusunConfig, random_weights
from qspec_b200.scheduler import Scheduler
from qspec_b200.state import SequenceTable, SlotPool

CFG = {"architecture": "Mutusun", "vocab": 31, "width": 16, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
       "layers": [
           {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 4, "scale": 0.25, "softcap": 10.0, "mask": {"size": 6}},
            "mlp": {"kind": "dense", "ff": 20}},
           {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 8, "scale": 0.5, "softcap": 10.0, "mask": {"size": 4}},
            "mlp": {"kind": "moe", "expert": {"ff": 6, "limit": 1.0}, "router": {"experts": 3, "identity": 2, "top": 2}}},
           {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 8, "scale": 0.5, "softcap": 10.0, "mask": {"size": 4}},
            "mlp": {"kind": "moe", "expert": {"ff": 6, "limit": 1.0}, "router": {"experts": 3, "identity": 2, "top": 2}}, "weights_of": 1},
           {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "softcap": 0, "mask": {"size": 3}},
            "mlp": None}]}


def test_config_round_trip_and_tensor_names():
    cfg = MutusunConfig.from_dict(CFG)
    assert MutusunConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.layers[2].weights_of == 1 and cfg.layers[3].mlp is None and cfg.layers[3].mixer.softcap == 0.0
    names = cfg.tensor_shapes()
    assert names["l0.mix.q"] == (16, 16) and names["l0.mix.k"] == (8, 16) and names["l0.mix.v"] == (4, 16)
    assert names["l1.mlp.router"] == (5, 16) and names["l1.mlp.e2.down"] == (16, 6) and names["l1.canon2"] == (16, 3)
    assert not any(n.startswith("l2.") for n in names) and "l3.norm2" not in names
    with pytest.raises(ValueError):
        MutusunConfig.from_dict({**CFG, "layers": [{**CFG["layers"][0], "type": "recurrent"}]})


def test_safetensors_round_trip(tmp_path):
    w = random_weights(MutusunConfig.from_dict(CFG), 1)
    w["table"] = torch.arange(6, dtype=torch.int32).view(2, 3)
    write_safetensors_file(str(tmp_path / "m.safetensors"), w)
    back = read_safetensors_file(str(tmp_path / "m.safetensors"))
    assert set(back) == set(w)
    for k in w:
        assert back[k].dtype == w[k].dtype and torch.equal(back[k], w[k])


def test_registry_knows_the_architectures(tmp_path):
    assert {"Mutusun", "LlamaForCausalLM", "Qwen2ForCausalLM"} <= set(registry.architectures())
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert registry.architecture_of(registry.read_config(str(tmp_path))) == "Mutusun"
    assert registry.supports_dtype("Mutusun", "float32") and registry.supports_dtype("Mutusun", "bfloat16")
    assert not registry.supports_dtype("LlamaForCausalLM", "float32")
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nothing"}))
    with pytest.raises(ValueError):
        registry.load_model(str(tmp_path))


def test_slot_pool_and_sequence_table():
    pool = SlotPool(2)
    a, b = pool.alloc(), pool.alloc()
    with pytest.raises(RuntimeError):
        pool.alloc()
    pool.release(a)
    assert pool.alloc() == a
    with pytest.raises(ValueError):
        pool.release(5)
    t = SequenceTable(2, "cpu", 16)
    m = t.plan([("x", 3), ("y", 2)])
    assert m.table.tolist() == [[0, 0, 0, 1, 1], [0, 1, 2, 0, 1], [0, 0, 0, 3, 3], [3, 3, 3, 5, 5], [0, 0, 0, 0, 0]]
    t.commit(m)
    m = t.plan([("y", 1)])
    assert m.table[:, 0].tolist() == [1, 2, 0, 1, 1]                  # position 2, tail phase flipped
    t.commit(m)
    t.close("x")
    m = t.plan([("z", 2)])                                            # the freed slot, counted from position 0 again
    assert m.table[0].tolist() == [0, 0] and m.table[1].tolist() == [0, 1]
    with pytest.raises(ValueError):
        t.plan([("z", 1), ("z", 1)])
    with pytest.raises(ValueError):
        t.plan([("y", 17)])


class _Recorder:
    """Stands in for a model: hidden row = (slot, position, token), logits = hidden."""
    n_slots, max_step_tokens, vocab_size, device = 2, 5, 3, "cpu"

    def __init__(self):
        self.passes = []

    def forward_batch(self, ids, meta):
        self.passes.append(meta.ntok)
        return torch.stack((meta.slot.float(), meta.pos.float(), ids.float()), 1)

    def logits(self, rows):
        return rows


def test_step_function_cuts_long_steps_and_keeps_the_order_of_wanted_rows():
    m = _Recorder()
    s = Scheduler(m)
    out = s.feed([("a", list(range(10, 22)), [11, 0, 6]), ("b", [7, 8], [1])])
    assert m.passes == [5, 5, 4]                                       # 12 + 2 tokens through passes of at most 5
    assert out.tolist() == [[0, 11, 21], [0, 0, 10], [0, 6, 16], [1, 1, 8]]
    out = s.feed([("b", [9], [0])])
    assert out.tolist() == [[1, 2, 9]]
    s.release("a")
    out = s.feed([("c", [1], [0])])
    assert out.tolist() == [[0, 0, 1]]
    with pytest.raises(ValueError):
        s.feed([("c", [1, 2], [2])])


def test_plain_implementation_is_causal_and_chunk_local():
    """Changing a token changes nothing before it, and nothing after the end of its chunk in a one-layer model without
    convolution (the only paths across a chunk border are the convolutions)."""
    cfg = {**CFG, "canon": {"taps": 1}, "layers": [CFG["layers"][3]]}
    w = {k: v.float() for k, v in random_weights(MutusunConfig.from_dict(cfg), 2).items()}
    a = [3, 1, 4, 1, 5, 9, 2, 6]
    b = list(a); b[4] = 8                                              # position 4 lies in chunk [3, 6)
    la, lb = O.forward(w, cfg, a), O.forward(w, cfg, b)
    same = [bool(torch.allclose(la[i], lb[i])) for i in range(len(a))]
    assert same == [True, True, True, True, False, False, True, True]
    assert O.chunk_visible(5, 3, 3) and not O.chunk_visible(5, 2, 3) and not O.chunk_visible(3, 4, 3)

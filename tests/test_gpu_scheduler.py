"""The scheduler serves the int4 decoder too: plain greedy decoding through its verify-mode (W4A16) path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_int4_decoder_through_the_scheduler():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from qspec_b200.model import QSpecLlamaConfig, QSpecLlamaModel
    from qspec_b200.scheduler import Scheduler
    cfg = QSpecLlamaConfig.tiny()
    model = QSpecLlamaModel(cfg, max_batch=2, max_tokens=16, device="cuda", seed=3)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (11, 3, 20)]
    outs = Scheduler(model, prefill_portion=8).generate(prompts, max_new_tokens=5)
    assert [len(o) for o in outs] == [5, 5, 5]
    # the same prompts one at a time, straight through the model
    match = total = 0
    for p, o in zip(prompts, outs):
        seq = list(p)
        slot = torch.zeros(1, dtype=torch.int32, device="cuda")
        h = model.forward(torch.tensor(seq[:16], device="cuda"), torch.arange(min(len(seq), 16), dtype=torch.int32, device="cuda"),
                          slot.expand(min(len(seq), 16)).contiguous(), w4a4=False)
        if len(seq) > 16:
            h = model.forward(torch.tensor(seq[16:], device="cuda"), torch.arange(16, len(seq), dtype=torch.int32, device="cuda"),
                              slot.expand(len(seq) - 16).contiguous(), w4a4=False)
        for t in o:
            nxt = int(model.greedy_tokens(h[-1:].clone())[0])
            total += 1
            match += nxt == t
            seq.append(t)
            h = model.forward(torch.tensor([t], device="cuda"), torch.tensor([len(seq) - 1], dtype=torch.int32, device="cuda"), slot,
                              w4a4=False)
    assert match >= 0.8 * total, f"{match} of {total} greedy tokens agree"      # float16 products differ by batch shape
    # a request longer than the cache is refused before anything runs
    with pytest.raises(RuntimeError):
        Scheduler(model).feed([("long", [1] * (cfg.max_seq_len + 1), [])])

"""Host-side parts of the text-only decoder LM: configuration, registry, checkpoint reader, scheduler, and the oracle's own
consistency (a prompt run whole equals the same prompt run in portions and token by token)."""
import json
import struct

import pytest
import torch

from moshi_b200.config import DECODER_ARCHITECTURES, DecoderLMConfig
from moshi_b200.serving import TokenScheduler
from moshi_b200.synth import iter_synth_decoder_tensors
from oracle.decoder_lm import DecoderOracle, sink_softmax


def small_cfg(**over):
    d = {"architecture": "Likosun", "vocab": 50, "width": 24, "embedding": {"scale": 3.0}, "residual_mult": 0.7, "norm": {"eps": 1e-5},
         "layers": [{"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "vdim": 5, "kv_rank": 12, "scale": 0.3},
                     "mlp": {"kind": "dense", "ff": 40}},
                    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 6, "vdim": 7, "kv_rank": 9, "scale": 0.5}, "mlp": None}]}
    d.update(over)
    return DecoderLMConfig.from_dict(d)


def test_config_round_trip_and_registry():
    cfg = small_cfg()
    assert DecoderLMConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.layers[1].mlp_kind is None and cfg.layers[1].ff == 0
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.uk"] == (24, 12) and shapes["l1.dwa"] == (3,) and "l1.mlp.up" not in shapes and "l1.rg2" not in shapes
    assert "Likosun" in DECODER_ARCHITECTURES
    with pytest.raises(ValueError):
        DecoderLMConfig.from_dict({**cfg.to_dict(), "architecture": "nope"})
    bad = cfg.to_dict()
    bad["layers"][0]["type"] = "ring_attention"
    with pytest.raises(ValueError):
        DecoderLMConfig.from_dict(bad)


def test_model_registry_picks_class_by_config():
    from moshi_b200.models import loaders
    from moshi_b200.models.decoder_lm import DecoderLM
    from moshi_b200.models.lm import LMModel
    assert loaders.model_class(small_cfg().to_dict()) is DecoderLM
    assert loaders.model_class({"dep_q": 8, "n_q": 16, "dim": 4096}) is LMModel
    with pytest.raises(ValueError):
        loaders.model_class({"architecture": "unknown"})


def test_safetensors_reader(tmp_path):
    from moshi_b200.models.loaders import read_safetensors
    a = torch.randn(3, 5).to(torch.bfloat16)
    b = torch.arange(7, dtype=torch.int32)
    blobs = {"a": ("BF16", a), "b": ("I32", b)}
    header, data = {}, b""
    for k, (dt, t) in blobs.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes()
        header[k] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [len(data), len(data) + len(raw)]}
        data += raw
    hj = json.dumps(header).encode()
    (tmp_path / "m.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + data)
    got = dict(read_safetensors(tmp_path / "m.safetensors"))
    assert torch.equal(got["a"], a) and torch.equal(got["b"], b)


def test_sink_softmax_counts_the_sink_once():
    s = torch.tensor([[0.5, -1.0, 2.0]], dtype=torch.float64)
    sink = torch.tensor([[0.25]], dtype=torch.float64)
    p = sink_softmax(s, sink)
    e = torch.exp(s)
    assert torch.allclose(p, e / (e.sum() + torch.exp(sink)))
    assert p.sum() < 1


def test_oracle_portions_equal_whole():
    cfg = small_cfg()
    orc = DecoderOracle(cfg, iter_synth_decoder_tensors(cfg, seed=5))
    toks = torch.randint(0, cfg.vocab, (19,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = orc.forward(toks)
    st = orc.new_state()
    parts = [orc.forward(toks[a:b], st) for a, b in ((0, 7), (7, 9), (9, 16), (16, 17), (17, 18), (18, 19))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-9)


class FakeGen:
    """Records steps; logits row = (slot, position, token) so that routing can be checked."""

    def __init__(self, slots, max_step_tokens, max_want):
        self.slots, self.max_step_tokens, self.max_want, self.vocab = slots, max_step_tokens, max_want, 3
        self.len = [0] * slots
        self.steps, self.released = [], []

    def step(self, entries, want):
        flat = []
        for slot, toks in entries:
            for t in toks:
                flat.append((slot, self.len[slot], t))
                self.len[slot] += 1
        assert sum(len(t) for _, t in entries) <= self.max_step_tokens and len(want) <= self.max_want
        self.steps.append([(s, list(t)) for s, t in entries])
        self._last = torch.tensor([flat[w] for w in want], dtype=torch.float32).reshape(len(want), 3)
        return self._last if len(want) else None

    def sample(self):
        return (self._last[:, 2].long() + 1) % 7          # next token = last token + 1 (mod 7)

    def release(self, slot):
        self.len[slot] = 0
        self.released.append(slot)


def test_scheduler_cuts_portions_and_routes_logits():
    gen = FakeGen(slots=2, max_step_tokens=4, max_want=3)
    s = TokenScheduler(gen)
    s.feed("a", [10, 11, 12, 13, 14, 15], want=[0, 5])
    s.feed("b", [20, 21, 22], want=[2])
    rows = {"a": [], "b": []}
    while (got := s.run_step()) is not None:
        for k, v in got.items():
            rows[k].append(v)
    assert [sum(len(t) for _, t in st) for st in gen.steps] == [4, 4, 1]
    a = torch.cat(rows["a"]).tolist()
    assert a == [[0.0, 0.0, 10.0], [0.0, 5.0, 15.0]]
    assert torch.cat(rows["b"]).tolist() == [[1.0, 2.0, 22.0]]
    s.end("a")
    assert gen.released == [0] and s.free_slots == 1
    s.feed("c", [1, 2], want=[1])            # the freed slot is used again, from position 0
    assert s.run_step()["c"].tolist() == [[0.0, 1.0, 2.0]]
    with pytest.raises(RuntimeError):
        s.feed("d", [1])


def test_scheduler_generates_until_budget_and_frees_slots():
    gen = FakeGen(slots=2, max_step_tokens=8, max_want=8)
    s = TokenScheduler(gen, eos=None)
    s.submit("x", [1, 2, 3], 4)
    s.submit("y", [5], 2)
    s.submit("z", [0, 0], 3)                 # waits for a slot
    out = s.run()
    assert out == {"x": [4, 5, 6, 0], "y": [6, 0], "z": [1, 2, 3]}
    assert s.free_slots == 2

"""The Govuvik decoder LM on the GPU against its float64 oracle (``oracle/govuvik.py``): every mechanism alone (the other
branch or sublayer switched off by its weights), whole prompts with every layer's output, prompts in portions down to one and
two tokens, token-by-token decoding, unequal batches, slots given back and used again, keys at the window's edges, far
memories of the recurrent mixers, the first tokens of a sequence, odd and aligned sizes, and greedy generation through the
scheduler and the command line."""
import copy
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from moshi_b200.config import DecoderLMConfig
from moshi_b200.synth import iter_synth_decoder_tensors
from oracle.decoder_lm import logit_error
from oracle.govuvik import F64, GovuvikOracle

from .test_gpu_zz_decoder_lm import gen_for, tokens, write_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {torch.float32: 3e-5, torch.bfloat16: 8e-2}


def window(heads, kv, dim, vdim, size, conv, rot_dims, scale, base=500.0, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv, "mask": {"size": size}, "rot": rot, "scale": scale, "vdim": vdim}


def parallel(left, heads, dim, vdim, tau, moe, rank=5):
    return {"type": "parallel", "mixer": {"left": left, "right": {"dim": dim, "heads": heads, "tau": tau, "vdim": vdim, "decay_rank": rank}}, "mlp": moe}


def mlstm(heads, dim, vdim, cap, moe):
    return {"type": "mlstm", "mixer": {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}, "mlp": moe}


def moe(experts, top, ff):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


def make_cfg(layers, vocab, width, taps, cap=9.0, eps=1e-5):
    return DecoderLMConfig.from_dict({"architecture": "Govuvik", "canon": {"taps": taps}, "layers": layers, "logit_softcap": cap,
                                      "norm": {"eps": eps}, "vocab": vocab, "width": width})


SCALING = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}      # with base 500 and 8 dims: one kept, one blended, two divided
# odd sizes: nothing is a multiple of 8; three query heads per key head and one; value size unlike key size; 1, 2 and all experts
ODD = make_cfg([mlstm(3, 10, 12, 7.5, moe(5, 2, 24)),
                parallel(window(6, 2, 12, 10, 9, 3, 8, 0.31, scaling=SCALING), 2, 9, 20, 5.0, moe(3, 3, 17)),
                parallel(window(4, 4, 14, 6, 5, 2, 14, 0.2), 3, 7, 9, 1.0, None),
                mlstm(2, 17, 5, 3.0, moe(4, 1, 30))], vocab=97, width=52, taps=4)
# aligned sizes: in bfloat16 every linear takes the tcgen05 GEMM and the experts the tensor-core grouped product; a layer order
# that starts with the pair; one key head for all query heads; no rotation scaling, rotation over the whole head
ALIGNED = make_cfg([parallel(window(4, 1, 32, 16, 40, 5, 32, 0.18), 2, 16, 32, 8.0, moe(8, 2, 48), rank=8),
                    mlstm(2, 16, 64, 10.0, moe(6, 3, 32)),
                    parallel(window(2, 2, 16, 48, 70, 1, 0, 0.25), 4, 40, 24, 3.0, moe(8, 2, 48), rank=16)], vocab=200, width=96, taps=2)


def build(cfg, dtype, seed=3, edit=None):
    from moshi_b200.models import DecoderLM
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=seed))
    if dtype == torch.bfloat16:
        # a bf16 rounding can turn a router's close call and swap an expert for that token; with random weights that happens
        # every few dozen tokens.  A small post-norm weight keeps such a swap inside the bf16 tolerance (float32 runs as drawn).
        for k in tensors:
            if k.endswith("norm2b"):
                tensors[k] = tensors[k] * 0.25
    if edit:
        edit(tensors)
    return DecoderLM(cfg, tensors, device="cuda:0", dtype=dtype), GovuvikOracle(cfg.to_dict(), tensors)


def assert_close(got, want, dtype, what="", tol=None):
    """float32: every row within the tolerance.  bfloat16: a rounding can turn a router's close call, which changes that token
    as a whole, so up to a tenth of the rows may be off while the median stays well inside."""
    e = logit_error(got.cpu(), want)
    tol = tol or TOL[dtype]
    if dtype == torch.float32:
        assert float(e.max()) < tol, f"{what}: relative logit error {float(e.max()):.3g}"
    else:
        assert int((e > tol).sum()) <= max(1, e.numel() // 10) and float(e.median()) < tol, f"{what}: relative logit errors {e.tolist()}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
def test_whole_prompt_and_every_layer(cfg, dtype):
    model, orc = build(cfg, dtype)
    toks = tokens(90, cfg.vocab, 1)
    want, layers = orc.forward(toks, return_layers=True)
    with gen_for(model, trace_layers=True) as gen:
        got = gen.step([(1, toks)], list(range(len(toks))))
        lo = gen.layer_outputs().cpu()
        assert gen.error_flags() == 0
    scale = float(layers.abs().max())
    for i in range(len(cfg.layers)):
        err = (lo[i].to(F64) - layers[i]).abs().amax(-1) / scale              # per token
        if dtype == torch.float32:
            assert float(err.max()) < 2e-5, f"layer {i}: {float(err.max()):.3g}"
        else:
            assert int((err > 8e-2).sum()) <= err.numel() // 4 and float(err.median()) < 4e-2, f"layer {i}: {err.tolist()}"
    assert_close(got, want, dtype)


def one_layer(kind, **kw):
    if kind == "mlstm":
        return make_cfg([mlstm(3, 12, 20, kw.get("cap", 6.0), kw.get("moe"))], vocab=64, width=40, taps=kw.get("taps", 1))
    left = window(kw.get("heads", 6), kw.get("kv", 3), 10, 14, kw.get("size", 7), kw.get("conv", 3), kw.get("rot", 6), 0.3, scaling=kw.get("scaling"))
    return make_cfg([parallel(left, 2, 11, 18, kw.get("tau", 4.0), kw.get("moe"))], vocab=64, width=40, taps=kw.get("taps", 1))


def zero(name):
    def edit(t):
        t[name] = torch.zeros_like(t[name])
    return edit


@pytest.mark.parametrize("what", ["window_attention", "window_no_conv", "window_conv_1", "window_rot_scaled", "window_one_kv_head", "gla", "gla_tau_1", "mlstm",
                                  "mlstm_tight_cap", "canon_2", "canon_5", "moe_top1", "moe_all", "softcap"])
def test_mechanisms_in_isolation(what):
    """One layer; the branch or sublayer that is not under test is switched off through its weights (an output norm of zero)."""
    edit = None
    if what.startswith("window"):
        kw = {"window_no_conv": {"conv": 0}, "window_conv_1": {"conv": 1}, "window_rot_scaled": {"rot": 10, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 40}},
              "window_one_kv_head": {"kv": 1}}.get(what, {})
        cfg, edit = one_layer("parallel", **kw), zero("l0.mix.right.out")
    elif what.startswith("gla"):
        cfg, edit = one_layer("parallel", tau=1.0 if what == "gla_tau_1" else 4.0), zero("l0.mix.left.out")
    elif what.startswith("mlstm"):
        cfg = one_layer("mlstm", cap=0.7 if what == "mlstm_tight_cap" else 6.0)
    elif what.startswith("canon"):
        cfg = one_layer("mlstm", taps=int(what[-1]))
    elif what == "moe_top1":
        cfg = one_layer("mlstm", moe=moe(7, 1, 12))
    elif what == "moe_all":
        cfg = one_layer("parallel", moe=moe(3, 3, 20))
    else:
        cfg = copy.deepcopy(one_layer("mlstm"))
        cfg.logit_softcap = 0.8             # deep into the tanh
    model, orc = build(cfg, torch.float32, seed=11, edit=edit)
    toks = tokens(40, cfg.vocab, 2)
    want, layers = orc.forward(toks, return_layers=True)
    with gen_for(model, trace_layers=True) as gen:
        got = gen.step([(0, toks)], list(range(len(toks))))
        lo = gen.layer_outputs().cpu()
    assert float((lo[0].to(F64) - layers[0]).abs().max()) < 3e-5 * float(layers.abs().max())
    assert_close(got, want, torch.float32, what)


def sharpen(t):
    """Large temperatures: one key takes almost all the weight, so a key that is wrongly seen or missed changes the result as a whole."""
    for k in list(t):
        if k.endswith(".temp"):
            t[k] = t[k] * 6.0
        if k.endswith(".sink"):
            t[k] = t[k] - 6.0


@pytest.mark.parametrize("size", [1, 2, 7, 32, 33, 40])
def test_keys_at_the_windows_edge(size):
    """Sharp attention over a window of `size`: positions whose strongest key is the oldest one still seen, or the first one no
    longer seen, come out wrong if the window is off by one.  Prompt (one step) and decoding (one token a step) alike; the test
    first shows that the oracle itself moves by far more than the tolerance when its window is changed by one."""
    cfg = one_layer("parallel", size=size, heads=4, kv=2, conv=2)
    model, orc = build(cfg, torch.float32, seed=5, edit=lambda t: (sharpen(t), zero("l0.mix.right.out")(t)))
    toks = tokens(100, cfg.vocab, 3)
    want = orc.forward(toks)
    other = cfg.to_dict()
    other["layers"][0]["mixer"]["left"]["mask"]["size"] = size + 1
    moved = GovuvikOracle(other, orc.W).forward(toks)
    assert float(logit_error(moved, want).max()) > 100 * TOL[torch.float32]
    with gen_for(model) as gen:
        got = gen.step([(0, toks[:60])], list(range(60)))
        rest = torch.cat([gen.step([(0, [t])], [0]) for t in toks[60:]])
    assert_close(torch.cat([got, rest]), want, torch.float32)


def keep_long(t):
    """Decays and forget gates next to one: what the recurrent mixers took in hundreds of tokens ago still weighs."""
    for k in list(t):
        if k.endswith("a2.b") or k.endswith("f.b"):
            t[k] = torch.full_like(t[k], 9.0)
        if k.endswith(".a2") or k.endswith("mix.f"):
            t[k] = t[k] * 0.1


@pytest.mark.parametrize("kind", ["gla", "mlstm"])
def test_far_tokens_reach_through_the_recurrent_state(kind):
    cfg = one_layer("parallel", size=3, tau=2.0) if kind == "gla" else one_layer("mlstm", cap=12.0)
    edit = (lambda t: (keep_long(t), zero("l0.mix.left.out")(t))) if kind == "gla" else keep_long
    model, orc = build(cfg, torch.float32, seed=6, edit=edit)
    toks = tokens(400, cfg.vocab, 4)
    want = orc.forward(toks)[-40:]
    swapped = [(toks[0] + 1) % cfg.vocab] + toks[1:]
    assert float(logit_error(orc.forward(swapped)[-40:], want).max()) > 30 * TOL[torch.float32], "token 0 must still matter at the end"
    with gen_for(model, capacity=512, max_step_tokens=512) as gen:
        gen.step([(0, toks[:150])])
        gen.step([(0, toks[150:360])])
        got = gen.step([(0, toks[360:])], list(range(40)))
    assert_close(got, want, torch.float32)


@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_portions_and_single_tokens_equal_the_whole_prompt(dtype, cfg):
    model, orc = build(cfg, dtype)
    toks = tokens(130, cfg.vocab, 7)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        whole = gen.step([(0, toks)], list(range(len(toks))))
        for cuts in ([2, 3, 1, 7, 2, 40, 1, 1, 2, 9, 33, 2, 27], [64, 66], [1] * 12 + [118], [5, 4, 3, 2] * 9 + [4]):
            assert sum(cuts) == len(toks)
            gen.release(2)
            parts, at = [], 0
            for n in cuts:
                parts.append(gen.step([(2, toks[at:at + n])], list(range(n))))
                at += n
            got = torch.cat(parts)
            assert_close(got, want, dtype, f"cuts {cuts[:4]}")
            assert_close(got, whole.cpu().to(F64), dtype, "a cut changes at most the order of sums")


def test_the_first_tokens_of_a_sequence():
    """Positions 0 .. 5: convolutions with nothing in front, the running maximum that starts at 0, the sink against a single key."""
    model, orc = build(ODD, torch.float32, seed=9)
    for n in (1, 2, 3, 6):
        toks = tokens(n, ODD.vocab, 20 + n)
        with gen_for(model) as gen:
            assert_close(gen.step([(0, toks)], list(range(n))), orc.forward(toks), torch.float32, f"{n} tokens at once")
            gen.release(0)
            one = torch.cat([gen.step([(0, [t])], [0]) for t in toks])
            assert_close(one, orc.forward(toks), torch.float32, f"{n} tokens one by one")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_token_by_token(dtype):
    cfg = ALIGNED
    model, orc = build(cfg, dtype, seed=4)
    toks = tokens(200, cfg.vocab, 8)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        gen.step([(1, toks[:20])])
        got = torch.cat([gen.step([(1, [t])], [0]) for t in toks[20:]])
        assert gen.error_flags() == 0
    assert_close(got, want[20:], dtype)


@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_batch_equals_each_request_alone(dtype, cfg):
    model, orc = build(cfg, dtype)
    reqs = [tokens(61, cfg.vocab, 30), tokens(9, cfg.vocab, 31), tokens(34, cfg.vocab, 32)]
    want = [orc.forward(r) for r in reqs]
    with gen_for(model) as gen:
        # different histories: 40 tokens, none, 33 tokens; then one step with 21 + 9 + 1 tokens
        gen.step([(2, reqs[0][:40]), (0, reqs[2][:33])])
        got = gen.step([(2, reqs[0][40:]), (1, reqs[1]), (0, reqs[2][33:])], list(range(31)))
    assert_close(got[:21], want[0][40:], dtype, "long history, many tokens")
    assert_close(got[21:30], want[1], dtype, "fresh request")
    assert_close(got[30:], want[2][33:], dtype, "single token")


def test_slots_are_given_back_and_used_again():
    """A shorter request in a slot that held a longer one: neither its cached keys, nor the carried convolution inputs, nor the
    matrix memories of the earlier request may show."""
    cfg = ODD
    model, orc = build(cfg, torch.float32)
    long_req, short_req = tokens(120, cfg.vocab, 50), tokens(11, cfg.vocab, 51)
    with gen_for(model, slots=1) as gen:
        gen.step([(0, long_req)])
        gen.release(0)
        assert gen.slot_length(0) == 0
        got = gen.step([(0, short_req[:2])], [0, 1])
        got = torch.cat([got, gen.step([(0, short_req[2:])], list(range(9)))])
        assert_close(got, orc.forward(short_req), torch.float32)
        gen.release(0)
        gen.step([(0, short_req)])
        with pytest.raises(Exception):
            gen.step([(0, tokens(300, cfg.vocab, 52))])             # would overflow the slot: refused whole
        assert gen.slot_length(0) == len(short_req)


def test_split_keys_equal_one_pass():
    """The window attention cut over several CTAs along the keys (what decoding with few requests does) against a single pass."""
    cfg = ALIGNED
    model, orc = build(cfg, torch.float32, seed=12)
    toks = tokens(140, cfg.vocab, 60)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        for split in (1, 2, 5):
            gen.release(0)
            gen.set_option("attn_split", split)
            got = gen.step([(0, toks)], list(range(len(toks))))
            assert_close(got, want, torch.float32, f"split {split}")


def test_greedy_generation_through_the_scheduler():
    from moshi_b200.serving import TokenScheduler
    cfg = ODD
    model, orc = build(cfg, torch.float32)
    prompts = {"a": tokens(23, cfg.vocab, 40), "b": tokens(3, cfg.vocab, 41), "c": tokens(40, cfg.vocab, 42)}
    with gen_for(model, slots=2, capacity=80, max_step_tokens=32) as gen:      # 3 requests over 2 slots, prompts cut at 32 tokens
        sched = TokenScheduler(gen)
        for k, p in prompts.items():
            sched.submit(k, p, 12)
        out = sched.run()
    for k, p in prompts.items():
        want, gaps = orc.greedy(p, 12)
        for i, (g, w, gap) in enumerate(zip(out[k], want, gaps)):
            if g != w:
                assert gap < 1e-3, f"request {k}: token {i} is {g}, the oracle says {w} with a gap of {gap}"
                break


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_command_line_replays_steps_and_generates(tmp_path, dtype):
    cfg = ODD
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=8))
    write_model(tmp_path / "m", cfg, tensors)
    orc = GovuvikOracle(json.loads((tmp_path / "m" / "config.json").read_text()), tensors)
    a, b = tokens(30, cfg.vocab, 50), tokens(6, cfg.vocab, 51)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[21:23], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[23:], "want": [6]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]}]
    (tmp_path / "out").mkdir()
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out", str(tmp_path / "out"),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    import numpy as np
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    read = lambda i, n: torch.from_numpy(np.fromfile(tmp_path / "out" / f"{i}.f32", dtype="<f4").reshape(n, cfg.vocab))
    fa = orc.forward(a)
    assert_close(read(0, 2), fa[[0, 20]], td)
    assert_close(read(2, 1), fa[[29]], td)
    assert_close(read(3, 1), orc.forward(b)[[5]], td)
    if dtype == "float32":
        r = subprocess.run([sys.executable, "-m", "moshi_b200.cli", "generate", "--model", str(tmp_path / "m"), "--dtype", dtype,
                            "--prompt", ",".join(map(str, b)), "--max-new", "5"], capture_output=True, text=True, timeout=600, cwd=ROOT)
        assert r.returncode == 0, r.stderr[-2000:]
        got = json.loads(r.stdout.strip().splitlines()[-1])["tokens"]
        want, gaps = orc.greedy(b, 5)
        for g, w, gap in zip(got, want, gaps):
            if g != w:
                assert gap < 1e-3
                break


@pytest.mark.parametrize("heads,kv,dim,vdim,size", [(4, 2, 16, 16, 5), (6, 3, 32, 80, 33), (16, 4, 32, 128, 70), (2, 1, 48, 32, 1), (8, 8, 16, 64, 32)])
def test_window_attention_on_tensor_cores(heads, kv, dim, vdim, size):
    """bf16 caches with fragment-sized heads take the tensor-core kernel (1, 2 or 4 accumulator items per warp): against the
    oracle and against the CUDA-core kernel on the same model, as one prompt, in portions, token by token and with split keys.
    Sharp attention (large temperatures), so that a key wrongly seen or missed at the window's edge would show."""
    left = window(heads, kv, dim, vdim, size, 2, 16, dim ** -0.5)
    cfg = make_cfg([parallel(left, 2, 16, 16, 4.0, None, rank=8)], vocab=120, width=64, taps=2)
    model, orc = build(cfg, torch.bfloat16, seed=21, edit=lambda t: (sharpen(t), zero("l0.mix.right.out")(t)))
    toks = tokens(150, cfg.vocab, 70)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        gen.set_option("attn_tc", 0)
        plain = gen.step([(0, toks)], list(range(len(toks))))
        gen.set_option("attn_tc", 1)
        for split in (0, 1, 3):
            gen.set_option("attn_split", split)
            whole = gen.step([(1, toks)], list(range(len(toks))))
            gen.release(1)
            assert_close(whole, want, torch.bfloat16, f"split {split}")
            assert_close(whole, plain.cpu().to(F64), torch.bfloat16, f"split {split}, against the CUDA-core kernel")
        gen.set_option("attn_split", 0)
        parts = [gen.step([(2, toks[:37])], list(range(37))), gen.step([(2, toks[37:39])], [0, 1]), gen.step([(2, toks[39:100])], list(range(61)))]
        parts += [gen.step([(2, [t])], [0]) for t in toks[100:125]]         # single tokens: the CUDA-core kernel
        gen.set_option("attn_tc", 2)                                            # and the tensor-core kernel on one-token tiles
        parts += [gen.step([(2, [t])], [0]) for t in toks[125:]]
        assert_close(torch.cat(parts), want, torch.bfloat16, "portions and single tokens")
        assert gen.error_flags() == 0


@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_portions_run_as_parallel_segments(dtype, cfg):
    """A portion of at least two segments is cut for the recurrences: the segments run side by side from empty memories, are
    chained, and the later ones get the carried state's share added.  Segments of 16 tokens here (256 by default), so that
    portions of 33 .. 150 tokens take that path: one prompt, portions with a ragged last segment, a batch of long and short
    requests on different histories, then single tokens on the state the chain left in the slot."""
    from moshi_b200 import _lib
    model, orc = build(cfg, dtype)
    _lib.check(model._lib.b200_dlm_set_option(model._h, b"scan_segment", 16))
    reqs = [tokens(150, cfg.vocab, 80), tokens(9, cfg.vocab, 81), tokens(120, cfg.vocab, 82)]
    want = [orc.forward(r) for r in reqs]
    with gen_for(model) as gen:
        assert_close(gen.step([(0, reqs[0])], list(range(150))), want[0], dtype, "one portion of 150 tokens")
        gen.release(0)
        parts = [gen.step([(0, reqs[0][:70])], list(range(70))), gen.step([(0, reqs[0][70:73])], [0, 1, 2]), gen.step([(0, reqs[0][73:110])], list(range(37)))]
        parts += [gen.step([(0, [t])], [0]) for t in reqs[0][110:]]
        assert_close(torch.cat(parts), want[0], dtype, "70 + 3 + 37 tokens, then one by one")
        gen.release(0)
        gen.step([(2, reqs[0][:40]), (0, reqs[2][:33])])
        got = gen.step([(2, reqs[0][40:]), (1, reqs[1]), (0, reqs[2][33:])], list(range(110 + 9 + 87)))
        assert_close(got[:110], want[0][40:], dtype, "110 tokens on a history of 40")
        assert_close(got[110:119], want[1], dtype, "a short fresh request beside them")
        assert_close(got[119:], want[2][33:], dtype, "87 tokens on a history of 33")
        assert gen.error_flags() == 0


def test_segments_of_the_default_length():
    cfg = ALIGNED
    model, orc = build(cfg, torch.float32, seed=13)
    toks = tokens(700, cfg.vocab, 90)
    want = orc.forward(toks)
    with gen_for(model, capacity=1024, max_step_tokens=1024) as gen:
        got = torch.cat([gen.step([(0, toks[:600])], list(range(600))), gen.step([(0, toks[600:])], list(range(100)))])
    assert_close(got, want, torch.float32)

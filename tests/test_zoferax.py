"""The Zoferax decoder against its plain implementation (``plain_zoferax``): each mechanism alone, then whole models
through trace replay (whole, decoded one by one, in portions down to two tokens, mixed batches on a pool that runs
full) and greedy generation through the engine.  Configurations and weights are made here; attention is made peaky
(score factors that let the largest scores reach about ten), so that much of a query's weight sits on a few keys
anywhere in the sequence, far back and at page borders alike, and a lost key shows in the logits, while the scores stay
small enough for bfloat16 queries and keys (a score of 50 carries a rounding error of 0.2 in the exponent)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zoferax as plain
from plain_qwen3 import read_model_folder
from tiny_configs import random_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def attention(heads, kv_heads, dim, vdim, scale, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def experts(count, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": count, "top": top}}


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


# P: sizes in multiples of 8, values narrower than keys, a sharing layer without feed-forward in the middle, a
# layer whose kv heads equal its heads.  Q: nothing a multiple of 8 but the cache rows, values WIDER than keys, one kv
# head for six query heads, one expert of three and three of three, the sharing layer last and reading layer 0.
CONFIG_P = {
    "architecture": "Zoferax", "width": 64, "vocab": 200, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        layer(attention(4, 2, 16, 8, 0.75), experts(4, 2, 32)),
        layer(attention(4, 2, 16, 8, 0.6, kv_from=0), None),
        layer(attention(2, 2, 32, 32, 0.35), experts(8, 3, 16)),
        layer(attention(4, 2, 16, 8, 0.8, kv_from=0), experts(4, 1, 32)),
    ],
}
CONFIG_Q = {
    "architecture": "Zoferax", "width": 100, "vocab": 131, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-3},
    "layers": [
        layer(attention(6, 1, 12, 20, 0.9), experts(3, 1, 20)),
        layer(attention(3, 3, 20, 4, 0.5), None),
        layer(attention(6, 1, 12, 20, 0.6, kv_from=0), experts(3, 3, 12)),
    ],
}
TINY = {"P": (CONFIG_P, 4, 3), "Q": (CONFIG_Q, 8, 4)}  # name -> (config, page size, seed)


def write_model(folder, raw, seed):
    import kirai_b200  # noqa: F401
    from kirai_b200.registry import config_from_dict
    from kirai_b200.weights import write_random_model

    write_random_model(folder, config_from_dict(raw), seed, std=0.08, norm_jitter=0.3, dtype=torch.bfloat16)


def tolerance(dtype, reference):
    dtype = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(dtype, dtype)
    peak = float(np.abs(np.asarray(reference)).max())
    return 3e-5 * max(1.0, peak) if dtype == "float32" else 0.035 * peak


# --------------------------------------------------------------------------- no GPU
def test_config_reads_every_size_and_round_trips():
    import kirai_b200  # noqa: F401
    from kirai_b200.config.base import ConfigError
    from kirai_b200.registry import config_from_dict, plan_for_config

    for raw in (CONFIG_P, CONFIG_Q):
        cfg = config_from_dict(raw)
        assert cfg.to_dict() == raw and config_from_dict(cfg.to_dict()) == cfg
        assert (cfg.width, cfg.vocab, cfg.norm_eps) == (raw["width"], raw["vocab"], raw["norm"]["eps"])
        plan = plan_for_config(cfg)
        own = [i for i, entry in enumerate(raw["layers"]) if "kv_from" not in entry["mixer"]]
        assert len(plan.cache_needs) == len(own)
        for call, entry in zip(plan.order, raw["layers"]):
            source = entry["mixer"].get("kv_from")
            assert call.write == (source is None)
            assert call.cache == own.index(call.block if source is None else source)
        names = set(plan.weight_specs())
        for i, entry in enumerate(raw["layers"]):
            shares = "kv_from" in entry["mixer"]
            assert (f"l{i}.mix.k" in names) != shares and (f"l{i}.mix.v.b" in names) != shares
            assert (f"l{i}.mix.k.norm" in names) != shares and f"l{i}.mix.q.norm" in names
            assert (f"l{i}.norm2" in names) == (entry["mlp"] is not None) == (f"l{i}.mlp.router" in names)
    bad = json.loads(json.dumps(CONFIG_P))
    bad["layers"][1]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(CONFIG_P))
    bad["layers"][3]["mixer"]["kv_from"] = 1  # layer 1 has no keys of its own
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(CONFIG_P))
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(CONFIG_P))
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_plain_attention_is_peaky_and_reaches_far_back(tmp_path):
    """What makes the comparisons below sharp: under these configurations most of a query's weight sits on a few keys, and for
    many queries the heaviest key lies more than 64 tokens and many pages back."""
    write_model(str(tmp_path), CONFIG_P, 3)
    raw, weights = read_model_folder(str(tmp_path))
    tokens = torch.tensor(random_tokens(160, raw["vocab"], 5))
    x = plain.scaled_embedding(weights["embed"], tokens, raw["embedding"]["scale"]) + plain.sinusoid_positions(torch.arange(160), raw["width"])
    mixer = raw["layers"][0]["mixer"]
    q = plain.rms_unit(plain.projection(x, weights["l0.mix.q"], weights["l0.mix.q.b"]), raw["norm"]["eps"]) * weights["l0.mix.q.norm"]
    k, _ = plain.keys_and_values(x, weights, "l0.mix.", raw["norm"]["eps"])
    far, heavy = 0, []
    for i in range(100, 160):
        w = torch.softmax((k[: i + 1, :16] @ q[i, :16]) * mixer["scale"], dim=0)
        heavy.append(float(w.max()))
        far += int(i - int(w.argmax()) > 64)
    assert np.mean(heavy) > 0.12 and far >= 8


# --------------------------------------------------------------------------- mechanisms (GPU)
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [64, 50, 7])
def test_scaled_sinusoid_embedding(dtype, width):
    from part_helpers import DEV, load_part
    from kirai_b200.parts import Embedding

    part = Embedding("embed", 40, width, scale=2.5, sinusoid_base=10000.0)
    weights = load_part(part, dtype, seed=1)
    tokens = torch.tensor([3, 0, 39, 7, 7], dtype=torch.int32)
    positions = torch.tensor([0, 1, 5000, 63, 64], dtype=torch.int32)
    got = part.forward(tokens.to(DEV), positions.to(DEV)).cpu()
    expected = plain.scaled_embedding(weights["embed"], tokens.long(), 2.5) + plain.sinusoid_positions(positions, width)
    assert got.dtype == torch.float32 and float((got - expected).abs().max()) < 2e-3  # angle 5000 in 32-bit: 5000 * 2^-24


@pytest.mark.gpu
@pytest.mark.parametrize("width", [64, 100, 7, 4096 + 8])
def test_norm_on_the_output(width):
    from part_helpers import DEV, load_part
    from kirai_b200.parts import RMSNorm

    for dtype in (torch.float32, torch.bfloat16):
        part = RMSNorm("n", width, 1e-3)
        weights = load_part(part, dtype, seed=2)
        g = torch.Generator().manual_seed(width)
        stream, y = torch.randn(5, width, generator=g), 3.0 * torch.randn(5, width, generator=g)
        expected = stream + plain.rms_unit(y, 1e-3) * weights["n"]
        resid = stream.clone().to(DEV)
        copy = part.add_normed(resid, y.to(DEV))
        assert float((resid.cpu() - expected).abs().max()) < 1e-5
        if dtype == torch.float32:
            assert copy is None
        else:
            assert copy.dtype == torch.bfloat16 and torch.equal(copy.cpu(), resid.cpu().to(torch.bfloat16))


def _expert_tensors(part, seed):
    """Random weights with a router four times as large (exact in bfloat16), so that router logits are rarely close."""
    from kirai_b200.weights.random_init import random_tensors

    tensors = random_tensors(part.weight_specs(), seed, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    tensors["m.router"] = tensors["m.router"] * 4.0
    return tensors


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("count,top,ff,width", [(8, 2, 16, 64), (3, 1, 20, 100), (3, 3, 12, 36), (40, 5, 8, 24), (1, 1, 8, 16), (3, 2, 10, 30)])
def test_routed_experts(dtype, count, top, ff, width):
    from part_helpers import DEV, load_part
    from kirai_b200.parts import RoutedExperts

    names = {"router": "router", "up": "e{e}.up", "down": "e{e}.down"}
    part = RoutedExperts("m.", width, ff, count, top, names=names, out_dtype=torch.float32)
    weights = load_part(part, dtype, tensors=_expert_tensors(part, count))
    x = torch.randn(9, width, generator=torch.Generator().manual_seed(7)).to(dtype)
    got = part.forward(x.to(DEV)).cpu()
    expected = plain.routed_experts(x.float(), weights, "m.", count, top)
    assert got.dtype == torch.float32
    assert float((got - expected).abs().max()) <= tolerance(dtype, expected)
    # the routing itself: the chosen experts and their weights
    gates, ids, mix = part.rt.ops.router_gates(x.to(DEV), part.router, top, want_chosen=True)
    logits = x.float() @ weights["m.router"].t()
    for t in range(x.shape[0]):
        chosen = torch.topk(logits[t], top).indices
        assert sorted(ids[t].tolist()) == sorted(chosen.tolist())
        want = torch.zeros(count)
        want[chosen] = torch.softmax(logits[t, chosen], dim=0)
        assert float((gates[t].cpu() - want).abs().max()) < 1e-5 and abs(float(mix[t].sum()) - 1.0) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("count,top,ff,width,tokens", [(4, 2, 128, 128, 300), (8, 1, 256, 384, 700), (5, 3, 128, 256, 171)])
def test_routed_experts_sorted_by_expert(count, top, ff, width, tokens):
    """Steps of many tokens sort their (token, expert) pairs by expert and run grouped products: against the plain
    function, and against the few-token path of the same part on the same rows."""
    from part_helpers import DEV, load_part
    from kirai_b200.parts import RoutedExperts, experts as experts_module

    names = {"router": "router", "up": "e{e}.up", "down": "e{e}.down"}
    part = RoutedExperts("m.", width, ff, count, top, names=names, out_dtype=torch.float32)
    weights = load_part(part, torch.bfloat16, tensors=_expert_tensors(part, count))
    assert part.grouped and tokens * top >= experts_module.GROUPED_MIN_ROWS
    x = torch.randn(tokens, width, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    before = dict(part.rt.ops.launch_counts)
    got = part.forward(x.to(DEV)).cpu()
    assert part.rt.ops.launch_counts.get("kirai_gemm_bf16_grouped", 0) - before.get("kirai_gemm_bf16_grouped", 0) == 2
    expected = plain.routed_experts(x.float(), weights, "m.", count, top)
    assert float((got - expected).abs().max()) <= tolerance(torch.bfloat16, expected)
    few = torch.cat([part.forward(x[i : i + 100].to(DEV)).cpu() for i in range(0, tokens, 100)])
    assert float((got - few).abs().max()) <= tolerance(torch.bfloat16, expected)
    # the norm on the output taken over by the part: the same stream as the part's output through the norm kernel
    from kirai_b200.parts import RMSNorm

    norm = RMSNorm("n", width, 1e-4)
    load_part(norm, torch.bfloat16, seed=3)
    stream = torch.randn(tokens, width, generator=torch.Generator().manual_seed(4))
    apart, fused = stream.clone().to(DEV), stream.clone().to(DEV)
    copy_apart = norm.add_normed(apart, part.forward(x.to(DEV)))
    assert part.adds_normed(tokens) and not part.adds_normed(GROUPED_FEW)
    copy_fused = part.forward_add_normed(x.to(DEV), None, fused, norm.fused_spec())
    assert float((apart - fused).abs().max()) < 1e-5 and float((copy_apart.float() - copy_fused.float()).abs().max()) < 0.02
    part.rt.ops.check_device_errors(DEV)


GROUPED_FEW = 8  # a step of this many tokens takes the few-token path


def _attention_part(mixer, width, shares=False):
    from kirai_b200.parts import GQAttention

    names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}
    return GQAttention("a.", width, mixer["heads"], mixer["kv_heads"], mixer["dim"], None, scale=mixer["scale"],
                       value_dim=mixer["vdim"], bias=True, qk_norm_eps=1e-4, qk_norm_over="projection", reads_only=shares,
                       names=names, out_dtype=torch.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mixer,width,page", [(attention(4, 2, 16, 8, 0.8), 64, 4), (attention(6, 1, 12, 20, 0.9), 100, 8),
                                              (attention(3, 3, 20, 4, 0.6), 40, 16), (attention(2, 1, 64, 64, 0.2), 32, 2),
                                              (attention(2, 1, 10, 6, 1.0), 30, 16), (attention(40, 2, 8, 8, 1.0), 64, 32),
                                              (attention(4, 2, 96, 48, 0.1), 64, 16), (attention(3, 1, 48, 80, 0.2), 48, 16),
                                              (attention(2, 2, 128, 64, 0.08), 64, 64), (attention(2, 1, 136, 8, 0.08), 32, 16)])
def test_attention_part_whole_in_portions_and_one_by_one(dtype, mixer, width, page):
    """One attention layer over 150 tokens: whole, in uneven portions, and token by token, against the plain function;
    then a second request on pages that the first gave back."""
    from part_helpers import DEV, Session, load_part

    part = _attention_part(mixer, width)
    weights = load_part(part, dtype, seed=11)
    total = 150
    x = torch.randn(total, width, generator=torch.Generator().manual_seed(3)).to(dtype)
    expected, _ = plain.attention_mixer(x.float(), weights, "a.", mixer, 1e-4)
    bound = tolerance(dtype, expected)
    pages = -(-total // page) + 2
    session = Session([part.cache_need()], dtype, page_size=page, num_pages=pages)
    for name, cuts in (("whole", [total]), ("portions", [37, 2, 61, 3, 2, 45]), ("single", [1] * total), ("again", [70, 80])):
        at, rows = 0, []
        for n in cuts:
            batch = session.batch([(name, n)])
            rows.append(part.forward(x[at : at + n].to(DEV), batch, session.cache.layer_view(0), True).cpu())
            session.commit()
            at += n
        got = torch.cat(rows)
        assert float((got - expected).abs().max()) <= bound, name
        session.cache.close(session.requests.pop(name))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_that_stands_out(dtype):
    """Queries and keys share their projection here (no biases on them), so a token whose input is three times that of
    an earlier token has that token's key (the norm removes the factor) but another value: it puts its weight on
    that one key and on itself.  The earlier token lies 2, 16, 17, 64 or 416 tokens back, in the same portion or
    decoded long after; without it the plain result is far outside the bound."""
    from part_helpers import DEV, Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    mixer, width, page = attention(2, 2, 16, 8, 6.0), 48, 16
    part = _attention_part(mixer, width)
    tensors = random_tensors(part.weight_specs(), 5, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    tensors["a.q.b"] = torch.zeros_like(tensors["a.q.b"])
    tensors["a.k"], tensors["a.k.b"], tensors["a.k.norm"] = tensors["a.q"].clone(), tensors["a.q.b"].clone(), tensors["a.q.norm"].clone()
    weights = load_part(part, dtype, tensors=tensors)
    total = 420
    x = torch.randn(total, width, generator=torch.Generator().manual_seed(9)).to(dtype)
    pairs = [(3, 419), (20, 84), (40, 57), (100, 116), (7, 9), (150, 165)]
    for early, late in pairs:
        x[late] = 3.0 * x[early]
    expected, _ = plain.attention_mixer(x.float(), weights, "a.", mixer, 1e-4)
    bound = tolerance(dtype, expected)
    for early, late in pairs:
        without = x.float().clone()
        without[early] = torch.randn(width, generator=torch.Generator().manual_seed(10))
        blind, _ = plain.attention_mixer(without, weights, "a.", mixer, 1e-4)
        assert float((blind[late] - expected[late]).abs().max()) > 4 * bound, (early, late)
    session = Session([part.cache_need()], dtype, page_size=page, num_pages=32)
    for name, cuts in (("whole", [total]), ("decoded", [100] + [1] * 320)):
        at, rows = 0, []
        for n in cuts:
            batch = session.batch([(name, n)])
            rows.append(part.forward(x[at : at + n].to(DEV), batch, session.cache.layer_view(0), True).cpu())
            session.commit()
            at += n
        assert float((torch.cat(rows) - expected).abs().max()) <= bound, name
        session.cache.close(session.requests.pop(name))


# --------------------------------------------------------------------------- whole models (GPU)
@pytest.fixture(scope="module", params=["P", "Q"])
def tiny(request, tmp_path_factory):
    raw, page, seed = TINY[request.param]
    folder = str(tmp_path_factory.mktemp(f"zoferax{request.param}"))
    write_model(folder, raw, seed)
    config, weights = read_model_folder(folder)
    assert config == raw
    sequences = {rid: random_tokens(n, raw["vocab"], 200 + k)
                 for k, (rid, n) in enumerate([("a", 75), ("b", 40), ("c", 53), ("d", 9), ("e", 61), ("f", 34)])}
    reference = {rid: reference_with_close_calls(config, weights, toks) for rid, toks in sequences.items()}
    return dict(name=request.param, folder=folder, raw=raw, config=config, weights=weights, page=page,
                sequences=sequences, reference=reference)


CLOSE_CALL = 0.03  # a router margin below this may fall the other way once activations are rounded to bfloat16


class Reference(np.ndarray):
    """Plain logits [T, vocab] with ``close`` [T]: whether a token's choice of experts is a close call in some layer.
    Such a token may take other experts in bfloat16 and then differs by far more than rounding; it is compared in
    32-bit only.  (A configuration has few of them: see ``test_close_calls_are_few``.)"""


def reference_with_close_calls(config, weights, tokens):
    margins = []
    logits = plain.forward(config, weights, tokens, margins=margins).numpy().view(Reference)
    logits.close = (torch.stack(margins).min(dim=0).values < CLOSE_CALL).numpy() if margins else np.zeros(len(tokens), bool)
    return logits


def check(dtype, got, reference, rows, what):
    expected = np.asarray(reference)[rows]
    assert got.shape == expected.shape, what
    diff = np.abs(got - expected).max(axis=1)
    if dtype in ("bfloat16", torch.bfloat16):
        diff = np.where(reference.close[rows], 0.0, diff)
    assert float(diff.max()) <= tolerance(dtype, reference), f"{what}: max abs diff {float(diff.max())} (bound {tolerance(dtype, reference)})"


@pytest.mark.gpu
def test_close_calls_are_few(tiny):
    """The tokens left out of the bfloat16 comparisons are a small share, so the comparisons still cover portions'
    edges, page borders and decoded tokens."""
    for rid, reference in tiny["reference"].items():
        assert reference.close.mean() <= 0.4, rid


@pytest.mark.gpu
def test_residual_stream_after_every_layer(tiny):
    """In 32-bit the stream after each layer equals the plain one: embedding, each layer's attention and experts."""
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner
    from kirai_b200.parts.block import Block

    runner = ModelRunner.from_folder(tiny["folder"], dtype="float32", page_size=tiny["page"], max_tokens=128, num_slots=2)
    tokens = tiny["sequences"]["b"]
    _, streams = plain.forward(tiny["config"], tiny["weights"], tokens, keep_layers=True)
    kept, original = [], Block.forward

    def recording(self, resid, *args, **kwargs):
        out = original(self, resid, *args, **kwargs)
        kept.append(out[0].clone())
        return out

    Block.forward = recording
    try:
        runner.step([StepEntry(runner.cache.open("b"), tokens, [0])])
    finally:
        Block.forward = original
    assert len(kept) == streams.shape[0]
    for index, stream in enumerate(kept):
        assert float((stream.cpu() - streams[index]).abs().max()) < 1e-4, f"after layer {index}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_last_tokens_one_by_one(tiny, dtype, tmp_path):
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=160, page_size=tiny["page"])
    for rid in ("a", "d"):
        toks = tiny["sequences"][rid]
        got = replay.step([(rid, toks, range(len(toks)))], end=[rid])
        check(dtype, got, tiny["reference"][rid], list(range(len(toks))), f"whole {rid}")
    for rid in ("a", "c"):
        toks = tiny["sequences"][rid]
        head = len(toks) - 32
        got = replay.step([(rid, toks[:head], [head - 1])])
        check(dtype, got, tiny["reference"][rid], [head - 1], f"{rid} prompt")
        for i in range(head, len(toks)):
            got = replay.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
            check(dtype, got, tiny["reference"][rid], [i], f"{rid} decode at {i}")
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(tiny, dtype, tmp_path):
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=96, page_size=tiny["page"])
    toks = tiny["sequences"]["a"]
    for sizes in ([13, 2, 7, 16, 5, 3, 2, 11, 9, 2, 5], [2] * 37 + [1], [64, 11]):
        assert sum(sizes) == len(toks)
        start = 0
        for size in sizes:
            got = replay.step([("a", toks[start : start + size], range(size))])
            check(dtype, got, tiny["reference"]["a"], list(range(start, start + size)), f"portion at {start}+{size}")
            start += size
        replay.step([], end=["a"])
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_on_a_pool_that_runs_full(tiny, dtype, tmp_path):
    """Six unequal requests, at most four live, portions of some beside single tokens of others, on a pool exactly as
    large as the most that live requests hold at once: later requests get pages that earlier ones gave back, and
    every logit equals what the request gives alone."""
    from replay_client import Replay
    from test_replay import mixed_schedule, tokens_held_at_most

    sequences, reference, page = tiny["sequences"], tiny["reference"], tiny["page"]
    steps = mixed_schedule(sequences)
    most = tokens_held_at_most(steps, page)
    everything = sum(-(-len(tokens) // page) * page for tokens in sequences.values())
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=most, page_size=page,
                    extra=("--stats", str(tmp_path / "out" / "stats.json"), "--max-requests", "4"))
    for entries, end in steps:
        batch = [(rid, sequences[rid][first : first + count], range(count)) for rid, first, count in entries]
        got = replay.step(batch, end=end)
        row = 0
        for rid, first, count in entries:
            check(dtype, got[row : row + count], reference[rid], list(range(first, first + count)), f"mixed {rid} at {first}+{count}")
            row += count
    assert replay.close() == 0
    stats = replay.stats()
    assert stats["live_requests"] == 0
    for group in stats["groups"]:
        assert group["pages"] == most // page == group["high_water"] and group["used"] == 0
        assert group["handed_out"] == everything // page > group["pages"]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(tiny, dtype, tmp_path):
    from replay_client import Replay

    toks = random_tokens(330, tiny["raw"]["vocab"], 17)
    reference = reference_with_close_calls(tiny["config"], tiny["weights"], toks)
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=352, page_size=tiny["page"])
    for i, token in enumerate(toks):
        got = replay.step([("long", [token], [0])])
        check(dtype, got, reference, [i], f"decode at {i}")
    assert replay.close() == 0


@pytest.mark.gpu
def test_bounds_would_show_a_lost_key_or_a_wrong_expert(tiny):
    """The bfloat16 bound is far below what a fault costs: the first key of a sequence lost, or the chosen experts
    weighted equally instead of by their softmax.  (Weights that are off by a factor common to a token's experts would
    not show: the norm on the feed-forward's output removes it.)"""
    tokens, true = tiny["sequences"]["a"], np.asarray(tiny["reference"]["a"])
    bound = tolerance("bfloat16", true)
    original = plain.causal_attention

    def blind_to_first(q, k, v, *args):
        k = k.clone()
        k[0] = -k[0]
        return original(q, k, v, *args)

    plain.causal_attention = blind_to_first
    try:
        other = plain.forward(tiny["config"], tiny["weights"], tokens).numpy()
    finally:
        plain.causal_attention = original
    assert float(np.abs(other[8:] - true[8:]).max()) > 3 * bound
    original_router = plain.routed_experts

    def equal_weights(x, weights, prefix, count, top, margins=None):
        logits = plain.projection(x, weights[prefix + "router"])
        out = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for e in torch.topk(logits[t], top).indices.tolist():
                out[t] += (1.0 / top) * plain.projection(plain.relu_squared(plain.projection(x[t], weights[f"{prefix}e{e}.up"])), weights[f"{prefix}e{e}.down"])
        return out

    plain.routed_experts = equal_weights
    try:
        other = plain.forward(tiny["config"], tiny["weights"], tokens).numpy()
    finally:
        plain.routed_experts = original_router
    assert float(np.abs(other - true).max()) > 3 * bound


# R: sizes at which steps of many tokens sort their rows by expert and take the router's tensor-core product (width and
# expert size multiples of 128), with a sharing layer.
CONFIG_R = {
    "architecture": "Zoferax", "width": 128, "vocab": 160, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
    "layers": [
        layer(attention(2, 1, 32, 16, 0.3), experts(4, 2, 128)),
        layer(attention(2, 1, 32, 16, 0.3, kv_from=0), experts(6, 1, 128)),
    ],
}


# S: sizes between the tiny ones and a real model's: heads of 96 with values of 48 (cache rows that are no power of two),
# eight experts, three layers of which the middle one shares and has no feed-forward.
CONFIG_S = {
    "architecture": "Zoferax", "width": 256, "vocab": 160, "embedding": {"scale": 16.0}, "norm": {"eps": 1e-6},
    "layers": [
        layer(attention(4, 2, 96, 48, 0.1), experts(8, 2, 64)),
        layer(attention(8, 2, 96, 48, 0.1, kv_from=0), None),
        layer(attention(2, 1, 40, 72, 0.15), experts(8, 2, 64)),
    ],
}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("raw", [CONFIG_R, CONFIG_S], ids=["R", "S"])
def test_long_prompts_whole_in_portions_and_beside_decoded_tokens(raw, dtype, tmp_path):
    """A prompt of 400 tokens in one step (in R 800 and 400 pairs of token and expert: the first layer sorts them, in
    bfloat16), then in portions that stay below the threshold, then a mixed step in which a long portion rides beside
    decoded tokens of another request: the same logits every way."""
    from replay_client import Replay

    folder = str(tmp_path / "model")
    write_model(folder, raw, 6)
    config, weights = read_model_folder(folder)
    long_tokens, short_tokens = random_tokens(400, 160, 31), random_tokens(40, 160, 32)
    reference = {"long": reference_with_close_calls(config, weights, long_tokens),
                 "short": reference_with_close_calls(config, weights, short_tokens)}
    assert reference["long"].close.mean() <= 0.4
    replay = Replay(folder, dtype, str(tmp_path / "out"), max_tokens=480, page_size=16)
    got = replay.step([("long", long_tokens, range(400))], end=["long"])
    check(dtype, got, reference["long"], list(range(400)), "whole")
    start = 0
    for size in (130, 7, 130, 133):
        got = replay.step([("again", long_tokens[start : start + size], range(size))])
        check(dtype, got, reference["long"], list(range(start, start + size)), f"portion at {start}+{size}")
        start += size
    replay.step([], end=["again"])
    got = replay.step([("short", short_tokens[:30], [29])])
    check(dtype, got, reference["short"], [29], "short prompt")
    got = replay.step([("short", [short_tokens[30]], [0]), ("third", long_tokens[:300], range(300))])
    check(dtype, got[:1], reference["short"], [30], "decoded beside a long portion")
    check(dtype, got[1:], reference["long"], list(range(300)), "long portion beside a decoded token")
    assert replay.close() == 0


def _margin_ok(config, weights, prompt, generated):
    logits = plain.forward(config, weights, list(prompt) + list(generated))
    top2 = torch.topk(logits[len(prompt) - 1 : -1], 2, dim=-1).values
    return bool(((top2[:, 0] - top2[:, 1]) > 2e-3).all())


def _plain_greedy(config, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits = plain.forward(config, weights, tokens)[-1]
        tokens.append(int(torch.nonzero(logits == logits.max())[0]))
    return tokens[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tiny, dtype):
    """Five prompts through the scheduler (three at a time, prompts in portions of 16, decode steps from captured
    graphs where the engine captures them) give the plain implementation's greedy tokens."""
    from kirai_b200 import Engine, SamplingParams

    engine = Engine(tiny["folder"], dtype=dtype, page_size=tiny["page"], max_prefill_tokens=16, max_concurrent_requests=3,
                    max_new_tokens=16, max_cache_tokens=256)
    prompts = [random_tokens(n, tiny["raw"]["vocab"], 50 + n) for n in (5, 11, 17, 3, 24)]
    outputs = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    compared = 0
    for prompt, output in zip(prompts, outputs):
        expected = _plain_greedy(tiny["config"], tiny["weights"], prompt, 8)
        assert output.finish_reason == "length" and (output.prompt_tokens, output.completion_tokens) == (len(prompt), 8)
        if dtype == "float32" or _margin_ok(tiny["config"], tiny["weights"], prompt, expected):
            assert output.token_ids == expected
            compared += 1
    assert compared >= 3
    stats = engine.stats()
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])


@pytest.mark.gpu
def test_eviction_and_recompute_give_the_same_sampled_tokens(tiny):
    """Seeded temperature sampling on a pool too small for both requests: one is evicted, its pages (of every layer
    that has keys of its own) go back, and its recomputation gives the tokens of the roomy run."""
    from kirai_b200 import Engine, SamplingParams

    params = SamplingParams(temperature=0.8, top_p=0.95, seed=5, max_new_tokens=14)
    prompts = [random_tokens(17, tiny["raw"]["vocab"], 1), random_tokens(18, tiny["raw"]["vocab"], 2)]
    roomy = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=256)
    expected = [o.token_ids for o in roomy.generate(prompts, params)]
    tight = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=48)
    outputs = tight.generate(prompts, params)
    assert [o.token_ids for o in outputs] == expected
    assert tight.stats()["scheduler"]["preemptions"] >= 1 and sum(o.preemptions for o in outputs) >= 1


@pytest.mark.gpu
def test_command_line_generates(tiny):
    prompt = random_tokens(9, tiny["raw"]["vocab"], 77)
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kirai"), "generate", "--snapshot", tiny["folder"],
                             "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                             "--dtype", "float32", "--page-size", str(tiny["page"])], capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    expected = _plain_greedy(tiny["config"], tiny["weights"], prompt, 6)
    assert json.loads(result.stdout.strip().splitlines()[-1])["token_ids"] == expected

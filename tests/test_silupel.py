"""The Silupel decoder against its plain implementation (``plain_silupel``): each mechanism alone (layer norm, token
shift, the minGRU recurrence walked and scanned, the stretched rotation table, attention with its rotated part, head
factors, soft cap, chunked mask and gate, latent attention, the gelu feed-forward), then whole models through trace
replay (whole, decoded one by one, in portions down to two tokens, mixed batches on a pool that runs full, long
prompts on the tensor-core kernels) and greedy generation through the engine and the command line.

Configurations and weights are made here.  Score factors are large enough that much of a query's weight sits on a few
keys, far back and at page and chunk borders alike; where random weights would still hide a fault (a key just outside
a chunk, a key hundreds of tokens back) the test scales single rows so that the key shows."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_silupel as plain
from plain_qwen3 import read_model_folder
from tiny_configs import random_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


def attn(heads, kv_heads, dim, vdim, scale, rotation, softcap=None, chunk=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation}
    if softcap:
        mixer["softcap"] = softcap
    if chunk:
        mixer["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": mixer}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                                                  "kv_rank": kv_rank, "scale": scale, "rot": rot(base, rot_dim, scaling)}}


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def layer(entry, ff):
    return {**entry, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# A: sizes in multiples of 8; a looped stretch in the middle; a chunk of two pages; an attention layer with neither
# chunk nor cap and a fully rotated head; a latent layer without feed-forward.  B: nothing a multiple of 8 (width,
# heads, ranks), no loop, one kv head for six query heads, a chunk of 5 tokens on pages of 8, two recurrent layers in
# a row, values wider than keys, a latent layer first.
CONFIG_A = {
    "architecture": "Silupel", "width": 64, "vocab": 200, "norm": {"eps": 1e-5},
    "layers": [
        layer(gru(48), 96),
        layer(attn(4, 2, 16, 8, 3.0, rot(500.0, 8, (4.0, 1.0, 4.0, 32)), softcap=6.0, chunk=8), 96),
        layer(latent(4, 8, 8, 16, 24, 16, 1.5), None),
        layer(attn(2, 2, 32, 32, 2.0, rot(10000.0, 32)), 80),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
CONFIG_B = {
    "architecture": "Silupel", "width": 100, "vocab": 131, "norm": {"eps": 1e-3},
    "layers": [
        layer(latent(6, 10, 6, 12, 20, 18, 1.2, base=300.0, scaling=(2.0, 1.0, 3.0, 16)), 60),
        layer(attn(6, 1, 12, 20, 2.0, rot(77.0, 4), softcap=3.5, chunk=5), 52),
        layer(gru(36), None),
        layer(gru(100), 36),
    ],
}
TINY = {"A": (CONFIG_A, 4, 11), "B": (CONFIG_B, 8, 12)}  # name -> (config, page size, seed)


def write_model(folder, raw, seed, std=0.08):
    import kirai_b200  # noqa: F401
    from kirai_b200.registry import config_from_dict
    from kirai_b200.weights import write_random_model

    write_random_model(folder, config_from_dict(raw), seed, std=std, norm_jitter=0.3, dtype=torch.bfloat16)


def tolerance(dtype, reference):
    dtype = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(dtype, dtype)
    peak = float(np.abs(np.asarray(reference)).max())
    return 3e-5 * max(1.0, peak) if dtype == "float32" else 0.035 * peak


def close(dtype, got, expected, what):
    got, expected = np.asarray(got, dtype=np.float64), np.asarray(expected, dtype=np.float64)
    assert got.shape == expected.shape, what
    worst = float(np.abs(got - expected).max())
    assert worst <= tolerance(dtype, expected), f"{what}: max abs diff {worst} (bound {tolerance(dtype, expected)})"


# --------------------------------------------------------------------------- no GPU
def test_config_reads_every_size_and_round_trips():
    import kirai_b200  # noqa: F401
    from kirai_b200.config.base import ConfigError
    from kirai_b200.parts.base import KVCacheNeed, StateNeed
    from kirai_b200.registry import config_from_dict, plan_for_config

    for raw in (CONFIG_A, CONFIG_B):
        cfg = config_from_dict(raw)
        assert cfg.to_dict() == raw and config_from_dict(cfg.to_dict()) == cfg
        assert list(cfg.layer_runs()) == plain.layer_runs(raw)
        plan = plan_for_config(cfg)
        runs = plain.layer_runs(raw)
        assert [call.block for call in plan.order] == runs
        assert len(plan.cache_needs) == 2 * len(runs)  # every run: its mixer's cache and its shift's slot
        for call in plan.order:
            kind = raw["layers"][call.block]["type"]
            need, shift = plan.cache_needs[call.cache], plan.cache_needs[call.shift_cache]
            assert shift == StateNeed((raw["width"],), torch.float32)
            if kind == "mingru":
                assert need == StateNeed((raw["layers"][call.block]["mixer"]["width"],), torch.float32)
            elif kind == "latent_attention":
                m = raw["layers"][call.block]["mixer"]
                assert isinstance(need, KVCacheNeed) and need.kv_heads == 1 and need.key_dim == m["kv_rank"] + m["rot_dim"]
            else:
                assert isinstance(need, KVCacheNeed) and need.kv_heads == raw["layers"][call.block]["mixer"]["kv_heads"]
        names = set(plan.weight_specs())
        for i, entry in enumerate(raw["layers"]):
            assert f"l{i}.shift" in names and (f"l{i}.norm2" in names) == (entry["mlp"] is not None) == (f"l{i}.mlp.gate" in names)
            assert (f"l{i}.mix.temp" in names) == (entry["type"] == "attention") == (f"l{i}.mix.o.b" in names)
            assert (f"l{i}.mix.dkv.norm" in names) == (entry["type"] == "latent_attention")
            assert (f"l{i}.mix.z.b" in names) == (entry["type"] == "mingru")
    for change in (lambda r: r["layers"][0].update(type="convolution"),
                   lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7),
                   lambda r: r["layers"][1]["mixer"].update(kv_heads=3),
                   lambda r: r["layers"][2]["mixer"].update(rot_dim=4),
                   lambda r: r.update(loop={"start": 2, "stop": 9, "times": 2}),
                   lambda r: r["layers"][0]["mlp"].update(kind="moe")):
        bad = json.loads(json.dumps(CONFIG_A))
        change(bad)
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_stretched_frequencies_cover_the_three_ranges():
    """Of the table of layer 1 of A (base 500, 8 dims, original 32, low 1, high 4, factor 4): wavelength 2 pi < 8 stays,
    wavelengths beyond 32 are divided by 4, the one between is blended."""
    import math

    import kirai_b200  # noqa: F401
    from kirai_b200.parts import RotaryEmbedding

    table = plain.rotary_frequencies(CONFIG_A["layers"][1]["mixer"]["rot"])
    raw = [500.0 ** (-2.0 * i / 8) for i in range(4)]
    assert [2 * math.pi / f for f in raw][0] < 8 < [2 * math.pi / f for f in raw][1] < 32 < [2 * math.pi / f for f in raw][2]
    assert table[0] == raw[0] and abs(table[2] - raw[2] / 4) < 1e-15 and abs(table[3] - raw[3] / 4) < 1e-15
    assert raw[1] / 4 < table[1] < raw[1]
    part = RotaryEmbedding(16, 500.0, 8, scaling={"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32})
    assert torch.equal(part.frequencies(), table.to(torch.float32))


def test_plain_attention_is_peaky_reaches_far_back_and_feels_its_chunk(tmp_path):
    """What makes the comparisons below sharp: the heaviest key of many queries carries much of the weight and lies
    many pages back (latent and unmasked layers), and dropping the chunked mask changes the model's logits by far
    more than any bound used below."""
    write_model(str(tmp_path), CONFIG_A, 11)
    raw, weights = read_model_folder(str(tmp_path))
    tokens = random_tokens(75, raw["vocab"], 200)
    w = {k: v.double() for k, v in weights.items()}
    n = plain.token_shift(plain.layer_norm(w["embed"][tokens], w["l3.norm1"], 1e-5), w["l3.shift"])
    probabilities = []
    plain.attention(n, w, raw["layers"][3]["mixer"], "l3.mix.", probabilities)
    far = sum(int(((p.max(dim=1).values > 0.3) & (torch.arange(75) - p.argmax(dim=1) > 16)).sum()) for p in probabilities)
    assert far >= 5
    unmasked = json.loads(json.dumps(raw))
    del unmasked["layers"][1]["mixer"]["mask"]
    logits = plain.forward(raw, weights, tokens)
    assert float((plain.forward(unmasked, weights, tokens) - logits).abs().max()) > 10 * tolerance("bfloat16", logits.numpy())


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 100, 7, 4096 + 24])
def test_layer_norm_with_add_bias_and_chosen_rows(dtype, width):
    from part_helpers import load_part, runtime
    from kirai_b200.parts import LayerNorm

    norm = LayerNorm("n", width, 1e-4)
    w = load_part(norm, dtype, seed=width)["n"].double()
    g = torch.Generator().manual_seed(width)
    x = torch.randn((9, width), generator=g) * 3 + 1.5
    delta = torch.randn((9, width), generator=g).to(dtype)
    bias = torch.randn((width,), generator=g)
    resid = x.cuda()
    got = norm.add_forward(resid, delta.cuda(), delta_bias=bias.cuda())
    total = x.double() + delta.double() + bias.double()
    close(torch.float32, resid.cpu(), total.float(), "the stream")
    close(dtype, got.float().cpu(), plain.layer_norm(total, w, 1e-4), "normed rows")
    wide = norm.add_forward(resid, None, wide=True)
    assert wide.dtype == torch.float32
    close(torch.float32, wide.cpu(), plain.layer_norm(total, w, 1e-4), "normed rows in 32-bit")
    rows = torch.tensor([7, 2, 2], dtype=torch.int32).cuda()
    before = resid.clone()
    picked = norm.add_forward_rows(resid, delta.cuda(), rows)
    assert torch.equal(resid, before)
    close(dtype, picked.float().cpu(), plain.layer_norm(total + delta.double(), w, 1e-4)[[7, 2, 2]], "chosen rows")
    assert runtime(dtype).dtype == dtype


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_token_shift_carries_the_last_row_between_steps_and_starts_from_zero(dtype):
    from part_helpers import Session, load_part
    from kirai_b200.parts import TokenShift

    width = 40
    shift = TokenShift("mu", width)
    mu = load_part(shift, dtype, seed=3)["mu"].double() * 8
    shift.weight = mu.float().cuda()
    session = Session([shift.cache_need()], dtype, num_slots=2)
    g = torch.Generator().manual_seed(1)
    rows = {name: torch.randn((n, width), generator=g) for name, n in (("p", 11), ("q", 6), ("r", 5))}
    expected = {name: plain.token_shift(r.double(), mu) for name, r in rows.items()}
    done = {name: 0 for name in rows}
    # unequal runs side by side, runs of one token, a request that sits a step out
    for step in ([("p", 4), ("q", 1)], [("q", 2), ("p", 1)], [("p", 1)], [("q", 3), ("p", 5)]):
        batch = session.batch([(name, count) for name, count in step])
        order = [name for name, count in step if count == 1] + [name for name, count in step if count != 1]
        x = torch.cat([rows[name][done[name] : done[name] + dict(step)[name]] for name in order]).cuda()
        got = shift.forward(x, batch, session.cache.layer_view(0)).float().cpu()
        at = 0
        for name in order:
            count = dict(step)[name]
            close(dtype, got[at : at + count], expected[name][done[name] : done[name] + count], f"{name} at {done[name]}")
            at, done[name] = at + count, done[name] + count
        session.commit()
    # a slot that is given back and used again starts from zeros
    session.cache.close(session.requests.pop("q"))
    batch = session.batch([("r", 5)])
    got = shift.forward(rows["r"].cuda(), batch, session.cache.layer_view(0)).float().cpu()
    close(dtype, got, expected["r"], "a request in a used slot")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 100, 7, 2048 + 8])
def test_norm_and_shift_in_one_kernel_for_steps_of_single_tokens(dtype, width):
    """Three requests, one token each a step: the norm's kernel mixes its row with the request's slot and leaves the
    row there; over five steps that equals norm then shift over each request's five rows."""
    from part_helpers import Session, load_part
    from kirai_b200.parts import LayerNorm, TokenShift

    norm, shift = LayerNorm("n", width, 1e-5), TokenShift("mu", width)
    w = load_part(norm, dtype, seed=1)["n"].double()
    mu = load_part(shift, dtype, seed=2)["mu"].double() * 6
    shift.weight = mu.float().cuda()
    session = Session([shift.cache_need()], dtype, num_slots=4)
    g = torch.Generator().manual_seed(width)
    streams = {name: torch.randn((5, width), generator=g) * 2 for name in "pqr"}
    deltas = {name: torch.randn((5, width), generator=g).to(dtype) for name in "pqr"}
    expected = {name: plain.token_shift(plain.layer_norm(streams[name].double() + deltas[name].double(), w, 1e-5), mu) for name in "pqr"}
    for t in range(5):
        batch = session.batch([(name, 1) for name in "pqr"])
        resid = torch.stack([streams[name][t] for name in "pqr"]).cuda()
        delta = torch.stack([deltas[name][t] for name in "pqr"]).cuda()
        got = norm.add_forward(resid, delta, shift=shift.fused_args(batch, session.cache.layer_view(0))).float().cpu()
        for row, name in enumerate("pqr"):
            close(dtype, got[row], expected[name][t], f"{name} at {t}")
        session.commit()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,hidden", [(48, 64), (36, 100), (7, 24), (200, 64)])
def test_mingru_walked_scanned_and_carried(dtype, width, hidden):
    """The recurrence over runs of 1 to 150 tokens, cut into steps in three ways; runs above the walk limit take the
    scan over pieces (one run ends inside a piece, one on a piece's border), and the state is carried in the slot.
    Gate biases are pushed towards -4, so that a state remembers hundreds of tokens and a lost carry shows."""
    from part_helpers import Session, load_part
    from kirai_b200.csrc import ops
    from kirai_b200.parts import MinGRU

    part = MinGRU("m.", hidden, width)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=width).items()}
    w["m.z.b"] = w["m.z.b"] * 10 - 4.0
    w["m.x.b"] = w["m.x.b"] * 10
    part.z_bias, part.x_bias = w["m.z.b"].float().cuda(), w["m.x.b"].float().cuda()
    g = torch.Generator().manual_seed(5)
    x = {name: (torch.randn((n, hidden), generator=g) * 4).to(dtype) for name, n in (("p", 150), ("q", 64 + 17), ("r", 9))}
    m = {"width": width}
    expected = {name: plain.mingru(rows.double(), w, m, "m.") for name, rows in x.items()}
    for cuts in ({"p": [150], "q": [64, 17], "r": [9]}, {"p": [1, 2, 128, 19], "q": [17, 1, 63], "r": [2, 2, 1, 1, 3]},
                 {"p": [70, 1, 1, 1, 77], "q": [1] * 5 + [76], "r": [8, 1]}):
        session = Session([part.cache_need()], dtype, num_slots=4)
        done = {name: 0 for name in x}
        for step in range(max(len(c) for c in cuts.values())):
            runs = [(name, cuts[name][step]) for name in x if step < len(cuts[name])]
            batch = session.batch(runs)
            order = [name for name, count in runs if count == 1] + [name for name, count in runs if count != 1]
            rows = torch.cat([x[name][done[name] : done[name] + dict(runs)[name]] for name in order]).cuda()
            got = part.forward(rows, batch, session.cache.layer_view(0)).float().cpu()
            at = 0
            for name in order:
                count = dict(runs)[name]
                close(dtype, got[at : at + count], expected[name][done[name] : done[name] + count], f"{name} at {done[name]}+{count}")
                at, done[name] = at + count, done[name] + count
            session.commit()
    assert ops.MINGRU_WALK_LIMIT < 64  # the cuts above reach both forms


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff", [(64, 96), (100, 52), (24, 7)])
def test_gelu_gated_feed_forward(dtype, width, ff):
    from part_helpers import load_part
    from kirai_b200.parts import GatedMLP

    part = GatedMLP("f.", width, ff, "gelu_tanh", names={"gate": "gate", "up": "up", "down": "down"})
    w = {k: v.double() for k, v in load_part(part, dtype, seed=ff).items()}
    x = (torch.randn((13, width), generator=torch.Generator().manual_seed(ff)) * 12).to(dtype)  # gate values reach +-3
    got = part.forward(x.cuda(), None).float().cpu()
    close(dtype, got, plain.feed_forward(x.double(), w, "f."), "feed-forward")


def _attention_part(mixer, width):
    import kirai_b200  # noqa: F401
    from kirai_b200.models.silupel import mixer_for_layer
    from kirai_b200.config.silupel import SilupelConfig

    raw = {"architecture": "Silupel", "width": width, "vocab": 8, "norm": {"eps": 1e-5}, "layers": [layer(mixer, None)]}
    cfg = SilupelConfig.from_dict(raw)
    return mixer_for_layer(cfg, cfg.layers[0], "a."), raw["layers"][0]


def _run_part(part, session, x, cuts, name="s"):
    """The part's output for rows x of one request, cut into steps of the given sizes."""
    out, start = [], 0
    for size in cuts:
        batch = session.batch([(name, size)])
        out.append(part.forward(x[start : start + size].cuda(), batch, session.cache.layer_view(0)).float().cpu())
        session.commit()
        start += size
    session.cache.close(session.requests.pop(name))
    return torch.cat(out)


PART_CASES = [
    (attn(4, 2, 16, 8, 3.0, rot(500.0, 8, (4.0, 1.0, 4.0, 32)), softcap=6.0, chunk=8), 64, 4),
    (attn(6, 1, 12, 20, 4.0, rot(77.0, 4), softcap=3.5, chunk=5), 100, 8),
    (attn(2, 2, 32, 32, 2.0, rot(10000.0, 32)), 64, 4),
    (attn(3, 3, 10, 10, 2.5, rot(50.0, 10), chunk=1), 24, 2),
    (attn(8, 2, 64, 64, 0.8, rot(10000.0, 48), softcap=9.0, chunk=48), 128, 16),
    (latent(4, 8, 8, 16, 24, 16, 1.5), 64, 4),
    (latent(6, 10, 6, 12, 20, 18, 1.2, base=300.0, scaling=(2.0, 1.0, 3.0, 16)), 100, 8),
    (latent(20, 16, 16, 8, 32, 48, 0.9), 64, 16),
    (latent(1, 24, 2, 24, 8, 30, 1.0), 40, 2),
    (latent(8, 32, 64, 32, 64, 192, 0.6), 128, 16),   # a cached row of 256 columns
    (latent(4, 16, 32, 24, 40, 168, 0.6), 96, 8),     # a row of 200 columns
    (attn(4, 2, 256, 136, 0.4, rot(10000.0, 64), softcap=15.0, chunk=40), 128, 16),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry,width,page", PART_CASES, ids=[f"{e['type']}{i}" for i, (e, _, _) in enumerate(PART_CASES)])
def test_attention_parts_whole_in_portions_and_one_by_one(dtype, entry, width, page):
    from part_helpers import Session, load_part

    part, raw = _attention_part(entry, width)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=width + page).items()}
    tokens = 90
    x = (torch.randn((tokens, width), generator=torch.Generator().manual_seed(page)) * 1.5).to(dtype)
    if raw["type"] == "attention":
        expected = plain.attention(x.double(), w, raw["mixer"], "a.")
    else:
        expected = plain.latent_attention(x.double(), w, raw["mixer"], "a.", 1e-5)
    session = Session([part.cache_need()], dtype, page_size=page, num_pages=2 * (-(-tokens // page)), num_slots=2)
    for cuts in ([tokens], [37, 2, 19, 1, 1, 3, 27], [80] + [1] * 10, [2] * 45):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:4]}...")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_just_inside_and_just_outside_a_chunk_show(dtype):
    """Rows 47 and 48 are made thirty times larger than the rest, with chunks of 48: row 47 is the last key of the
    first chunk, row 48 the first of the second.  Queries 48.. must not see row 47 (whose values would swamp them)
    and must see row 48; query 47 sees itself.  In a prompt portion that crosses the border and decoded one by one."""
    from part_helpers import Session, load_part

    entry = attn(8, 2, 64, 64, 0.8, rot(10000.0, 48), softcap=9.0, chunk=48)
    part, raw = _attention_part(entry, 128)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=9).items()}
    x = torch.randn((70, 128), generator=torch.Generator().manual_seed(2)) * 1.5
    x[47] *= 30
    x[48] *= 30
    x = x.to(dtype)
    expected = plain.attention(x.double(), w, raw["mixer"], "a.")
    off_by_one = json.loads(json.dumps(raw["mixer"]))
    for size in (47, 49):
        off_by_one["mask"]["size"] = size
        wrong = plain.attention(x.double(), w, off_by_one, "a.")
        assert float((wrong - expected)[44:54].abs().max()) > 20 * tolerance(dtype, expected.numpy())
    session = Session([part.cache_need()], dtype, page_size=16, num_pages=16, num_slots=2)
    for cuts in ([70], [40, 30], [47, 1, 1, 21], [46] + [1] * 24):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:4]}...")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
def test_a_far_key_that_stands_out(dtype, kind):
    """Among 600 keys, those at positions 3 to 12 are made the heaviest for the last ten queries: the first key head
    gets the first query head's weights, and each of the last rows repeats one of those far rows, so that its query
    equals that far key (up to the rotated part).  The output must follow it, in a prompt and decoded."""
    from part_helpers import Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    entry = attn(4, 2, 64, 64, 0.5, rot(10000.0, 4)) if kind == "attention" else latent(4, 32, 16, 32, 48, 48, 0.8)
    part, raw = _attention_part(entry, 96)
    tensors = random_tensors(part.weight_specs(), 21, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    if kind == "attention":
        tensors["a.k"][:64] = tensors["a.q"][:64]
        tensors["a.k.b"][:64] = tensors["a.q.b"][:64]
    else:
        tensors["a.dkv"][:48] = tensors["a.dq"]
        tensors["a.dkv.norm"] = tensors["a.dq.norm"].clone()
        tensors["a.uk"][:32] = tensors["a.uq"][:32]
    w = {k: v.double() for k, v in load_part(part, dtype, seed=21, tensors=tensors).items()}
    x = torch.randn((600, 96), generator=torch.Generator().manual_seed(8))
    x[590:] = x[3:13]
    x = x.to(dtype)
    probabilities = []
    if kind == "attention":
        expected = plain.attention(x.double(), w, raw["mixer"], "a.", probabilities)
    else:
        expected = plain.latent_attention(x.double(), w, raw["mixer"], "a.", 1e-5, probabilities)
    far = [float(probabilities[0][590 + i, 3 + i]) for i in range(10)]
    assert min(far) > 0.05 and max(far) > 0.3  # the far keys hold much of head 0's weight (one of 600 evenly: 0.002)
    session = Session([part.cache_need()], dtype, page_size=16, num_pages=80, num_slots=2)
    for cuts in ([600], [570] + [1] * 30, [300, 290, 10]):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:3]}...")


# ------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request, tmp_path_factory):
    raw, page, seed = TINY[request.param]
    folder = str(tmp_path_factory.mktemp(f"silupel_{request.param}"))
    write_model(folder, raw, seed)
    config, weights = read_model_folder(folder)
    assert config == raw
    sequences = {rid: random_tokens(n, raw["vocab"], 200 + k)
                 for k, (rid, n) in enumerate([("a", 75), ("b", 40), ("c", 53), ("d", 9), ("e", 61), ("f", 34)])}
    reference = {rid: plain.forward(config, weights, toks).numpy() for rid, toks in sequences.items()}
    return dict(name=request.param, folder=folder, raw=raw, config=config, weights=weights, page=page,
                sequences=sequences, reference=reference)


def check_rows(dtype, got, reference, rows, what):
    expected = np.asarray(reference)[rows]
    assert got.shape == expected.shape, what
    worst = float(np.abs(got - expected).max())
    assert worst <= tolerance(dtype, reference), f"{what}: max abs diff {worst} (bound {tolerance(dtype, reference)})"


@pytest.mark.gpu
def test_residual_stream_after_every_layer_run(tiny):
    """In 32-bit the stream after each layer run (a looped layer counts each time) equals the plain one."""
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner
    from kirai_b200.parts.block import Block

    runner = ModelRunner.from_folder(tiny["folder"], dtype="float32", page_size=tiny["page"], max_tokens=128, num_slots=2)
    tokens = tiny["sequences"]["b"]
    _, streams = plain.forward(tiny["config"], tiny["weights"], tokens, keep_layers=True)
    kept, original = [], Block.forward

    def recording(self, resid, *args, **kwargs):
        out = original(self, resid, *args, **kwargs)
        kept.append(out[0].clone() + (out[1].float() if torch.is_tensor(out[1]) else 0.0))
        return out

    Block.forward = recording
    try:
        runner.step([StepEntry(runner.cache.open("b"), tokens, [0])])
    finally:
        Block.forward = original
    assert len(kept) == streams.shape[0] == len(plain.layer_runs(tiny["raw"]))
    for index, stream in enumerate(kept):
        assert float((stream.cpu() - streams[index]).abs().max()) < 1e-4, f"after layer run {index}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_last_tokens_one_by_one(tiny, dtype, tmp_path):
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=160, page_size=tiny["page"])
    for rid in ("a", "d"):
        toks = tiny["sequences"][rid]
        got = replay.step([(rid, toks, range(len(toks)))], end=[rid])
        check_rows(dtype, got, tiny["reference"][rid], list(range(len(toks))), f"whole {rid}")
    for rid in ("a", "c"):
        toks = tiny["sequences"][rid]
        head = len(toks) - 40
        got = replay.step([(rid, toks[:head], [0, head - 1])])
        check_rows(dtype, got, tiny["reference"][rid], [0, head - 1], f"{rid} prompt")
        for i in range(head, len(toks)):
            got = replay.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
            check_rows(dtype, got, tiny["reference"][rid], [i], f"{rid} decode at {i}")
    # a sequence decoded from its very first token
    toks = tiny["sequences"]["f"]
    for i, token in enumerate(toks):
        got = replay.step([("f", [token], [0])], end=["f"] if i == len(toks) - 1 else [])
        check_rows(dtype, got, tiny["reference"]["f"], [i], f"f decode at {i}")
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(tiny, dtype, tmp_path):
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=96, page_size=tiny["page"])
    toks = tiny["sequences"]["a"]
    for sizes in ([13, 2, 7, 16, 5, 3, 2, 11, 9, 2, 5], [2] * 37 + [1], [64, 11], [1, 2, 72]):
        assert sum(sizes) == len(toks)
        start = 0
        for size in sizes:
            got = replay.step([("a", toks[start : start + size], range(size))])
            check_rows(dtype, got, tiny["reference"]["a"], list(range(start, start + size)), f"portion at {start}+{size}")
            start += size
        replay.step([], end=["a"])
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_on_a_pool_that_runs_full(tiny, dtype, tmp_path):
    """Six unequal requests, at most four live in four state slots, portions of some beside single tokens of others,
    on a pool exactly as large as the most that live requests hold at once: later requests get pages and slots that
    earlier ones gave back, and every logit equals what the request gives alone."""
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
            check_rows(dtype, got[row : row + count], reference[rid], list(range(first, first + count)), f"mixed {rid} at {first}+{count}")
            row += count
    assert replay.close() == 0
    stats = replay.stats()
    assert stats["live_requests"] == 0
    for group in stats["groups"]:
        assert group["pages"] == most // page == group["high_water"] and group["used"] == 0
        assert group["handed_out"] == everything // page > group["pages"]


# C: sizes of a small real model, on which bfloat16 takes the tensor-core kernels: heads of 64 in a group of 4 (the
# tcgen05 prompt kernel, the decode kernels), heads of 128 in a group of 3 with narrower values (the mma prompt
# kernel), a latent row of 128, chunks of 100 and 64 tokens on pages of 16, a stretch that runs twice.
CONFIG_C = {
    "architecture": "Silupel", "width": 256, "vocab": 320, "norm": {"eps": 1e-6},
    "layers": [
        layer(attn(8, 2, 64, 64, 0.9, rot(10000.0, 32, (8.0, 1.0, 4.0, 256)), softcap=12.0, chunk=100), 384),
        layer(latent(8, 32, 32, 32, 96, 96, 0.7), 384),
        layer(gru(256), None),
        layer(attn(6, 2, 128, 64, 0.6, rot(50000.0, 128), chunk=64), 256),
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_whole_in_portions_and_beside_decoded_tokens(dtype, tmp_path):
    from replay_client import Replay

    folder = str(tmp_path / "model")
    write_model(folder, CONFIG_C, 31, std=0.05)
    config, weights = read_model_folder(folder)
    long_a, long_b = random_tokens(650, 320, 1), random_tokens(420, 320, 2)
    ref_a, ref_b = plain.forward(config, weights, long_a).numpy(), plain.forward(config, weights, long_b).numpy()
    replay = Replay(folder, dtype, str(tmp_path / "out"), max_tokens=1200, page_size=16)
    want = [0, 63, 64, 99, 100, 101, 199, 200, 399, 400, 511, 512, 600, 649]
    got = replay.step([("a", long_a, want)], end=["a"])
    check_rows(dtype, got, ref_a, want, "whole")
    start = 0
    for size in (300, 2, 97, 1, 113, 87, 50):
        rows = sorted({0, size - 1, size // 2})
        got = replay.step([("a", long_a[start : start + size], rows)])
        check_rows(dtype, got, ref_a, [start + r for r in rows], f"portion at {start}+{size}")
        start += size
    assert start == 650
    # b's prompt in two portions beside nothing, then b decoding beside a second run of a's prompt
    got = replay.step([("b", long_b[:390], [389])], end=["a"])
    check_rows(dtype, got, ref_b, [389], "b prompt")
    position, a_at = 390, 0
    for size in (128, 2, 200, 1, 64, 255):
        entries = [("a2", long_a[a_at : a_at + size], [size - 1])]
        if position < 420:
            entries.append(("b", [long_b[position]], [0]))
        got = replay.step(entries)
        check_rows(dtype, got[:1], ref_a, [a_at + size - 1], f"a beside b at {a_at}+{size}")
        if position < 420:
            check_rows(dtype, got[1:], ref_b, [position], f"b decode at {position}")
            position += 1
        a_at += size
    while position < 420:
        got = replay.step([("b", [long_b[position]], [0])])
        check_rows(dtype, got, ref_b, [position], f"b decode at {position}")
        position += 1
    assert replay.close() == 0


def random_configuration(seed, wide=False):
    """A configuration drawn from sizes that are and are not multiples of 8, any order and number of layers, layers
    without feed-forward, every option present or absent, a loop over any stretch.  ``wide``: heads and latent rows of
    up to 256 columns, which the tensor-core kernels take in other forms than narrow ones."""
    import random

    r = random.Random(seed + (1000 if wide else 0))
    width = r.choice([32, 40, 72, 96, 130])
    layers = []
    for _ in range(r.randint(2, 5)):
        kind = r.choice(["mingru", "attention", "latent_attention"])
        if kind == "mingru":
            entry = gru(r.choice([8, 20, 64, 100]))
        elif kind == "attention":
            kv_heads, dim = r.choice([1, 2, 3, 4]), r.choice([96, 128, 136, 200, 256] if wide else [8, 12, 16, 24, 32, 40, 64])
            dims = r.choice([d for d in (2, 4, 6, 8, 16, 32, 64) if d <= dim] + [dim])
            scaling = r.choice([None, (r.choice([2.0, 8.0]), 1.0, r.choice([2.0, 4.0]), r.choice([8, 64]))])
            entry = attn(kv_heads * r.choice([1, 2, 3, 4, 5, 8]), kv_heads, dim, r.choice([64, 128, 160, 256] if wide else [8, 12, 16, 24, 32, 40, 64]),
                         r.uniform(0.5, 1.5) * 4 / dim ** 0.5, rot(r.choice([50.0, 10000.0, 1e6]), dims, scaling),
                         softcap=r.choice([None, 2.5, 8.0, 30.0]), chunk=r.choice([None, 1, 3, 7, 16, 33, 64, 200]))
        else:
            rot_dim = r.choice([2, 4, 6, 8, 16, 32])
            entry = latent(r.choice([1, 2, 4, 6, 8, 20]), r.choice([4, 8, 10, 16, 32]), rot_dim, r.choice([4, 8, 12, 16]),
                           r.choice([8, 20, 24, 48]), r.choice([100, 128, 192, 224] if wide else [6, 16, 18, 32, 64]), r.uniform(0.5, 1.5),
                           base=r.choice([100.0, 10000.0]), scaling=r.choice([None, (4.0, 1.0, 2.0, 16)]))
        layers.append(layer(entry, r.choice([None, 16, 36, 52, 96])))
    raw = {"architecture": "Silupel", "width": width, "vocab": r.choice([50, 97, 260]), "norm": {"eps": r.choice([1e-6, 1e-5, 1e-3])},
           "layers": layers}
    if r.random() < 0.6:
        start = r.randrange(len(layers))
        raw["loop"] = {"start": start, "stop": r.randint(start + 1, len(layers)), "times": r.randint(1, 3)}
    return raw, r.choice([4, 8, 16, 16])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(8)) + [-1, -2, -3, -4])
def test_random_configurations_whole_in_portions_and_mixed(seed, dtype, tmp_path):
    """Three requests of a randomly drawn configuration: one whole, one in portions with its last tokens one by one,
    and all three side by side in unequal runs, on four slots that are given back and used again."""
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner

    raw, page = random_configuration(abs(seed), wide=seed < 0)  # negative seeds draw wide heads and rows
    folder = str(tmp_path / "model")
    write_model(folder, raw, 100 + seed, std=0.05 if seed < 0 else 0.08)
    config, weights = read_model_folder(folder)
    sequences = {rid: random_tokens(n, raw["vocab"], 300 + seed + k) for k, (rid, n) in enumerate([("a", 83), ("b", 37), ("c", 58)])}
    reference = {rid: plain.forward(config, weights, toks).numpy() for rid, toks in sequences.items()}
    bound = {rid: (3e-5 * max(1.0, float(np.abs(ref).max())) if dtype == "float32" else 0.05 * float(np.abs(ref).max()))
             for rid, ref in reference.items()}
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=page, max_tokens=3 * 96, num_slots=4)

    def run(steps):
        live, done = {}, {rid: 0 for rid in sequences}
        for step in steps:
            entries, names = [], []
            for rid, count in step:
                if rid not in live:
                    live[rid] = runner.cache.open((rid, id(steps)))
                tokens = sequences[rid][done[rid] : done[rid] + count]
                entries.append(StepEntry(live[rid], tokens, list(range(count))))
                names.append((rid, done[rid], count))
                done[rid] += count
            logits = runner.step(entries).cpu().numpy()
            row = 0
            for rid, first, count in names:
                worst = float(np.abs(logits[row : row + count] - reference[rid][first : first + count]).max())
                assert worst <= bound[rid], f"{raw}: {rid} at {first}+{count}: max abs diff {worst} (bound {bound[rid]})"
                row += count
        for request in live.values():
            runner.cache.close(request)

    run([[("a", 83)]])
    run([[("b", 9)], [("b", 2)], [("b", 16)], [("b", 5)]] + [[("b", 1)]] * 5)
    run([[("a", 30), ("c", 1)], [("c", 1), ("b", 20)], [("a", 1), ("b", 1), ("c", 40)], [("a", 52), ("b", 16), ("c", 16)]])
    run([[("c", 58), ("a", 2)], [("a", 81), ("b", 37)]])


# ---------------------------------------------------------------------- generation
def _greedy_within_rounding(config, weights, prompt, generated, dtype):
    """Whether every generated token is the plain implementation's choice given the tokens before it, or, in bfloat16,
    as good as that choice within the bound on the logits (two logits closer than rounding may fall either way, and
    the sequences part from there on, so each token is judged after the tokens that were in fact generated)."""
    logits = plain.forward(config, weights, list(prompt) + list(generated))[len(prompt) - 1 : -1]
    slack = 0.0 if dtype == "float32" else 2 * tolerance(dtype, logits.numpy())
    chosen = logits[torch.arange(len(generated)), torch.tensor(generated)]
    return bool((chosen >= logits.max(dim=-1).values - slack).all())


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
    outputs = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10))
    compared = 0
    for prompt, output in zip(prompts, outputs):
        expected = _plain_greedy(tiny["config"], tiny["weights"], prompt, 10)
        assert output.finish_reason == "length" and (output.prompt_tokens, output.completion_tokens) == (len(prompt), 10)
        if dtype == "float32":
            assert output.token_ids == expected
        assert _greedy_within_rounding(tiny["config"], tiny["weights"], prompt, output.token_ids, dtype)
        compared += output.token_ids == expected
    assert compared >= (5 if dtype == "float32" else 1)
    stats = engine.stats()
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])
    if dtype == "bfloat16":
        assert engine.runner.model.plan.capture_safe()


@pytest.mark.gpu
def test_eviction_and_recompute_give_the_same_sampled_tokens(tiny):
    """Seeded temperature sampling on a pool too small for both requests: one is evicted, its pages and its state
    slot go back, and its recomputation (recurrent state and shift rows from zero again) gives the roomy run's tokens."""
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

"""The Sadosun decoder in the engine against the plain implementation
(``plain_sadosun.py``): its configuration and mechanisms one at a time, then
whole prompts layer by layer, decoding through the cache and the state,
portions, mixed batches, pages and slots that come back, keys at the window's
edge and at page borders, the first tokens, long decoding, generation through
the scheduler and the trace program. Every model here is tiny, made for the
test with random weights, and differs from layer to layer."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_sadosun as plain
import replay_helpers as cuts
from conftest import ROOT, random_ids


# ------------------------------------------------------------ configurations
def attention(heads, kv_heads, dim, vdim, scale, window, rot):
    out = {"heads": heads, "dim": dim, "scale": scale}
    if kv_heads:
        out["kv_heads"] = kv_heads
    if vdim:
        out["vdim"] = vdim
    if window:
        out["mask"] = {"size": window}
    if rot:
        out["rot"] = {"base": rot[0], "dims": rot[1]}
    return out


def scan(inner, state, rank, conv):
    return {"inner": inner, "state": state, "dt_rank": rank, "conv": conv}


def experts(ff, count, identity, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": count, "identity": identity, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# SMALL: sizes that are no power of two; values wider (24) and narrower (8)
# than keys; part of a head rotated; two query heads per key/value head and one;
# a window shorter than a page of 8 and one that spans several; a layer
# without feed-forward; identity experts 1, 2 and 0; top 1, 2 and 3; the
# block's convolutions (3 taps) unlike the mixers' (2 and 5).
SMALL = {"architecture": "Sadosun", "vocab": 211, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.7},
         "canon": {"taps": 3}, "token_side": {"dim": 10},
         "layers": [
             layer("mamba1", scan(40, 6, 5, 2), experts(24, 5, 1, 2)),
             layer("attention", attention(4, 2, 16, 24, 0.3, 5, (100.0, 8)), None),
             layer("attention", attention(3, 3, 12, 8, 0.45, 37, (1.0e4, 12)), experts(16, 3, 2, 3)),
             layer("mamba1", scan(100, 17, 3, 5), experts(40, 7, 0, 1))]}
# WIDE: heads of 64 and 128 values with values as wide as keys (the tensor-core
# kernels' sizes), windows that end inside a page of 16 and inside a key tile
# of 128, sixteen states a channel, more channels than a block of the scan.
WIDE = {"architecture": "Sadosun", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
        "canon": {"taps": 4}, "token_side": {"dim": 16},
        "layers": [
            layer("attention", attention(6, 2, 64, 64, 0.11, 70, (1.0e5, 64)), experts(48, 8, 3, 4)),
            layer("mamba1", scan(256, 16, 8, 4), None),
            layer("attention", attention(4, 1, 128, 128, 0.08, 150, (1.0e4, 32)), experts(32, 4, 1, 2))]}
# BARE: the switches' other position: no scale of the embedding, no convolution
# ahead of the sublayers, no input from the token, no window, no rotation, a
# key/value head per query head by default, values as wide as keys by default;
# every expert chosen; one real expert among three that return their input; a
# window of one position (a query sees itself alone); one state a channel.
BARE = {"architecture": "Sadosun", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
        "layers": [
            layer("attention", attention(2, 0, 8, 0, 0.5, 0, None), experts(20, 2, 0, 2)),
            layer("mamba1", scan(24, 1, 1, 2), None),
            layer("attention", attention(4, 4, 32, 32, 0.2, 1, (50.0, 2)), experts(8, 1, 3, 2))]}
MODELS = {"small": (SMALL, 31, 8, 1.0), "wide": (WIDE, 32, 16, 1.0), "bare": (BARE, 33, 4, 1.0),
          # score scales five times as large: which keys a query sees, and the sink, decide its output
          # (float32 only, a bound of its own)
          "sharp": (SMALL, 34, 8, 5.0)}
CASES = [(name, dtype) for name in MODELS for dtype in ("float32", "bfloat16") if (name, dtype) != ("sharp", "bfloat16")]
TOL = {"float32": 1e-4, "bfloat16": 2.5e-1}
TOL_SHARP = 5e-4


def bound(name, dtype):
    return TOL_SHARP if name == "sharp" else TOL[dtype]


def compare_replay(name, dtype, seen, reference):
    """Whether the logits a replay has seen are the plain side's. float32:
    every position within the bound. bfloat16: a router's close call may go
    the other way at a position or two (and another expert moves the logits
    by more than rounding does), so the bound holds for 19 positions out of 20,
    the median lies well inside it, and at most one position in fifty is
    off by the size of a logit; a lost state or a wrong key would put every
    position behind it there."""
    errors = np.asarray([float(np.abs(row - reference[key][at]).max()) for (key, at), row in seen.items()])
    assert len(errors)
    if dtype == "float32":
        assert errors.max() < bound(name, dtype), errors.max()
    else:
        assert np.median(errors) < 0.3 * TOL[dtype] and np.quantile(errors, 0.95) < TOL[dtype] \
            and (errors > 1.0).mean() <= 0.02, (np.median(errors), np.quantile(errors, 0.95), (errors > 1.0).mean())


def sharpened(raw, factor):
    raw = json.loads(json.dumps(raw))
    for spec in raw["layers"]:
        if spec["type"] == "attention":
            spec["mixer"]["scale"] *= factor
    return raw


def write_folder(folder, raw, seed, sharpen):
    """config.json + model.safetensors: bfloat16 matrices, float32 vectors (so
    that the engine and the plain side hold the same values). Projections are
    larger than the generator's (0.02) so that scores, gates and states move;
    step sizes are small so that the state reaches far back; the router's
    correction is as large as the scores so that it changes the choice."""
    from metallix_b200.config import SadosunConfig
    from metallix_b200.weights import random_tensors
    from metallix_b200.weights.safetensors_io import write_file
    config = SadosunConfig.from_dict(sharpened(raw, sharpen))
    tensors = random_tensors(config, seed, dtype="bfloat16", norm_dtype="float32")
    for name, value in tensors.items():
        last = name.rsplit(".", 1)[-1]
        if last == "A_log":
            tensors[name] = (value.float() * 25.0).to(torch.bfloat16)
        elif last in ("conv", "canon1", "canon2") or name == "side.embed":
            tensors[name] = (value.float() * 15.0).to(torch.bfloat16)
        elif last == "correction":
            tensors[name] = (value.float() * 6.0).to(value.dtype)
        elif name.endswith("dt.b"):
            tensors[name] = value - 2.5
        elif value.dim() == 2:
            tensors[name] = (value.float() * (8.0 if name in ("head", "embed") else 4.0)).to(torch.bfloat16)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config.to_dict(), handle)
    write_file(os.path.join(folder, "model.safetensors"), {k: v.cpu() for k, v in tensors.items()},
               order=list(config.tensor_shapes()))
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """name -> (folder, config dict, tensors as float64 numpy, page size)."""
    out = {}
    for name, (raw, seed, page, sharpen) in MODELS.items():
        folder = write_folder(str(tmp_path_factory.mktemp(f"sadosun_{name}")), raw, seed, sharpen)
        config, tensors = plain.read_model(folder)
        out[name] = (folder, config, tensors, page)
    return out


def make_engine(folders, name, dtype, pages=96, **options):
    from metallix_b200.engine import Engine
    folder, _, _, page = folders[name]
    return Engine.from_folder(folder, dtype=dtype, page_tokens=page, num_pages=pages,
                              max_requests=options.pop("max_requests", 8), **options)


def reference_logits(folders, name, requests):
    _, config, tensors, _ = folders[name]
    return {key: plain.forward_logits(config, tensors, ids) for key, ids in requests.items()}


def some_requests(name, seed, lengths):
    vocab = MODELS[name][0]["vocab"]
    return {f"r{n}": random_ids(seed + n, length, vocab) for n, length in enumerate(lengths)}


# ------------------------------------------------ configuration (no GPU needed)
def test_configuration_round_trip_and_registry():
    from metallix_b200.config import ConfigError, SadosunConfig, parse_config, resolve
    for raw in (SMALL, WIDE, BARE):
        config = parse_config(raw)
        assert isinstance(config, SadosunConfig) and resolve(raw).kind == "sadosun"
        assert SadosunConfig.from_dict(config.to_dict()) == config
        assert json.loads(json.dumps(config.to_dict())) == config.to_dict()
        shapes, w, count = config.tensor_shapes(), raw["width"], len(raw["layers"])
        side = (raw.get("token_side") or {}).get("dim", 0)
        taps = (raw.get("canon") or {}).get("taps", 0)
        assert shapes["embed"] == shapes["head"] == (raw["vocab"], w) and shapes["final.norm"] == ()
        assert ("side.embed" in shapes) == bool(side) and (not side or shapes["side.embed"] == (raw["vocab"], count * side))
        for index, spec in enumerate(raw["layers"]):
            base, mixer = f"l{index}", spec["mixer"]
            assert shapes[f"{base}.norm1"] == () and (f"{base}.norm2" in shapes) == (spec["mlp"] is not None)
            assert (f"{base}.canon1" in shapes) == bool(taps) and (not taps or shapes[f"{base}.canon1"] == (w, taps))
            assert (f"{base}.canon2" in shapes) == (bool(taps) and spec["mlp"] is not None)
            assert (f"{base}.side.gate" in shapes) == bool(side) and (not side or shapes[f"{base}.side.proj"] == (w, side))
            if spec["type"] == "attention":
                heads, kv = mixer["heads"], mixer.get("kv_heads") or mixer["heads"]
                vdim = mixer.get("vdim") or mixer["dim"]
                assert shapes[f"{base}.mix.q"] == (heads * mixer["dim"], w) and shapes[f"{base}.mix.k"] == (kv * mixer["dim"], w)
                assert shapes[f"{base}.mix.v"] == (kv * vdim, w) and shapes[f"{base}.mix.o"] == (w, heads * vdim)
            else:
                n = mixer["inner"]
                assert shapes[f"{base}.mix.in"] == (2 * n, w) and shapes[f"{base}.mix.conv"] == (n, mixer["conv"])
                assert shapes[f"{base}.mix.x"] == (mixer["dt_rank"] + 2 * mixer["state"], n)
                assert shapes[f"{base}.mix.dt"] == (n, mixer["dt_rank"]) and shapes[f"{base}.mix.A_log"] == (n, mixer["state"])
            if spec["mlp"] is not None:
                router = spec["mlp"]["router"]
                outputs = router["experts"] + router["identity"]
                assert shapes[f"{base}.mlp.router"] == (outputs, w) and shapes[f"{base}.mlp.correction"] == (outputs,)
                assert shapes[f"{base}.mlp.e{router['experts'] - 1}.down"] == (w, spec["mlp"]["expert"]["ff"])
                assert f"{base}.mlp.e{router['experts']}.up" not in shapes      # identity experts have no tensors
        model = config.to_model_spec()
        assert [run.layer for run in model.order] == list(range(count)) and not model.streams
        assert [spec.mixer.kind for spec in model.layers] == \
            ["gqa_attention" if s["type"] == "attention" else "selective_scan" for s in raw["layers"]]
    refusals = [
        ("UnsupportedLayerType", lambda c: c["layers"][0].update(type="mlstm")),
        ("InvalidGroupedQueryLayout", lambda c: c["layers"][1]["mixer"].update(kv_heads=3)),
        ("InvalidRotaryWidth", lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18)),
        ("InvalidRotaryWidth", lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7)),
        ("InvalidRotaryWidth", lambda c: c["layers"][1]["mixer"].update(vdim=23)),
        ("UnsupportedFeedForward", lambda c: c["layers"][0]["mlp"].update(kind="dense")),
        ("Json", lambda c: c["layers"][0]["mlp"]["router"].update(top=7)),
        ("Json", lambda c: c["layers"][0]["mlp"]["router"].update(identity=-1)),
        ("Json", lambda c: c["layers"][1]["mixer"].update(scale=0.0)),
        ("MissingDimension", lambda c: c["layers"][0]["mixer"].update(state=0)),
        ("InvalidRmsNormEpsilon", lambda c: c["norm"].update(eps=0.0)),
        ("MissingDimension", lambda c: c.update(layers=[]))]
    for kind, change in refusals:
        raw = json.loads(json.dumps(SMALL))
        change(raw)
        with pytest.raises(ConfigError) as caught:
            parse_config(raw)
        assert caught.value.kind == kind, (kind, caught.value.kind)


def test_random_weights_by_kind_of_tensor(tmp_path):
    from metallix_b200.config import SadosunConfig
    from metallix_b200.weights import CheckpointError, load_tensors, random_tensors, write_model_folder
    config = SadosunConfig.from_dict(SMALL)
    tensors = random_tensors(config, 3, dtype="float32")
    assert tensors["l0.norm1"].shape == () and abs(float(tensors["l0.norm1"]) - 1.0) <= 0.1
    assert abs(float(tensors["l3.mix.D"].mean()) - 1.0) < 0.05 and float(tensors["l0.mix.dt.b"].abs().max()) <= 0.1
    assert float(tensors["l2.mlp.correction"].abs().max()) < 0.2 and float(tensors["l0.mix.A_log"].abs().max()) < 0.2
    folder = write_model_folder(str(tmp_path / "m"), config, 3)
    loaded = load_tensors(folder, config)
    assert set(loaded) == set(config.tensor_shapes()) and "l1.norm2" not in loaded and "l1.canon2" not in loaded
    other = json.loads(json.dumps(SMALL))
    other["layers"][3]["mixer"]["state"] = 16
    with pytest.raises(CheckpointError):
        load_tensors(folder, SadosunConfig.from_dict(other))


def test_cache_needs_a_layer_s_states_beside_its_pages():
    """An attention layer keeps pages and the two convolutions' last inputs; a
    state-space layer its state, its own convolution's inputs and the block's;
    a layer without feed-forward has one convolution less."""
    from metallix_b200.config import SadosunConfig
    from metallix_b200.engine.model import DecoderModel
    from metallix_b200.parts.registry import Runtime
    from metallix_b200.weights import random_tensors
    config = SadosunConfig.from_dict(SMALL)
    spec = config.to_model_spec()
    model = DecoderModel(spec, random_tensors(config, 1, dtype="float32"),
                         Runtime(device=torch.device("cpu"), dtype=torch.float32, max_positions=64))
    needs = model.cache_needs()
    flat = [[(n.kind, tuple(n.state_shape) if n.kind == "state" else (n.kv_heads, n.head_dim, n.window)) for n in need.flat()]
            for need in needs]
    assert flat[0] == [("state", (40, 6)), ("state", (1, 40)), ("state", (2, 72)), ("state", (2, 72))]
    assert flat[1] == [("kv_pages", (2, 24, 5)), ("state", (2, 72))]
    assert flat[2] == [("kv_pages", (3, 12, 37)), ("state", (2, 72)), ("state", (2, 72))]
    assert flat[3][0] == ("state", (100, 17)) and flat[3][1] == ("state", (4, 100))
    assert all(need.has_state() for need in needs)
    bare = SadosunConfig.from_dict(BARE)
    model = DecoderModel(bare.to_model_spec(), random_tensors(bare, 1, dtype="float32"),
                         Runtime(device=torch.device("cpu"), dtype=torch.float32, max_positions=64))
    needs = model.cache_needs()
    assert not needs[0].has_state() and needs[1].has_state() and not needs[2].has_state()
    assert [n.window for n in needs[2].flat()] == [1] and [n.window for n in needs[0].flat()] == [None]


def test_the_plain_side_in_pieces():
    """The plain implementation itself: a sequence's logits do not change when
    more tokens follow; the convolution and the recurrence run in pieces, their
    state handed on, equal one run; the sink takes its share; a value turned by
    its position and turned back by the query's has turned by their distance."""
    from metallix_b200.config import SadosunConfig
    rng = np.random.default_rng(0)
    shapes = SadosunConfig.from_dict(SMALL).tensor_shapes()
    tensors = {name: rng.normal(size=shape) * (0.1 if len(shape) <= 1 else 0.3) for name, shape in shapes.items()}
    ids = random_ids(1, 30, 211)
    whole = plain.forward_logits(SMALL, tensors, ids)
    assert np.allclose(plain.forward_logits(SMALL, tensors, ids[:19]), whole[:19], atol=1e-10)
    x, w, bias = rng.normal(size=(25, 7)), rng.normal(size=(7, 4)), rng.normal(size=7)
    once, _ = plain.causal_conv(x, w, bias)
    first, kept = plain.causal_conv(x[:2], w, bias)
    second, kept = plain.causal_conv(x[2:11], w, bias, kept)
    third, _ = plain.causal_conv(x[11:], w, bias, kept)
    assert np.allclose(np.concatenate([first, second, third]), once, atol=1e-12)
    assert np.allclose(once[0], bias + w[:, 3] * x[0]) and np.allclose(once[1], bias + w[:, 3] * x[1] + w[:, 2] * x[0])
    dt, a = rng.uniform(0.01, 0.3, size=(25, 7)), -np.exp(rng.normal(size=(7, 3)))
    b, c, d = rng.normal(size=(25, 3)), rng.normal(size=(25, 3)), rng.normal(size=7)
    once, last = plain.selective_recurrence(x, dt, a, b, c, d)
    first, state = plain.selective_recurrence(x[:9], dt[:9], a, b[:9], c[:9], d)
    second, again = plain.selective_recurrence(x[9:], dt[9:], a, b[9:], c[9:], d, state)
    assert np.allclose(np.concatenate([first, second]), once, atol=1e-12) and np.allclose(again, last, atol=1e-12)
    scores = rng.normal(size=(4, 9))
    seen = np.ones((4, 9), dtype=bool)
    p = plain.sink_softmax(scores, seen, 0.0)
    assert np.allclose(p.sum(axis=1), 1.0 - 1.0 / (1.0 + np.exp(scores).sum(axis=1)))
    assert np.allclose(plain.sink_softmax(scores, seen, None).sum(axis=1), 1.0)
    assert plain.window_mask(6, 2).sum() == 11 and plain.window_mask(6, 0).sum() == 21 and plain.window_mask(6, 1).sum() == 6
    value = rng.normal(size=(1, 1, 10))
    there = plain.turn_pairs(plain.turn_pairs(value, [13], 30.0, 10), [20], 30.0, 10, sign=-1.0)
    assert np.allclose(there, plain.turn_pairs(value, [-7], 30.0, 10), atol=1e-12)
    logits = np.log(np.array([[0.4, 0.3, 0.2, 0.1]]))
    chosen, weights = plain.choose_experts(logits, np.array([0.0, 0.0, 0.0, 0.35]), 2)
    assert chosen.tolist() == [[3, 0]] and np.allclose(weights, [[0.2, 0.8]])      # chosen by s + c, weighed by s


# --------------------------------------------------------- mechanisms alone
gpu = pytest.mark.gpu


def dev(array, dtype=torch.float32):
    return torch.tensor(np.asarray(array), dtype=dtype, device="cuda")


def rounded(array, dtype):
    return torch.tensor(np.asarray(array), dtype=dtype).double().numpy()


def rows_of(lengths):
    """Packed tokens of request rows: starts, and the request of every token."""
    starts, owner, cursor = [], [], 0
    for row, length in enumerate(lengths):
        starts.append(cursor)
        owner += [row] * length
        cursor += length
    return starts, owner


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels, taps, bias, residual, activation", [
    (72, 3, False, True, None), (40, 2, True, False, "silu"), (100, 5, True, False, "silu"), (331, 4, False, True, None),
    (7, 9, True, True, "silu"), (264, 4, True, True, None), (64, 1, False, True, "silu")])
@pytest.mark.parametrize("left", [3, 8])     # columns ahead of x in the wider product: 8 lets whole vectors be read
def test_short_convolution_with_its_inputs_in_state_slots(dtype, channels, taps, bias, residual, activation, left):
    """Four request rows of unequal length in one launch (a single token, a
    padding row, a row shorter than the taps), continued twice from the slots'
    state, against the plain convolution of each whole sequence; x is a column
    range of a wider product; an untouched slot keeps its values."""
    from metallix_b200 import ops
    rng = np.random.default_rng(channels * taps)
    # the last steps bring single tokens only: the launch that reads a slot moves it on as well
    pieces = [[6, 1, 0, 2], [1, 1, 0, 13], [2, 9, 0, 1], [1, 1, 0, 1], [1, 0, 0, 1], [1, 3, 0, 0]]
    slots = [3, 0, 1, 2]
    w, b = rounded(rng.normal(size=(channels, taps)), torch.float32), rounded(rng.normal(size=channels), torch.float32)
    totals = [sum(p[row] for p in pieces) for row in range(4)]
    x = [rounded(rng.normal(size=(total, channels)), dtype) for total in totals]
    state = torch.full((5, taps - 1, channels), 7.0, device="cuda")
    for slot in slots:
        state[slot].zero_()       # what the cache does when a sequence starts
    got = [[] for _ in totals]
    done = [0] * 4
    for lengths in pieces:
        starts, owner = rows_of(lengths)
        packed = np.concatenate([x[row][done[row]:done[row] + n] for row, n in enumerate(lengths)])
        wide = dev(np.pad(packed, ((0, 0), (left, 16 - left))), dtype)
        out = ops.short_conv(wide[:, left:left + channels], dev(np.ascontiguousarray(w.T)), dev(b) if bias else None, state, dev(owner, torch.int32),
                             dev(starts, torch.int32), dev(lengths, torch.int32), dev(slots, torch.int32),
                             residual=residual, activation=activation, longest=max(lengths))
        ops.check_status("cuda")
        for row, n in enumerate(lengths):
            got[row].append(out[starts[row]:starts[row] + n].double().cpu().numpy())
            done[row] += n
    assert taps == 1 or (float(state[4].min()) == 7.0 and float(state[1].abs().max()) == 0.0)
    for row, total in enumerate(totals):
        if not total:
            continue
        want, kept = plain.causal_conv(x[row], w, b if bias else None)
        if residual:
            want = want + x[row]
        if activation == "silu":
            want = plain.silu(want)
        assert np.abs(np.concatenate(got[row]) - want).max() < (1e-5 if dtype == torch.float32 else 5e-2)
        if taps > 1:
            assert np.abs(state[slots[row]].double().cpu().numpy() - kept).max() < 1e-6     # the last taps - 1 inputs, as they came


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels, states", [(40, 6), (100, 17), (24, 1), (256, 16), (33, 64), (8, 130)])
def test_selective_scan_kernel(dtype, channels, states):
    """The recurrence over request rows of unequal length in one launch, then
    continued from the state the first launch left, against the plain
    recurrence in one piece; slow decays and a large first token, so that it
    still counts at the end (without it the result differs by far more than
    the bound, which is taken value by value)."""
    from metallix_b200 import ops
    rng = np.random.default_rng(channels + states)
    pieces = [[23, 1, 0, 5], [1, 1, 0, 40], [8, 3, 0, 1]]
    slots = [2, 0, 1, 3]
    totals = [sum(p[row] for p in pieces) for row in range(4)]
    a = rounded(-np.exp(rng.normal(size=(channels, states)) * 0.5), torch.float32)
    step_bias, skip = rounded(rng.normal(size=channels) * 0.3 - 3.0, torch.float32), rounded(rng.normal(size=channels), torch.float32)
    seq = []
    for total in totals:
        first = np.where(np.arange(total) == 0, 32.0 if total > 20 else 1.0, 1.0)[:, None]      # a first token that stands out
        seq.append({"x": rounded(rng.normal(size=(total, channels)), dtype) * first, "z": rounded(rng.normal(size=(total, channels)), dtype),
                    "b": rounded(rng.normal(size=(total, states)), dtype), "c": rounded(rng.normal(size=(total, states)), dtype),
                    "p": rounded(rng.normal(size=(total, channels)), torch.float32)})
    state = torch.full((5, channels, states), 3.0, device="cuda")
    for slot in slots:
        state[slot].zero_()
    got = [[] for _ in totals]
    done = [0] * 4
    for lengths in pieces:
        starts, _ = rows_of(lengths)
        pack = lambda key: np.concatenate([seq[row][key][done[row]:done[row] + n] for row, n in enumerate(lengths)])
        both = dev(np.concatenate([pack("x"), pack("z")], axis=1), dtype)         # x and z as halves of one product
        picked = dev(np.concatenate([np.zeros((sum(lengths), 2)), pack("b"), pack("c")], axis=1), dtype)
        out = ops.selective_scan(both[:, :channels], dev(pack("p")), dev(step_bias), dev(a), picked[:, 2:2 + states],
                                 picked[:, 2 + states:], dev(skip), both[:, channels:], state, dev(starts, torch.int32),
                                 dev(lengths, torch.int32), dev(slots, torch.int32))
        ops.check_status("cuda")
        for row, n in enumerate(lengths):
            got[row].append(out[starts[row]:starts[row] + n].double().cpu().numpy())
            done[row] += n
    assert float(state[4].min()) == 3.0 and float(state[1].abs().max()) == 0.0
    tolerance = 1e-4 if dtype == torch.float32 else 6e-2
    for row, total in enumerate(totals):
        if not total:
            continue
        s = seq[row]
        dt = plain.softplus(s["p"] + step_bias[None, :])
        y, last = plain.selective_recurrence(s["x"], dt, a, s["b"], s["c"], skip)
        want = y * plain.silu(s["z"])
        assert (np.abs(np.concatenate(got[row]) - want) < tolerance * (1.0 + np.abs(want))).all()
        assert np.abs(state[slots[row]].double().cpu().numpy() - last).max() < 1e-4 * max(1.0, np.abs(last).max())
        if total > 20 and dtype == torch.float32:      # the state is what carries the first token to the last
            later, _ = plain.selective_recurrence(s["x"][1:], dt[1:], a, s["b"][1:], s["c"][1:], skip)
            gap = np.abs((later[-1] - y[-1]) * plain.silu(s["z"][-1]))
            assert (gap > 20 * tolerance * (1.0 + np.abs(want[-1]))).mean() > 0.1


@gpu
@pytest.mark.parametrize("outputs, real, top", [(6, 5, 2), (5, 3, 3), (7, 7, 1), (2, 2, 2), (4, 1, 2), (40, 33, 6), (300, 290, 8)])
def test_router_choice_by_corrected_scores_weights_by_scores(outputs, real, top):
    """Softmax over all outputs, identity experts included; the correction
    moves the choice and not the weights; a tie goes to the lower index; what
    falls on identity experts is summed."""
    from metallix_b200 import ops
    rng = np.random.default_rng(outputs * top)
    logits = rounded(rng.normal(size=(37, outputs)) * 2.0, torch.float32)
    correction = rounded(rng.normal(size=outputs) * (1.0 / outputs), torch.float32)
    logits[3] = 0.0                      # all scores alike: the correction alone decides
    logits[4, :] = logits[4, 0]          # ... and here as well
    chosen, weights, dense, on_identity = ops.route_experts(dev(logits), dev(correction), real, top)
    want_chosen, want_weights = plain.choose_experts(logits, correction, top)
    plain_scores = plain.choose_experts(logits, np.zeros(outputs), top)[0]
    assert (np.sort(plain_scores, axis=1) != np.sort(want_chosen, axis=1)).any() or top == outputs   # the correction matters here
    assert np.array_equal(chosen.cpu().numpy(), want_chosen)
    assert np.abs(weights.double().cpu().numpy() - want_weights).max() < 1e-6
    want_dense, want_identity = np.zeros((37, real)), np.zeros(37)
    for t in range(37):
        for e, w in zip(want_chosen[t], want_weights[t]):
            if e < real:
                want_dense[t, e] = w
            else:
                want_identity[t] += w
    assert np.abs(dense.double().cpu().numpy() - want_dense).max() < 1e-6
    assert np.abs(on_identity.double().cpu().numpy() - want_identity).max() < 1e-6
    flat = torch.zeros((2, outputs), device="cuda")
    chosen, weights, _, _ = ops.route_experts(flat, torch.zeros(outputs, device="cuda"), real, top)
    assert chosen.cpu().tolist() == [list(range(top))] * 2 and np.allclose(weights.cpu().numpy(), 1.0 / top)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width, ff, count, identity, top", [(72, 24, 5, 1, 2), (48, 8, 1, 3, 2), (128, 64, 8, 3, 5),
                                                              (40, 20, 2, 0, 2), (96, 33, 7, 0, 1), (64, 16, 0, 3, 2)])
def test_routed_experts_both_ways_through_them(dtype, width, ff, count, identity, top):
    """The feed-forward part on a few tokens (row by row through the chosen
    experts' weights) and on many (in 16 bits the pairs sorted by expert and
    two grouped products, where the sizes allow them; several tiles for an
    expert at 700 tokens) against the plain mixture; identity experts return
    their input."""
    from metallix_b200.config.spec import PartSpec
    from metallix_b200.parts.registry import Runtime, StepContext, WeightStore, build_part  # noqa: F401
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(width + ff)
    tensors = {"m.router": rng.normal(size=(count + identity, width)) * 0.3, "m.correction": rng.normal(size=count + identity) * 0.1}
    for e in range(count):
        tensors[f"m.e{e}.up"] = rng.normal(size=(ff, width)) * 0.2
        tensors[f"m.e{e}.down"] = rng.normal(size=(width, ff)) * 0.2
    tensors = {k: rounded(v, torch.float32 if k.endswith("correction") else torch_dtype) for k, v in tensors.items()}
    runtime = Runtime(device=torch.device("cuda"), dtype=torch_dtype, max_positions=16)
    store = WeightStore({k: torch.tensor(v, dtype=torch.float32 if k.endswith("correction") else torch_dtype)
                         for k, v in tensors.items()})
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": width, "intermediate_size": ff, "experts": count, "identity": identity, "top": top,
        "activation": "relu_squared", "up_proj": "m.e{}.up", "down_proj": "m.e{}.down", "router": "m.router",
        "correction": "m.correction"}), store, runtime)
    for tokens in (1, 5, part.ROUTED_TOKENS, part.ROUTED_TOKENS + 1, 70, 300, 700):
        h = rounded(rng.normal(size=(tokens, width)), torch_dtype)
        chosen = []
        want = plain.expert_mixture(h, tensors, "m", experts=count, identity=identity, top=top, chosen_out=chosen)
        got = part.forward(dev(h, torch_dtype), None).double().cpu().numpy()
        assert got.shape == want.shape
        if dtype == "float32":
            assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())
        else:       # a close call of the router in 16-bit inputs may differ for a token; most must agree closely
            errors = np.abs(got - want).max(axis=1) / max(1.0, np.abs(want).max())
            assert np.median(errors) < 3e-2 and (errors < 3e-2).mean() >= 0.9
        if identity and count:
            assert (chosen[0] >= count).any() or tokens < 5       # identity experts do get chosen


@gpu
@pytest.mark.parametrize("tokens, top, experts, extra, k, n", [(300, 2, 5, 1, 72, 40), (700, 3, 4, 0, 64, 136),
                                                                (40, 1, 9, 2, 136, 264), (1000, 2, 3, 1, 200, 64)])
def test_pairs_sorted_by_expert_and_the_grouped_product(tokens, top, experts, extra, k, n):
    """Every (token, choice) pair gets a row of its own inside its expert's
    tiles, choices that are no real expert get none, and the grouped product
    multiplies each tile by its expert's matrix (against a float32 product row
    by row), with and without the squared relu; an expert without tokens has
    no tile."""
    from metallix_b200 import ops, tensor_core
    rng = np.random.default_rng(tokens + k)
    chosen = rng.integers(0, experts + extra, size=(tokens, top)).astype(np.int32)
    chosen[chosen == 1] = 0                                     # expert 1 stays without tokens
    position, tile_group, rows = ops.expert_rows(dev(chosen, torch.int32), experts)
    tile = ops.expert_rows_tile()
    position, tile_group = position.cpu().numpy(), tile_group.cpu().numpy()
    assert rows == tile * len(tile_group) and rows >= tokens * top
    real = chosen < experts
    assert (position[~real] == -1).all() and (position[real] >= 0).all()
    assert len(np.unique(position[real])) == real.sum()         # no row is given twice
    assert np.array_equal(tile_group[position[real] // tile], chosen[real])
    used = tile_group[tile_group >= 0]
    assert (np.diff(used) >= 0).all() and 1 not in used and (tile_group[len(used):] == -1).all()
    for e in range(experts):                                    # an expert's rows fill its tiles from the front
        mine = np.sort(position[chosen == e])
        if len(mine):
            assert np.array_equal(mine, mine[0] + np.arange(len(mine))) and mine[0] % tile == 0
            assert (tile_group == e).sum() == -(-len(mine) // tile)
    h = rounded(rng.normal(size=(tokens, k)), torch.bfloat16)
    w = rounded(rng.normal(size=(experts * n, k)) * 0.2, torch.bfloat16)
    sorted_rows = ops.expert_gather_rows(dev(h, torch.bfloat16), dev(position, torch.int32), rows)
    group = dev(tile_group, torch.int32)
    plain_product = np.einsum("tk,tnk->tn", h[:, None, :].repeat(top, 1).reshape(-1, k),
                              w.reshape(experts, n, k)[np.minimum(chosen, experts - 1).reshape(-1)])
    where = position.reshape(-1)
    for epilogue, want in ((tensor_core.STORE_F32, plain_product),
                           (tensor_core.RELU_SQUARED, np.maximum(plain_product, 0.0) ** 2)):
        got = tensor_core.gemm_grouped(sorted_rows, dev(w, torch.bfloat16), group, experts, epilogue)
        got = got.double().cpu().numpy()[where[where >= 0]]
        bound = 1e-4 if epilogue == tensor_core.STORE_F32 else 2e-2
        assert np.abs(got - want[where >= 0]).max() < bound * max(1.0, np.abs(want).max())
    weights = rng.random(size=(tokens, top)).astype(np.float32)
    on_identity = rng.random(size=tokens).astype(np.float32)
    out_rows = rng.normal(size=(rows, k)).astype(np.float32)
    got = ops.expert_combine_rows(dev(out_rows), dev(position, torch.int32), dev(weights), dev(on_identity),
                                  dev(h, torch.bfloat16)).double().cpu().numpy()
    want = on_identity[:, None] * h
    for j in range(top):
        want = want + np.where(position[:, j:j + 1] >= 0, weights[:, j:j + 1] * out_rows[np.maximum(position[:, j], 0)], 0.0)
    assert np.abs(got - want).max() < 1e-5


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_input_scaled_embedding_and_scalar_norms(dtype):
    """gelu_tanh(gate) times a layer's columns of the token's table row; the
    sum into the stream with a cast; an embedding times a constant; a norm
    whose weight is one number, and one without a weight."""
    from metallix_b200 import ops
    from metallix_b200.config.spec import PartSpec
    from metallix_b200.parts.registry import Runtime, WeightStore, build_part
    rng = np.random.default_rng(8)
    tokens, dim, columns, offset, vocab = 9, 10, 47, 20, 31
    gate = rounded(rng.normal(size=(tokens, dim)) * 2.0, dtype)
    table = rounded(rng.normal(size=(vocab, columns)), dtype)
    ids = rng.integers(0, vocab, size=tokens)
    got = ops.gelu_gate_rows(dev(gate, dtype), dev(table, dtype), dev(ids, torch.int32), offset)
    want = plain.gelu_tanh(gate) * table[ids][:, offset:offset + dim]
    assert np.abs(got.double().cpu().numpy() - want).max() < (1e-5 if dtype == torch.float32 else 3e-2)
    x, d = rounded(rng.normal(size=(tokens, 33)), torch.float32), rounded(rng.normal(size=(tokens, 33)), dtype)
    stream = dev(x)
    cast = ops.add_cast(stream, dev(d, dtype), dtype)
    assert np.abs(stream.double().cpu().numpy() - (x + d)).max() < 1e-6
    assert np.abs(cast.double().cpu().numpy() - rounded(stream.cpu().numpy(), dtype)).max() == 0.0
    rows = ops.embed(dev(ids, torch.int32), dev(table, dtype), scale=3.7)
    assert rows.dtype == torch.float32
    assert np.abs(rows.double().cpu().numpy() - table[ids] * float(np.float32(3.7))).max() < 1e-5
    runtime = Runtime(device=torch.device("cuda"), dtype=dtype, max_positions=16)
    store = WeightStore({"n": torch.tensor(1.25)})
    one = build_part("norm", PartSpec("rmsnorm", {"size": 33, "eps": 1e-3, "weight": "n", "scalar": True}), store, runtime)
    none = build_part("norm", PartSpec("rmsnorm", {"size": 33, "eps": 1e-3, "weight": None}), store, runtime)
    assert np.abs(one.forward(dev(x), torch.float32).double().cpu().numpy() - plain.norm(x, 1.25, 1e-3)).max() < 1e-5
    assert np.abs(none.forward(dev(x), torch.float32).double().cpu().numpy() - plain.unit_rms(x, 1e-3)).max() < 1e-5
    with pytest.raises(ValueError):
        build_part("norm", PartSpec("rmsnorm", {"size": 33, "eps": 1e-3, "weight": "w", "scalar": True}),
                   WeightStore({"w": torch.ones(33)}), runtime)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, page", [
    (4, 2, 16, 24, 5, 8), (3, 3, 12, 8, 37, 8), (6, 1, 40, 40, 0, 4), (2, 1, 64, 64, 70, 16), (2, 2, 8, 8, 1, 4)])
def test_attention_kernel_sink_and_keys_at_the_window_s_edge(dtype, heads, kv_heads, dim, vdim, window, page):
    """The attention kernel with a sink of score 0 and a window. Single
    queries are made to look for the key just inside the window, the key just
    outside it (which they must not find), a key at a page's border and, with
    no window, a key hundreds of positions back; one query has only negative
    scores, so that the sink takes most of its weight."""
    from metallix_b200 import ops
    rng = np.random.default_rng(dim * heads + vdim + window)
    context, tail, scale = 301, 19, 0.4
    width = max(dim, vdim)
    pages = -(-context // page)
    order = rng.permutation(pages + 2)[:pages]
    keys = rng.normal(size=(context, kv_heads, dim)) * 0.5
    keys[:, :, 0] = 1.5
    values = rng.normal(size=(context, kv_heads, vdim))
    q = rng.normal(size=(tail, heads, dim)) * 0.5
    group = heads // kv_heads
    first = context - tail
    reach = window if window else context

    def look_for(t, key, factor=5.0):
        keys[key] *= factor
        q[t] = np.repeat(keys[key], group, axis=0) * 1.2

    inside, outside = first + 4 - (reach - 1), first + 7 - reach
    if window and inside >= 0:
        look_for(4, inside)                       # the oldest key query 4 still sees
    if window and outside >= 0:
        look_for(7, outside)                      # one older than the oldest that query 7 sees
    if not window:
        look_for(tail - 1, 6, 6.0)                # far back
    border = (first + 10) // page * page
    if first + 10 - border < reach:
        look_for(10, border)                      # a page's first row
    q[12] = 0.0
    q[12, :, 0] = -10.0                           # against the keys' first value, which is positive: every score -6 or less
    keys, values, q = rounded(keys, dtype), rounded(values, dtype), rounded(q, dtype)
    pool = torch.zeros((pages + 2, 2, kv_heads, page, width), dtype=dtype, device="cuda")
    for p in range(pages):
        span = slice(p * page, min((p + 1) * page, context))
        n = span.stop - span.start
        pool[order[p], 0, :, :n, :dim] = dev(keys[span].transpose(1, 0, 2), dtype)
        pool[order[p], 1, :, :n, :vdim] = dev(values[span].transpose(1, 0, 2), dtype)
    q_rows = np.pad(q, ((0, 0), (0, 0), (0, width - dim)))
    positions = np.arange(first, context)
    starts = [0, 16]
    results = {}
    for sink in (0.0, None):
        out = torch.empty((tail, heads, vdim), dtype=dtype, device="cuda")
        ops.paged_attention_tile(dev(q_rows, dtype), pool, out, dev(order[None, :], torch.int32), dev([0, 0], torch.int32),
                                 dev(starts, torch.int32), dev([16, tail - 16], torch.int32), dev(positions, torch.int32),
                                 scale, window, sink=sink)
        ops.check_status("cuda")
        results[sink] = out.double().cpu().numpy()
    k_all, v_all = np.repeat(keys, group, axis=1), np.repeat(values, group, axis=1)
    tolerance = 2e-5 if dtype == torch.float32 else 3e-2
    for sink in (0.0, None):
        want = np.zeros((tail, heads, vdim))
        for t, p in enumerate(positions):
            low = max(0, p - reach + 1)
            s = np.einsum("hd,jhd->hj", q[t], k_all[low:p + 1]) * scale
            w = plain.sink_softmax(s, np.ones_like(s, dtype=bool), sink)
            want[t] = np.einsum("hj,jhv->hv", w, v_all[low:p + 1])
            if sink is not None and t == 4 and window and inside >= 0:
                assert w[:, 0].min() > 0.5 or reach == 1       # the key at the window's edge carries the output
            if sink is not None and t == 12:
                assert w.sum(axis=1).max() < 0.75              # the sink has taken a good share
        assert np.abs(results[sink] - want).max() < tolerance, sink
    if dtype != torch.float32:
        return
    assert np.abs(results[0.0] - results[None]).max() > 20 * tolerance      # with and without the sink differ
    if window and outside >= 0:     # had query 7 seen one key more, its output would be another
        low = outside
        s = np.einsum("hd,jhd->hj", q[7], k_all[low:first + 8]) * scale
        w = plain.sink_softmax(s, np.ones_like(s, dtype=bool), 0.0)
        assert np.abs(np.einsum("hj,jhv->hv", w, v_all[low:first + 8]) - results[0.0][7]).max() > 20 * tolerance


@gpu
@pytest.mark.parametrize("dtype, head_dim, heads, kv_heads, context, page, window", [
    (torch.bfloat16, 64, 6, 6, 300, 16, 0), (torch.bfloat16, 128, 16, 8, 4500, 16, 1000), (torch.bfloat16, 128, 8, 2, 700, 4, 129),
    (torch.bfloat16, 128, 4, 1, 2300, 16, 0), (torch.bfloat16, 256, 4, 4, 400, 16, 70), (torch.float32, 64, 4, 2, 500, 8, 128),
    (torch.float32, 128, 2, 1, 260, 16, 0)])
def test_sink_in_the_split_key_and_prompt_kernels(dtype, head_dim, heads, kv_heads, context, page, window):
    """One more key of score 0 without a value inside the split-key decode
    kernels (four single tokens behind contexts of unequal length; the sink
    joins once, where the splits are put together) and inside both tensor-core
    prompt kernels (a portion behind cached keys, alone or with its keys shared
    out among blocks), with a window. Queries are small, so that the sink
    takes a good share of every softmax, and one query has only low scores."""
    from metallix_b200 import ops
    rng = np.random.default_rng(head_dim + context)
    scale, rows = 0.05, 4
    lengths = [context, context // 2 + 3, 1, context - 7]
    pages_each = -(-context // page)
    pool_pages = rows * pages_each + 2
    keys = rounded(rng.normal(size=(rows, context, kv_heads, head_dim)), dtype)
    keys[:, :, :, 0] = 2.0
    values = rounded(rng.normal(size=(rows, context, kv_heads, head_dim)), dtype)
    order = rng.permutation(pool_pages)[:rows * pages_each].reshape(rows, pages_each)
    pool = torch.zeros((pool_pages, 2, kv_heads, page, head_dim), dtype=dtype, device="cuda")
    for r in range(rows):
        k_pages = np.zeros((pages_each * page, kv_heads, head_dim))
        v_pages = np.zeros_like(k_pages)
        k_pages[:context], v_pages[:context] = keys[r], values[r]
        index = torch.tensor(order[r], device="cuda")
        pool[index, 0] = dev(k_pages.reshape(pages_each, page, kv_heads, head_dim).transpose(0, 2, 1, 3), dtype)
        pool[index, 1] = dev(v_pages.reshape(pages_each, page, kv_heads, head_dim).transpose(0, 2, 1, 3), dtype)
    group = heads // kv_heads
    shares_of_the_sink = []

    def attend(q, row, last, sink=0.0):      # q [heads, head_dim] at position `last` of request `row`
        low = max(0, last - window + 1) if window else 0
        k = np.repeat(keys[row, low:last + 1], group, axis=1)
        v = np.repeat(values[row, low:last + 1], group, axis=1)
        scores = np.einsum("hd,jhd->hj", q, k) * scale
        weights = plain.sink_softmax(scores, np.ones_like(scores, dtype=bool), sink)
        shares_of_the_sink.append(1.0 - weights.sum(axis=1).min())
        return np.einsum("hj,jhd->hd", weights, v)

    tolerance = 2e-5 if dtype == torch.float32 else 3e-2
    q = rounded(rng.normal(size=(rows, heads, head_dim)), dtype)
    q[0, :, 0] = -128.0       # every score of the longest request's query is low: the sink takes nearly all
    out = torch.empty((rows, heads, head_dim), dtype=dtype, device="cuda")
    positions = [length - 1 for length in lengths]
    if ops.decode_attention_supported(head_dim, heads, kv_heads, dtype):
        ops.paged_attention_decode(dev(q, dtype), pool, out, dev(order, torch.int32), dev(range(rows), torch.int32),
                                   dev(range(rows), torch.int32), dev(positions, torch.int32), scale, max(lengths),
                                   window, sink=0.0)
        ops.check_status("cuda")
        want = np.stack([attend(q[r], r, positions[r]) for r in range(rows)])
        assert shares_of_the_sink[0] > 0.5 and shares_of_the_sink[2] > 0.3
        assert np.abs(out.double().cpu().numpy() - want).max() < tolerance
        without = np.stack([attend(q[r], r, positions[r], None) for r in range(rows)])
        assert np.abs(want - without).max() > 10 * tolerance
    if ops.flash_prefill_supported(head_dim, heads, kv_heads, dtype):
        cached, portion = context // 3, min(150, context - context // 3)
        q = rounded(rng.normal(size=(portion, heads, head_dim)), dtype)
        q[5, :, 0] = -128.0
        out = torch.empty((portion, heads, head_dim), dtype=dtype, device="cuda")
        tile = ops.flash_prefill_tile()
        starts = list(range(0, portion, tile))
        want = np.stack([attend(q[t], 0, cached + t) for t in range(portion)])
        for kernel in ("tcgen05", "mma"):
            if kernel == "tcgen05" and not ops.flash_prefill_tcgen05_supported(head_dim, heads, kv_heads, page, dtype):
                continue
            for longest in (0, cached + portion):      # unknown: a block per tile; known: the keys may be shared out
                out.zero_()
                ops.flash_prefill(dev(q, dtype), pool, out, dev(order[:1], torch.int32), dev([0] * len(starts), torch.int32),
                                  dev(starts, torch.int32), dev([min(tile, portion - s) for s in starts], torch.int32),
                                  dev(range(cached, cached + portion), torch.int32), scale, window, kernel=kernel,
                                  longest_context=longest, sink=0.0)
                ops.check_status("cuda")
                assert np.abs(out.double().cpu().numpy() - want).max() < tolerance, (kernel, longest)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, width, base", [(3, 24, 100.0), (1, 8, 1.0e4), (2, 64, 50.0), (5, 2, 7.0)])
def test_values_turned_by_their_position_and_back(dtype, heads, width, base):
    """Neighbouring pairs over a value's whole width turned by the position
    (for the cache) and by minus the position (for a head's output)."""
    from metallix_b200.config.spec import PartSpec
    from metallix_b200.parts.registry import Runtime, WeightStore, build_part
    from metallix_b200 import ops
    rng = np.random.default_rng(width)
    positions = np.array([0, 1, 2, 57, 300, 301, 1999])
    x = rounded(rng.normal(size=(len(positions), heads, width)), dtype)
    runtime = Runtime(device=torch.device("cuda"), dtype=dtype, max_positions=2048)
    turn = build_part("position", PartSpec("rope_interleaved", {"theta": base, "rotary_dim": width, "head_dim": width,
                                                               "scaling": None}), WeightStore({}), runtime)
    flat = dev(x.reshape(len(positions), heads * width), dtype)
    there = ops.norm_rotate_heads(flat, width, dev(positions, torch.int32), cos=turn.cos, sin=turn.sin, interleaved=True)
    back = ops.norm_rotate_heads(flat, width, dev(positions, torch.int32), cos=turn.cos, sin=turn.inverse_sin(),
                                 interleaved=True)
    tolerance = 2e-4 if dtype == torch.float32 else 3e-2
    assert np.abs(there.double().cpu().numpy() - plain.turn_pairs(x, positions, base, width)).max() < tolerance
    assert np.abs(back.double().cpu().numpy() - plain.turn_pairs(x, positions, base, width, sign=-1.0)).max() < tolerance


# ------------------------------------------------- the engine: whole prompts
@gpu
@pytest.mark.parametrize("name, dtype", CASES)
def test_whole_prompts_layer_by_layer(folders, name, dtype):
    """A prompt in one step: the residual stream after every layer, then the
    logits at every position; a single token; two tokens."""
    from metallix_b200.engine import StepEntry
    engine = make_engine(folders, name, dtype)
    _, config, tensors, _ = folders[name]
    ids = random_ids(7, 45, config["vocab"])
    want_taps = []
    want = plain.forward_logits(config, tensors, ids, want_taps)
    got_taps = []
    logits = engine.step([StepEntry("a", ids, list(range(len(ids))))], tap=lambda i, r: got_taps.append(r.double().cpu().numpy()))
    engine.check()
    assert len(got_taps) == len(want_taps) == len(config["layers"])
    slack = 1.0 if dtype == "float32" else 4.0
    for index, (have, should) in enumerate(zip(got_taps, want_taps)):
        errors = np.abs(have - should).max(axis=1) / max(1.0, np.abs(should).max())
        if dtype == "float32":
            assert errors.max() < slack * bound(name, dtype), index
        else:       # a router's close call may send a token or two to another expert
            assert np.quantile(errors, 0.9) < slack * bound(name, dtype), index
    if dtype == "float32":
        assert np.abs(logits.double().cpu().numpy() - want).max() < bound(name, dtype)
    else:
        compare_replay(name, dtype, {("a", t): row for t, row in enumerate(logits.double().cpu().numpy())}, {"a": want})
    engine.release("a")
    for length in (1, 2):
        logits = engine.step([StepEntry("b", ids[:length], list(range(length)))])
        assert np.abs(logits.double().cpu().numpy() - want[:length]).max() < (bound(name, dtype) if dtype == "float32" else 1.0)
        engine.release("b")
    engine.check()


def test_the_models_of_these_tests_show_a_window_a_sink_and_a_state(folders):
    """What the tests below can see: on the plain side, a window one position
    longer, a softmax without the sink, and a state lost at one position each
    move the logits by far more than the bound the engine is held to."""
    _, config, tensors, _ = folders["sharp"]
    ids = random_ids(40, 75, config["vocab"])
    base = plain.forward_logits(config, tensors, ids)
    longer = json.loads(json.dumps(config))
    for spec in longer["layers"]:
        if spec["type"] == "attention":
            spec["mixer"]["mask"]["size"] += 1
    gaps = {"window": np.abs(plain.forward_logits(longer, tensors, ids) - base)[40:].max(),
            "sink": np.abs(plain.forward_logits(config, tensors, ids, sink=None) - base).max(),
            "state": np.abs(plain.forward_logits(config, tensors, ids, forget_at=60) - base)[60:].max()}
    assert min(gaps.values()) > 100 * TOL_SHARP, gaps


@gpu
@pytest.mark.parametrize("name, dtype", CASES)
def test_decoding_and_portions_against_whole_prompts(folders, name, dtype):
    """The same requests as whole prompts, with their tails decoded one by one
    (over more tokens than the longest window, so that it passes over decoded
    tokens), and in portions of changing size down to two tokens (and one)."""
    from metallix_b200.engine import StepEntry
    requests = some_requests(name, 40, (75, 9, 33, 170 if name == "wide" else 50))
    reference = reference_logits(folders, name, requests)
    for schedule in (cuts.whole(requests), cuts.tail_by_one(requests, tail=45), cuts.ragged(requests),
                     cuts.ragged(requests, sizes=(2, 2, 3, 1, 2, 4, 9, 2))):
        engine = make_engine(folders, name, dtype, pages=48, max_requests=2)
        _, seen = cuts.replay(engine, schedule, reference, StepEntry)
        compare_replay(name, dtype, seen, reference)


@gpu
@pytest.mark.parametrize("name, dtype", CASES)
def test_mixed_batches_with_pages_and_slots_that_come_back(folders, name, dtype):
    """Up to four requests live at once in a pool made for just that many:
    portions beside single tokens, requests that sit a step out, ended requests
    whose pages and state slots the next ones take over. Each position's
    logits equal those of the request run alone."""
    from metallix_b200.engine import StepEntry
    requests = some_requests(name, 60, (70, 41, 5, 90, 23, 1, 37, 64, 2, 55))
    reference = reference_logits(folders, name, requests)
    steps, peak = cuts.mixed(requests, seed=5, max_live=4)
    page = folders[name][3]
    engine = make_engine(folders, name, dtype, pages=-(-peak // page), max_requests=4)
    _, mixed_seen = cuts.replay(engine, steps, reference, StepEntry)
    compare_replay(name, dtype, mixed_seen, reference)
    assert engine.manager.pages_reused() > 0 and len(requests) > engine.manager.max_requests()
    if dtype == "float32":     # against the engine itself, each request alone: rounding of the products only
        alone = make_engine(folders, name, dtype, pages=48, max_requests=2)
        _, alone_seen = cuts.replay(alone, cuts.whole(requests), reference, StepEntry)
        gap = max(float(np.abs(row - alone_seen[key]).max()) for key, row in mixed_seen.items())
        assert gap < 0.3 * bound(name, dtype)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(folders, dtype):
    """Three requests decoded together for 160 steps (captured graphs), one of
    them leaving on the way and another joining with a prompt: the recurrent
    state, the convolutions' inputs and the pages stay each request's own."""
    from metallix_b200.engine import StepEntry
    name = "small"
    requests = some_requests(name, 80, (190, 170, 120))
    reference = reference_logits(folders, name, requests)
    engine = make_engine(folders, name, dtype, pages=80, max_requests=3)
    heads = {"r0": 30, "r1": 12}
    seen = {}
    engine.step([StepEntry(k, requests[k][:n], [n - 1]) for k, n in heads.items()])
    at = dict(heads)
    for step in range(160):
        if step == 40:       # r2 joins with a prompt of its own beside the decoded tokens
            at["r2"] = 0
        entries, places = [], []
        for key in list(at):
            ids = requests[key]
            if at[key] >= len(ids):
                engine.release(key)
                del at[key]
                continue
            count = 17 if key == "r2" and at[key] == 0 else 1
            entries.append(StepEntry(key, ids[at[key]:at[key] + count], [count - 1]))
            places.append((key, at[key] + count - 1))
            at[key] += count
        if not entries:
            break
        logits = engine.step(entries).double().cpu().numpy()
        for row, place in enumerate(places):
            seen[place] = logits[row]
    engine.check()
    assert len(seen) > 400
    compare_replay(name, dtype, seen, reference)
    if engine.graphs is not None:
        assert engine.graphs.sizes_captured()      # decode steps did run as graphs


@gpu
def test_fork_copies_pages_and_state(folders):
    from metallix_b200.engine import StepEntry
    name = "small"
    _, config, tensors, _ = folders[name]
    ids = random_ids(3, 40, config["vocab"])
    other = ids[:22] + random_ids(4, 18, config["vocab"])
    engine = make_engine(folders, name, "float32", pages=64)
    engine.step([StepEntry("p", ids[:22], [])])
    engine.fork("p", "c")
    a = engine.step([StepEntry("p", ids[22:], list(range(18))), StepEntry("c", other[22:], list(range(18)))])
    engine.check()
    want = np.concatenate([plain.forward_logits(config, tensors, ids)[22:], plain.forward_logits(config, tensors, other)[22:]])
    assert np.abs(a.double().cpu().numpy() - want).max() < TOL["float32"]


# ------------------------------------- generation, scheduler, command line
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(folders, dtype):
    """``generate`` (scheduler, continuous batching, captured decode steps):
    every generated token is the plain side's argmax, or (bfloat16) within a
    near tie of it."""
    from metallix_b200.engine.generate import generate
    name = "small"
    _, config, tensors, _ = folders[name]
    engine = make_engine(folders, name, dtype, pages=64, max_requests=4)
    prompts = [random_ids(90 + n, length, config["vocab"]) for n, length in enumerate((5, 31, 1, 12, 18, 2))]
    results = generate(engine, prompts, max_new_tokens=12, eos_ids=())
    for prompt, result in zip(prompts, results):
        assert len(result.generated_ids) == 12 and not result.failed
        ids = list(prompt)
        for token in result.generated_ids:
            row = plain.forward_logits(config, tensors, ids)[-1]
            best = int(np.argmax(row))
            if token != best:
                assert dtype == "bfloat16" and row[best] - row[token] < 0.5, (dtype, token, best)
            ids.append(token)


@gpu
def test_trace_program_and_command_line(folders, tmp_path):
    """bin/trace_run on a mixed schedule and bin/mxb gen, as programs."""
    name = "small"
    folder, config, tensors, page = folders[name]
    requests = some_requests(name, 70, (30, 12, 44))
    reference = reference_logits(folders, name, requests)
    steps, peak = cuts.mixed(requests, seed=9, max_live=2, decode_tail=6)
    out = tmp_path / "logits"
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(peak)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    offsets = {}
    for step in steps:
        for e in step["entries"]:
            offsets.setdefault(e["id"], 0)
        want = cuts.expected_rows(step, offsets, reference)
        if want is not None:
            got = np.fromfile(out / f"{step['step']}.f32", dtype="<f4").reshape(want.shape)
            assert np.abs(got - want).max() < TOL["float32"]
        for e in step["entries"]:
            offsets[e["id"]] += len(e["tokens"])
    prompt = requests["r1"]
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mxb"), "gen", "--model", folder, "--input-ids",
                           ",".join(map(str, prompt)), "--max-tokens", "4", "--dtype", "float32", "--verify-cache"],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    receipt = json.loads(done.stdout.strip().splitlines()[-1])
    ids = list(prompt)
    for _ in range(4):
        ids.append(int(np.argmax(plain.forward_logits(config, tensors, ids)[-1])))
    assert receipt["generated_ids"] == ids[len(prompt):]
    assert receipt["operation"] == "sadosun_greedy_cached_generation"
    assert receipt["cache_comparisons"]["logits_within_bound"]

"""The Dimorax decoder in the engine against the plain implementation
(``plain_dimorax.py``): its configuration and mechanisms one at a time, then
whole prompts layer by layer, decoding through the cache and the state,
portions, mixed batches, pages and slots that come back, keys at a window's
edge, far back and at page borders, the first tokens, long decoding,
generation through the scheduler and the trace program. Every model here is
tiny, made for the test with random weights, and differs from layer to layer."""
import dataclasses
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_dimorax as plain
import replay_helpers as cuts
from conftest import ROOT, random_ids


# ------------------------------------------------------------ configurations
def delta(heads, kv_heads, dim, vdim, conv, ranks):
    out = {"heads": heads, "dim": dim, "conv": conv, "ranks": {"decay": ranks[0], "gate": ranks[1]}}
    if kv_heads:
        out["kv_heads"] = kv_heads
    if vdim:
        out["vdim"] = vdim
    return out


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, window=0, rot=None, scaling=None, kv_from=None):
    out = {"heads": heads, "dim": dim, "scale": scale}
    if kv_heads:
        out["kv_heads"] = kv_heads
    if vdim:
        out["vdim"] = vdim
    if softcap:
        out["softcap"] = softcap
    if window:
        out["mask"] = {"size": window}
    if rot:
        out["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling:
            out["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def latent(heads, dim, rot_dim, vdim, rank, scale, window=0, base=1.0e4):
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
           "rot": {"base": base, "dims": rot_dim}}
    if window:
        out["mask"] = {"size": window}
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale=None, groups=None, shared=0):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# SMALL: sizes that are no power of two; values wider than keys; part of a head rotated with all three bands of
# the stretch; two heads per query/key group in the recurrence and one; a window shorter than a page of 8; a layer
# without feed-forward; a layer that reads another's keys and values through a window of its own; groups of two
# experts of which two of three are kept; every expert chosen; low ranks that differ.
SMALL = {"architecture": "Dimorax", "vocab": 197, "width": 72, "norm": {"eps": 1e-6}, "residual_mult": 0.45,
         "layers": [
             layer("channel_delta", delta(4, 2, 12, 20, 3, (5, 7)), moe(24, 6, 2, 1.7, (3, 2), 16)),
             layer("attention", attention(4, 2, 16, 24, 0.3, 5.0, 0, (100.0, 8), (4.0, 64, 4.0, 0.5)), dense(40)),
             layer("latent_attention", latent(3, 8, 4, 10, 20, 0.4, 7), None),
             layer("attention", attention(4, 2, 16, 24, 0.25, None, 13, (100.0, 8), (4.0, 64, 4.0, 0.5), kv_from=1),
                   moe(16, 3, 3)),
             layer("channel_delta", delta(2, 0, 40, 8, 2, (3, 2)), dense(56))]}
# WIDE: heads of 64 and 128 values with values as wide as keys (the tensor-core kernels' sizes), four query heads
# per key/value head, an attention with a window that ends inside a page of 16 and a reader of its keys with a
# shorter one, a latent attention whose keys are padded from 96 to 128 with a window that ends inside a key tile,
# a recurrence with one query/key group for four heads, 64 key channels and 128 value columns (two blocks a head).
WIDE = {"architecture": "Dimorax", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "residual_mult": 0.3,
        "layers": [
            layer("attention", attention(8, 2, 64, 64, 0.11, 30.0, 70, (1.0e5, 64)), moe(64, 8, 2, 2.0, (2, 1), 32)),
            layer("channel_delta", delta(4, 1, 64, 128, 4, (16, 8)), dense(192)),
            layer("latent_attention", latent(4, 64, 32, 64, 48, 0.09, 150), moe(32, 4, 1, None, None, 24)),
            layer("attention", attention(8, 2, 64, 64, 0.2, None, 33, (1.0e5, 64), kv_from=0), None)]}
# BARE: the switches' other position: no residual multiplier, no rotation, no cap, no window anywhere, a key/value
# head per query head and values as wide as keys by default, experts without groups, scale or shared expert, one
# expert of which one is chosen, a convolution of one tap (the current token alone).
BARE = {"architecture": "Dimorax", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
        "layers": [
            layer("attention", attention(2, 0, 8, 0, 0.5), moe(20, 1, 1)),
            layer("channel_delta", delta(1, 0, 5, 0, 1, (1, 1)), None),
            layer("latent_attention", {"heads": 2, "dim": 16, "rot_dim": 2, "vdim": 16, "kv_rank": 8, "scale": 0.2,
                                       "rot": {"base": 50.0, "dims": 2}}, dense(24))]}
MODELS = {"small": (SMALL, 41, 8, 1.0), "wide": (WIDE, 42, 16, 1.0), "bare": (BARE, 43, 4, 1.0),
          # score scales four times as large: which keys a query sees, and the sinks, decide its output
          "sharp": (SMALL, 44, 8, 4.0)}
CASES = [(name, dtype) for name in MODELS for dtype in ("float32", "bfloat16") if (name, dtype) != ("sharp", "bfloat16")]
TOL = {"float32": 1e-4, "bfloat16": 2.5e-1}
TOL_SHARP = 5e-4


def bound(name, dtype):
    return TOL_SHARP if name == "sharp" else TOL[dtype]


def compare_replay(name, dtype, seen, reference):
    """float32: every position within the bound. bfloat16: a router's close
    call may go the other way at a position or two, so the bound holds for 19
    positions out of 20, the median lies well inside it, and at most one
    position in fifty is off by the size of a logit; a lost state or a wrong
    key would put every position behind it there."""
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
        if spec["type"] != "channel_delta":
            spec["mixer"]["scale"] *= factor
    return raw


def write_folder(folder, raw, seed, sharpen):
    """config.json + model.safetensors: bfloat16 matrices, float32 vectors (so
    that the engine and the plain side hold the same values). Projections are
    larger than the generator's (0.02) so that scores, gates and states move;
    step sizes are small so that the state reaches far back; sinks and
    biases are of the size of the scores; the router's correction is large
    enough to change the choice."""
    from metallix_b200.config import DimoraxConfig
    from metallix_b200.weights import random_tensors
    from metallix_b200.weights.safetensors_io import write_file
    config = DimoraxConfig.from_dict(sharpened(raw, sharpen))
    tensors = random_tensors(config, seed, dtype="bfloat16", norm_dtype="float32")
    for name, value in tensors.items():
        last = name.rsplit(".", 1)[-1]
        if last == "conv":
            tensors[name] = (value.float() * 15.0).to(torch.bfloat16)
        elif last == "sink":
            tensors[name] = value * 15.0
        elif last == "correction":
            tensors[name] = value * 3.0
        elif last == "dt_bias":
            tensors[name] = value - 3.0
        elif last == "b" and value.dim() == 1:
            tensors[name] = value * 5.0
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
        folder = write_folder(str(tmp_path_factory.mktemp(f"dimorax_{name}")), raw, seed, sharpen)
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
    from metallix_b200.config import ConfigError, DimoraxConfig, parse_config, resolve
    for raw in (SMALL, WIDE, BARE):
        config = parse_config(raw)
        assert isinstance(config, DimoraxConfig) and resolve(raw).kind == "dimorax"
        assert DimoraxConfig.from_dict(config.to_dict()) == config
        assert json.loads(json.dumps(config.to_dict())) == config.to_dict()
        shapes, w = config.tensor_shapes(), raw["width"]
        assert shapes["embed"] == shapes["head"] == (raw["vocab"], w) and shapes["final.norm"] == (w,)
        for index, spec in enumerate(raw["layers"]):
            base, mixer = f"l{index}", spec["mixer"]
            assert shapes[f"{base}.norm1"] == (w,) and (f"{base}.norm2" in shapes) == (spec["mlp"] is not None)
            heads = mixer["heads"]
            if spec["type"] == "channel_delta":
                groups, vdim = mixer.get("kv_heads") or heads, mixer.get("vdim") or mixer["dim"]
                assert shapes[f"{base}.mix.q"] == shapes[f"{base}.mix.k"] == (groups * mixer["dim"], w)
                assert shapes[f"{base}.mix.v.conv"] == (heads * vdim, mixer["conv"]) and shapes[f"{base}.mix.norm"] == (vdim,)
                assert shapes[f"{base}.mix.a2"] == (heads * mixer["dim"], mixer["ranks"]["decay"])
                assert shapes[f"{base}.mix.g1"] == (mixer["ranks"]["gate"], w) and shapes[f"{base}.mix.b"] == (heads, w)
            elif spec["type"] == "attention":
                kv, vdim = mixer.get("kv_heads") or heads, mixer.get("vdim") or mixer["dim"]
                assert shapes[f"{base}.mix.q.b"] == (heads * mixer["dim"],) and shapes[f"{base}.mix.sink"] == (heads,)
                assert (f"{base}.mix.k" in shapes) == (f"{base}.mix.v.b" in shapes) == ("kv_from" not in mixer)
                assert "kv_from" in mixer or shapes[f"{base}.mix.v"] == (kv * vdim, w)
            else:
                assert shapes[f"{base}.mix.q"] == (heads * (mixer["dim"] + mixer["rot_dim"]), w)
                assert shapes[f"{base}.mix.dkv"] == (mixer["kv_rank"] + mixer["rot_dim"], w)
                assert shapes[f"{base}.mix.uv"] == (heads * mixer["vdim"], mixer["kv_rank"])
            if spec["mlp"] is not None and spec["mlp"]["kind"] == "moe":
                count = spec["mlp"]["router"]["experts"]
                assert shapes[f"{base}.mlp.router"] == (count, w) and shapes[f"{base}.mlp.e{count - 1}.gate"][1] == w
                assert (f"{base}.mlp.shared.sg" in shapes) == ("shared" in spec["mlp"])
        model = config.to_model_spec()
        assert [run.layer for run in model.order] == list(range(len(raw["layers"])))
        for run, spec in zip(model.order, raw["layers"]):       # a layer without keys reads the entry of the layer it names
            source = spec["mixer"].get("kv_from")
            assert (run.cache_entry(), run.write_cache) == ((run.layer, True) if source is None else (source, False))
        assert all(spec.block.kind == "parallel_residual" for spec in model.layers)
    open_ranks = json.loads(json.dumps(SMALL))
    del open_ranks["layers"][0]["mixer"]["ranks"]
    assert parse_config(open_ranks).tensor_shapes()["l0.mix.a1"] == (None, 72)     # left to the checkpoint's tensor
    refusals = [
        ("UnsupportedLayerType", lambda c: c["layers"][0].update(type="mamba1")),
        ("InvalidGroupedQueryLayout", lambda c: c["layers"][1]["mixer"].update(kv_heads=3)),
        ("InvalidGroupedQueryLayout", lambda c: c["layers"][0]["mixer"].update(kv_heads=3)),
        ("InvalidRotaryWidth", lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18)),
        ("InvalidRotaryWidth", lambda c: c["layers"][2]["mixer"]["rot"].update(dims=2)),
        ("UnsupportedFeedForward", lambda c: c["layers"][1]["mlp"].update(kind="relu")),
        ("Json", lambda c: c["layers"][0]["mlp"]["router"].update(top=5)),              # two kept groups hold four experts
        ("Json", lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4)),
        ("Json", lambda c: c["layers"][1]["mixer"].update(scale=0.0)),
        ("Json", lambda c: c["layers"][3]["mixer"].update(kv_from=2)),                  # not an attention layer
        ("Json", lambda c: c["layers"][3]["mixer"].update(kv_from=3)),                  # not an earlier layer
        ("Json", lambda c: c["layers"][3]["mixer"].update(kv_heads=1)),                 # another head layout than its source
        ("Json", lambda c: c["layers"][1]["mixer"].update(mask={"size": 5})),           # the source keeps fewer keys than the reader needs
        ("MissingDimension", lambda c: c.update(width=70)),
        ("InvalidRmsNormEpsilon", lambda c: c["norm"].update(eps=0.0)),
        ("MissingDimension", lambda c: c.update(layers=[]))]
    for kind, change in refusals:
        raw = json.loads(json.dumps(SMALL))
        change(raw)
        with pytest.raises(ConfigError) as caught:
            parse_config(raw)
        assert caught.value.kind == kind, (kind, caught.value.kind)


def test_random_weights_and_sizes_left_to_the_checkpoint(tmp_path):
    from metallix_b200.config import DimoraxConfig
    from metallix_b200.weights import CheckpointError, load_tensors, random_tensors, write_model_folder
    config = DimoraxConfig.from_dict(SMALL)
    tensors = random_tensors(config, 3, dtype="float32")
    assert float(tensors["l0.norm1"].abs().max()) <= 0.1 and float(tensors["final.norm"].abs().max()) <= 0.1
    assert abs(float(tensors["l0.mix.norm"].mean()) - 1.0) < 0.1 and float(tensors["l1.mix.sink"].abs().max()) <= 0.1
    assert float(tensors["l1.mix.q.b"].abs().max()) <= 0.1 and tensors["l0.mix.b"].shape == (4, 72)
    folder = write_model_folder(str(tmp_path / "m"), config, 3)
    assert set(load_tensors(folder, config)) == set(config.tensor_shapes())
    # the same folder under a config.json that does not name the two low ranks: the tensors give them
    raw = json.loads(json.dumps(SMALL))
    for spec in raw["layers"]:
        spec["mixer"].pop("ranks", None)
    unnamed = DimoraxConfig.from_dict(raw)
    assert load_tensors(folder, unnamed)["l0.mix.a1"].shape == (5, 72)
    with pytest.raises(ValueError):
        random_tensors(unnamed, 3)
    raw["layers"][4]["mixer"]["dim"] = 32
    with pytest.raises(CheckpointError):
        load_tensors(folder, DimoraxConfig.from_dict(raw))


def test_cache_needs_and_the_shared_entry():
    """A recurrence keeps its matrix and its convolution's inputs; an attention
    pages; a layer without keys of its own has no entry and is handed its
    source's, read only."""
    from metallix_b200.config import DimoraxConfig
    from metallix_b200.engine.model import DecoderModel
    from metallix_b200.parts.registry import Runtime
    from metallix_b200.weights import random_tensors
    config = DimoraxConfig.from_dict(SMALL)
    model = DecoderModel(config.to_model_spec(), random_tensors(config, 1, dtype="float32"),
                         Runtime(device=torch.device("cpu"), dtype=torch.float32, max_positions=64))
    needs = model.cache_needs()
    flat = [None if need is None else [(n.kind, tuple(n.state_shape) if n.kind == "state" else (n.kv_heads, n.head_dim, n.window))
                                       for n in need.flat()] for need in needs]
    assert flat[0] == [("state", (4, 20, 12)), ("state", (2, 2 * 2 * 12 + 4 * 20))]
    assert flat[1] == [("kv_pages", (2, 24, None))] and flat[2] == [("kv_pages", (3, 64, 7))]
    assert flat[3] is None and flat[4] == [("state", (2, 8, 40)), ("state", (1, 2 * 2 * 40 + 2 * 8))]
    assert not model.blocks[3].mixer.own_keys and model.blocks[3].mixer.qkv.out_features == 4 * 16


def test_the_plain_side_in_pieces():
    """The plain implementation itself: logits do not change when more tokens
    follow; the recurrence in pieces, its state and its convolutions' inputs
    handed on, equals one run; the sink takes its share; experts outside the
    kept groups cannot be chosen even where all corrected scores are negative;
    the stretch keeps fast pairs and slows the slow ones."""
    from metallix_b200.config import DimoraxConfig
    rng = np.random.default_rng(0)
    shapes = DimoraxConfig.from_dict(SMALL).tensor_shapes()
    tensors = {name: rng.normal(size=shape) * (0.1 if len(shape) <= 1 else 0.3) for name, shape in shapes.items()}
    ids = random_ids(1, 30, 197)
    whole = plain.forward_logits(SMALL, tensors, ids)
    assert np.allclose(plain.forward_logits(SMALL, tensors, ids[:19]), whole[:19], atol=1e-10)
    h = rng.normal(size=(25, 72))
    mixer = SMALL["layers"][0]["mixer"]
    once, _ = plain.channel_delta(h, tensors, "l0.mix", mixer, 1e-6)
    first, carry = plain.channel_delta(h[:2], tensors, "l0.mix", mixer, 1e-6)
    second, carry = plain.channel_delta(h[2:11], tensors, "l0.mix", mixer, 1e-6, carry)
    third, _ = plain.channel_delta(h[11:], tensors, "l0.mix", mixer, 1e-6, carry)
    assert np.allclose(np.concatenate([first, second, third]), once, atol=1e-12)
    # one step of the rule by hand: a write into an empty state is read back by the same token
    q, k, v = np.array([[0.6, 0.8]]), np.array([[1.0, 0.0]]), np.array([[2.0, -1.0, 0.5]])
    out, state = plain.delta_rule(q, k, v, np.array([0.5]), np.array([[0.9, 0.9]]))
    assert np.allclose(state, np.outer(k[0], 0.5 * v[0])) and np.allclose(out[0], 0.6 * 0.5 * v[0])
    out, state = plain.delta_rule(q, k, v, np.array([1.0]), np.array([[0.5, 0.5]]), state)
    assert np.allclose(state[0], v[0])      # beta 1: the key's row now holds the value whatever it held
    scores = rng.normal(size=(4, 9))
    seen = np.ones((4, 9), dtype=bool)
    p = plain.sink_softmax(scores, seen, 0.7)
    assert np.allclose(p.sum(axis=1), 1.0 - np.exp(0.7) / (np.exp(0.7) + np.exp(scores).sum(axis=1)))
    assert plain.seen_keys(6, 2).sum() == 11 and plain.seen_keys(6, 0).sum() == 21
    logits = np.array([[-9.0, -8.0, -1.0, -7.0, -2.0, -9.5]])       # sigmoids near 0; corrections make every choice score negative
    correction = np.full(6, -1.0)
    chosen, weights = plain.choose_experts(logits, correction, 2, {"count": 3, "keep": 1}, 2.0)
    assert sorted(chosen[0].tolist()) == [2, 3] and np.isclose(weights.sum(), 2.0)       # group 1 = experts 2, 3 has the largest two-sum
    chosen, _ = plain.choose_experts(logits, correction, 2)
    assert sorted(chosen[0].tolist()) == [2, 4]
    f, magnitude = plain.yarn_frequencies(100.0, 8, {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 0.5})
    plain_f = 100.0 ** (-2.0 * np.arange(4) / 8)
    assert np.isclose(f[0], plain_f[0]) and np.isclose(f[3], plain_f[3] / 4.0) and plain_f[1] / 4 < f[1] < plain_f[1]
    assert np.isclose(magnitude, 0.1 * np.log(4.0) + 1.0)


def test_the_models_of_these_tests_show_a_window_a_sink_a_state_and_a_source(folders):
    """What the tests below can see: on the plain side, windows one position
    longer, a softmax without the sinks, a state lost at one position and keys
    of its own layer instead of its source's each move the logits by far more
    than the bound the engine is held to."""
    _, config, tensors, _ = folders["sharp"]
    tensors = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    ids = random_ids(40, 75, config["vocab"])
    base = plain.forward_logits(config, tensors, ids)
    longer = json.loads(json.dumps(config))
    for spec in longer["layers"]:
        if "mask" in spec["mixer"]:
            spec["mixer"]["mask"]["size"] += 1
    own = json.loads(json.dumps(config))
    own["layers"][3]["mixer"]["kv_from"] = 3        # the plain side then looks its keys up under its own index: missing
    lost = np.concatenate([plain.forward_logits(config, tensors, ids[:60]), plain.forward_logits(config, tensors, ids[60:])])
    gaps = {"window": np.abs(plain.forward_logits(longer, tensors, ids) - base)[20:].max(),
            "sink": np.abs(plain.forward_logits(config, tensors, ids, use_sink=False) - base).max(),
            "state": np.abs(lost - base)[60:].max()}
    assert min(gaps.values()) > 100 * TOL_SHARP, gaps
    with pytest.raises(KeyError):
        plain.forward_logits(own, tensors, ids)


# --------------------------------------------------------- mechanisms alone
gpu = pytest.mark.gpu


def dev(array, dtype=torch.float32):
    return torch.tensor(np.asarray(array), dtype=dtype, device="cuda")


def rounded(array, dtype):
    return torch.tensor(np.asarray(array), dtype=dtype).double().numpy()


def rows_of(lengths):
    starts, cursor = [], 0
    for length in lengths:
        starts.append(cursor)
        cursor += length
    return starts


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, groups, dim, vdim", [(4, 2, 12, 20), (2, 2, 40, 8), (1, 1, 5, 5), (4, 1, 64, 128), (3, 3, 128, 72),
                                                      (2, 1, 200, 33)])
def test_delta_rule_kernel(dtype, heads, groups, dim, vdim):
    """The recurrence over request rows of unequal length in one launch (a
    single token, a padding row), continued twice from the state the launch
    before left, against the plain rule in one piece. Decays are slow, the
    first token's value is large and the last token's query is the first
    token's key, so that what the first token wrote is what the last one
    reads."""
    from metallix_b200 import ops
    rng = np.random.default_rng(heads * dim + vdim)
    pieces = [[23, 1, 0, 5], [1, 1, 0, 40], [9, 3, 0, 1]]
    slots = [2, 0, 1, 3]
    totals = [sum(p[row] for p in pieces) for row in range(4)]
    rate = rounded(np.exp(rng.normal(size=heads) * 0.3), torch.float32)
    bias = rounded(rng.normal(size=heads * dim) * 0.5 - 4.0, torch.float32)
    seq = []
    for total in totals:
        first = np.where(np.arange(total) == 0, 64.0, 1.0)[:, None]
        q_rows, k_rows = rng.normal(size=(total, groups * dim)), rng.normal(size=(total, groups * dim))
        if total > 30:
            q_rows[-1] = k_rows[0]
        seq.append({"q": rounded(q_rows, dtype), "k": rounded(k_rows, dtype),
                    "v": rounded(rng.normal(size=(total, heads * vdim)) * first, dtype),
                    "b": rounded(rng.normal(size=(total, heads)) * 2.0, dtype),
                    "s": rounded(rng.normal(size=(total, heads * dim)), torch.float32)})
    state = torch.full((5, heads, vdim, dim), 3.0, device="cuda")      # S transposed: a column's channels side by side
    for slot in slots:
        state[slot].zero_()
    got = [[] for _ in totals]
    done = [0] * 4
    for lengths in pieces:
        starts = rows_of(lengths)
        pack = lambda key: np.concatenate([seq[row][key][done[row]:done[row] + n] for row, n in enumerate(lengths)])
        qkv = dev(np.concatenate([np.zeros((sum(lengths), 8)), pack("q"), pack("k"), pack("v")], axis=1), dtype)
        wide = dev(np.concatenate([pack("b"), np.zeros((sum(lengths), 3))], axis=1), dtype)
        out = ops.delta_rule(qkv, (8, 8 + groups * dim, 8 + 2 * groups * dim), wide[:, :heads], dev(pack("s")), dev(bias), dev(rate),
                             state, dev(starts, torch.int32), dev(lengths, torch.int32), dev(slots, torch.int32), heads, groups, dim, vdim)
        ops.check_status("cuda")
        for row, n in enumerate(lengths):
            got[row].append(out[starts[row]:starts[row] + n].double().cpu().numpy())
            done[row] += n
    assert float(state[4].min()) == 3.0 and float(state[1].abs().max()) == 0.0      # an untouched slot, a padding row's slot
    unit = lambda x: x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)
    for row, total in enumerate(totals):
        if not total:
            continue
        s = seq[row]
        q = unit(s["q"].reshape(total, groups, dim)) * dim ** -0.5
        k = unit(s["k"].reshape(total, groups, dim))
        decay = np.exp(-rate[None, :, None] * plain.softplus(s["s"] + bias).reshape(total, heads, dim))
        for head in range(heads):
            group = head // (heads // groups)
            want, last = plain.delta_rule(q[:, group], k[:, group], s["v"][:, head * vdim:(head + 1) * vdim],
                                          plain.sigmoid(s["b"][:, head]), decay[:, head])
            have = np.concatenate(got[row])[:, head * vdim:(head + 1) * vdim]
            assert np.abs(have - want).max() < 2e-4 * max(1.0, np.abs(want).max()), (row, head)
            assert np.abs(state[slots[row], head].double().cpu().numpy().T - last).max() < 2e-4 * max(1.0, np.abs(last).max())
            if total > 30:       # without the first token's write the last output is another
                again, _ = plain.delta_rule(q[1:, group], k[1:, group], s["v"][1:, head * vdim:(head + 1) * vdim],
                                            plain.sigmoid(s["b"][1:, head]), decay[1:, head])
                assert np.abs(again[-1] - want[-1]).max() > 10 * 2e-4 * max(1.0, np.abs(want).max())


@gpu
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("size", [72, 128, 2056])
def test_the_sum_of_two_sublayers_and_both_norms(out_dtype, size):
    """x += m (a + b) with a and b of either type or absent, then two norms of
    the same row with weights of their own; the sum alone; picked rows; a
    projection's bias joining its float32 result ahead of the rounding."""
    from metallix_b200 import ops
    rng = np.random.default_rng(size)
    rows, m, eps = 9, 0.3, 1e-5
    x = rounded(rng.normal(size=(rows, size)) * 3.0, torch.float32)
    w1, w2 = rounded(1.0 + rng.normal(size=size) * 0.2, torch.float32), rounded(1.0 + rng.normal(size=size) * 0.2, torch.float32)
    tolerance = 1e-5 if out_dtype == torch.float32 else 4e-2
    for a_type, b_type in ((torch.bfloat16, torch.float32), (torch.float32, None), (None, torch.bfloat16), (None, None)):
        a = rounded(rng.normal(size=(rows, size)), a_type) if a_type else None
        b = rounded(rng.normal(size=(rows, size)), b_type) if b_type else None
        stream = dev(x)
        first, second = ops.pair_add_rmsnorm(stream, dev(a, a_type) if a_type else None, dev(b, b_type) if b_type else None, m,
                                             dev(w1), dev(w2), eps, out_dtype)
        total = x + m * ((a if a is not None else 0.0) + (b if b is not None else 0.0))
        assert np.abs(stream.double().cpu().numpy() - total).max() < 1e-5
        assert np.abs(first.double().cpu().numpy() - plain.over_rms(total, eps) * w1).max() < tolerance
        assert np.abs(second.double().cpu().numpy() - plain.over_rms(total, eps) * w2).max() < tolerance
        only = ops.pair_add_rmsnorm(dev(x), dev(a, a_type) if a_type else None, None, m, dev(w1), None, eps, out_dtype)
        assert np.abs(only.double().cpu().numpy() - plain.over_rms(x + m * (a if a is not None else 0.0), eps) * w1).max() < tolerance
    stream = dev(x)
    assert ops.pair_add_rmsnorm(stream, dev(a, torch.bfloat16) if False else None, dev(x), 2.0, None, None, 0.0, torch.float32) is None
    assert np.abs(stream.double().cpu().numpy() - 3.0 * x).max() < 1e-5
    picked = ops.pair_add_rmsnorm(dev(x), None, None, 1.0, dev(w1), None, eps, out_dtype, rows_index=dev([7, 0, 3], torch.int32))
    assert np.abs(picked.double().cpu().numpy() - (plain.over_rms(x, eps) * w1)[[7, 0, 3]]).max() < tolerance
    product, bias = rounded(rng.normal(size=(rows, size + 8)), torch.float32), rounded(rng.normal(size=size), torch.float32)
    summed = ops.add_bias(dev(product)[:, 8:], dev(bias), out_dtype)
    assert np.abs(summed.double().cpu().numpy() - rounded(product[:, 8:] + bias, out_dtype)).max() < 1e-6


@gpu
@pytest.mark.parametrize("experts, top, groups", [(6, 2, (3, 2)), (8, 2, (2, 1)), (8, 3, (4, 3)), (3, 3, None), (1, 1, None),
                                                   (64, 6, (8, 3)), (12, 4, (12, 5))])
def test_router_with_sigmoid_scores_and_groups(experts, top, groups):
    """Scores are sigmoids; the choice goes by score plus correction inside the
    kept groups; weights are the chosen scores over their sum times a scale.
    Half of the rows have corrections that make every choice score negative:
    an expert outside the kept groups must still not be chosen. The logits are
    a column range of a wider product."""
    from metallix_b200 import ops
    rng = np.random.default_rng(experts * top)
    tokens = 37
    logits = rounded(rng.normal(size=(tokens, experts)) * 2.0, torch.float32)
    logits[tokens // 2:] -= 6.0
    correction = rounded(rng.normal(size=experts) * 0.3 - 0.5, torch.float32)
    wide = dev(np.concatenate([logits, np.zeros((tokens, 3))], axis=1))
    chosen, weights, dense, on_identity = ops.route_experts(wide[:, :experts], dev(correction), experts, top, scores="sigmoid",
                                                           groups=groups, scale=2.5)
    want_chosen, want_weights = plain.choose_experts(logits, correction, top,
                                                     {"count": groups[0], "keep": groups[1]} if groups else None, 2.5)
    assert (np.sort(chosen.cpu().numpy(), axis=1) == np.sort(want_chosen, axis=1)).all()
    order = np.argsort(chosen.cpu().numpy(), axis=1)
    want_order = np.argsort(want_chosen, axis=1)
    assert np.abs(np.take_along_axis(weights.double().cpu().numpy(), order, 1) -
                  np.take_along_axis(want_weights, want_order, 1)).max() < 1e-5
    assert float(on_identity.abs().max()) == 0.0 and np.abs(dense.sum(dim=1).double().cpu().numpy() - 2.5).max() < 1e-4


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [1, 5, 300])
def test_gated_experts_row_by_row_and_grouped(dtype, tokens):
    """Experts down(silu(gate(h)) * up(h)) through the part itself: one token
    and float32 go row by row through the chosen experts' rows, more tokens in
    bfloat16 through the grouped tensor-core products with the activation in
    the first one's epilogue; a shared expert behind its gate joins both."""
    from metallix_b200.config.spec import PartSpec
    from metallix_b200.parts.registry import Runtime, WeightStore, build_part
    rng = np.random.default_rng(tokens)
    hidden, ff, experts, top, shared_ff = 64, 40, 5, 2, 24
    names = {}
    for e in range(experts):
        names.update({f"e{e}.gate": (ff, hidden), f"e{e}.up": (ff, hidden), f"e{e}.down": (hidden, ff)})
    names.update({"router": (experts, hidden), "shared.gate": (shared_ff, hidden), "shared.up": (shared_ff, hidden),
                  "shared.down": (hidden, shared_ff), "shared.sg": (1, hidden)})
    tensors = {f"m.{k}": rounded(rng.normal(size=shape) * 0.3, torch.bfloat16) for k, shape in names.items()}
    tensors["m.correction"] = rounded(rng.normal(size=experts) * 0.2, torch.float32)
    spec = PartSpec("routed_experts", {
        "hidden_size": hidden, "intermediate_size": ff, "experts": experts, "identity": 0, "top": top, "activation": "swiglu",
        "scores": "sigmoid", "scale": 1.5, "groups": None, "gate_proj": "m.e{}.gate", "up_proj": "m.e{}.up",
        "down_proj": "m.e{}.down", "router": "m.router", "correction": "m.correction", "shared_gate": "m.shared.sg",
        "shared": PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": shared_ff, "gate_proj": "m.shared.gate",
                                      "up_proj": "m.shared.up", "down_proj": "m.shared.down", "activation": "silu"})})
    part = build_part("feed_forward", spec, WeightStore({k: torch.tensor(v) for k, v in tensors.items()}),
                      Runtime(device=torch.device("cuda"), dtype=dtype, max_positions=16))
    h = rounded(rng.normal(size=(tokens, hidden)), dtype)
    got = part.forward(dev(h, dtype), None).double().cpu().numpy()
    mlp = {"router": {"experts": experts, "top": top, "scale": 1.5}, "shared": {"ff": shared_ff}}
    chosen = []
    want = plain.expert_mixture(h, tensors, "m", mlp, chosen)
    errors = np.abs(got - want).max(axis=1)
    if dtype == torch.float32:
        assert errors.max() < 1e-4
    else:       # a close call of the router may go the other way for a token in a hundred
        assert np.quantile(errors, 0.97) < 6e-2 * max(1.0, np.abs(want).max())


@gpu
@pytest.mark.parametrize("rows", [1, 8, 40, 1600])
def test_gated_feed_forward_with_the_tanh_form_of_gelu(rows):
    """act(gate) * up with gelu in every kernel that holds the activation: the
    pass of its own, the few-row products' epilogue, the tensor-core product's."""
    from metallix_b200 import ops, tensor_core
    rng = np.random.default_rng(rows)
    hidden, ff = 128, 192
    x = rounded(rng.normal(size=(rows, hidden)), torch.bfloat16)
    w = rounded(rng.normal(size=(2 * ff, hidden)) * 0.2, torch.bfloat16)
    gate_up = rounded(x @ w.T, torch.bfloat16)
    want = plain.gelu_tanh(gate_up[:, :ff]) * gate_up[:, ff:]
    tolerance = 3e-2 * max(1.0, np.abs(want).max())
    for dtype in (torch.float32, torch.bfloat16):
        got = ops.silu_mul(dev(rounded(gate_up, dtype), dtype), activation="gelu_tanh")
        assert np.abs(got.double().cpu().numpy() - want).max() < (1e-5 if dtype == torch.float32 else tolerance)
        assert np.abs(ops.silu_mul(dev(gate_up, dtype)).double().cpu().numpy() - plain.silu(gate_up[:, :ff]) * gate_up[:, ff:]).max() < tolerance
    if rows <= 16:
        for kernel in ("stream", "load"):
            got = ops.gemm_skinny(dev(x, torch.bfloat16), dev(w, torch.bfloat16), swiglu=True, kernel=kernel, activation="gelu_tanh")
            assert np.abs(got.double().cpu().numpy() - want).max() < tolerance, kernel
    got = tensor_core.gemm_swiglu(dev(x, torch.bfloat16), dev(w, torch.bfloat16), activation="gelu_tanh")
    assert np.abs(got.double().cpu().numpy() - want).max() < tolerance


@gpu
def test_stretched_wavelengths_in_the_position_tables():
    from metallix_b200.config.spec import PartSpec
    from metallix_b200.parts.registry import Runtime, WeightStore, build_part
    runtime = Runtime(device=torch.device("cuda"), dtype=torch.float32, max_positions=700)
    for base, dims, scaling in ((100.0, 8, {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 0.5}),
                                (1.0e6, 48, {"factor": 16.0, "original": 512, "fast": 8.0, "slow": 2.0}), (50.0, 2, None)):
        part = build_part("position", PartSpec("rope_half", {"theta": base, "rotary_dim": dims, "head_dim": dims + 4,
                                                             "scaling": scaling}), WeightStore({}), runtime)
        f, magnitude = plain.yarn_frequencies(base, dims, scaling)
        angle = np.arange(700)[:, None] * f[None, :]
        assert np.abs(part.cos.double().cpu().numpy() - np.cos(angle) * magnitude).max() < 1e-6
        assert np.abs(part.sin.double().cpu().numpy() - np.sin(angle) * magnitude).max() < 1e-6
        x = np.random.default_rng(dims).normal(size=(5, 3, dims + 4))
        positions = [0, 1, 77, 300, 699]
        from metallix_b200 import ops
        got = ops.norm_rotate_heads(dev(x.reshape(5, -1)), dims + 4, dev(positions, torch.int32), cos=part.cos, sin=part.sin)
        assert np.abs(got.double().cpu().numpy() - plain.turn_halves(x, positions, base, dims, scaling)).max() < 1e-4


@gpu
@pytest.mark.parametrize("dtype, head_dim, heads, kv_heads, context, page, window", [
    (torch.bfloat16, 64, 8, 2, 700, 16, 150), (torch.bfloat16, 128, 4, 4, 2300, 16, 0), (torch.float32, 64, 4, 2, 500, 8, 129),
    (torch.float32, 24, 3, 1, 200, 4, 0), (torch.bfloat16, 40, 6, 3, 300, 8, 37)])
def test_a_learned_sink_per_head_in_every_attention_kernel(dtype, head_dim, heads, kv_heads, context, page, window):
    """Every query head has a sink score of its own (of the size of all its keys' weights together) in the
    general kernel, the split-key decode kernels and both tensor-core prompt
    kernels. One query looks for the oldest key its window still holds and one
    for the key just outside it; with no window one looks hundreds of
    positions back."""
    from metallix_b200 import ops
    rng = np.random.default_rng(head_dim + context)
    scale, tail = 0.15, 24
    sink = rounded(rng.uniform(-3.0, 3.0, size=heads) + np.log(window or context), torch.float32)   # of the size of the keys' sum
    keys = rng.normal(size=(context, kv_heads, head_dim)) * 0.5
    values = rng.normal(size=(context, kv_heads, head_dim))
    q = rng.normal(size=(tail, heads, head_dim)) * 0.5
    group, first, reach = heads // kv_heads, context - tail, window or context

    def look_for(t, key, factor=6.0):
        keys[key] *= factor
        q[t] = np.repeat(keys[key], group, axis=0) * 1.5

    if window:
        look_for(4, first + 4 - (reach - 1))       # the oldest key query 4 still sees
        look_for(7, first + 7 - reach)             # one older than the oldest that query 7 sees
    else:
        look_for(tail - 1, 5)                      # far back
    look_for(10, (first + 10) // page * page)      # a page's first row
    keys, values, q = rounded(keys, dtype), rounded(values, dtype), rounded(q, dtype)
    pages = -(-context // page)
    order = rng.permutation(pages + 2)[:pages]
    pool = torch.zeros((pages + 2, 2, kv_heads, page, head_dim), dtype=dtype, device="cuda")
    for p in range(pages):
        span = slice(p * page, min((p + 1) * page, context))
        n = span.stop - span.start
        pool[order[p], 0, :, :n] = dev(keys[span].transpose(1, 0, 2), dtype)
        pool[order[p], 1, :, :n] = dev(values[span].transpose(1, 0, 2), dtype)
    positions = np.arange(first, context)
    k_all, v_all = np.repeat(keys, group, axis=1), np.repeat(values, group, axis=1)
    want, plain_softmax = np.zeros((tail, heads, head_dim)), np.zeros((tail, heads, head_dim))
    for t, p in enumerate(positions):
        low = max(0, p - reach + 1)
        s = np.einsum("hd,jhd->hj", q[t], k_all[low:p + 1]) * scale
        for h in range(heads):
            w = plain.sink_softmax(s[h:h + 1], np.ones_like(s[h:h + 1], dtype=bool), float(sink[h]))
            want[t, h] = w[0] @ v_all[low:p + 1, h]
            plain_softmax[t, h] = plain.sink_softmax(s[h:h + 1], np.ones_like(s[h:h + 1], dtype=bool), None)[0] @ v_all[low:p + 1, h]
    tolerance = 3e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(want - plain_softmax).max() > 10 * tolerance      # the sinks take a share that shows
    tables, sinks = dev(order[None, :], torch.int32), dev(sink)
    out = torch.empty((tail, heads, head_dim), dtype=dtype, device="cuda")
    ops.paged_attention_tile(dev(q, dtype), pool, out, tables, dev([0, 0], torch.int32), dev([0, 16], torch.int32),
                             dev([16, tail - 16], torch.int32), dev(positions, torch.int32), scale, window, sink=sinks)
    ops.check_status("cuda")
    assert np.abs(out.double().cpu().numpy() - want).max() < tolerance
    if ops.decode_attention_supported(head_dim, heads, kv_heads, dtype):
        for t in (4, 7, 10, tail - 1):      # each as a single decoded token behind its context
            one = torch.empty((1, heads, head_dim), dtype=dtype, device="cuda")
            ops.paged_attention_decode(dev(q[t:t + 1], dtype), pool, one, tables, dev([0], torch.int32), dev([0], torch.int32),
                                       dev(positions[t:t + 1], torch.int32), scale, int(positions[t]) + 1, window, sink=sinks)
            ops.check_status("cuda")
            assert np.abs(one.double().cpu().numpy()[0] - want[t]).max() < tolerance, t
    if ops.flash_prefill_supported(head_dim, heads, kv_heads, dtype):
        for kernel in ("tcgen05", "mma"):
            if kernel == "tcgen05" and not ops.flash_prefill_tcgen05_supported(head_dim, heads, kv_heads, page, dtype):
                continue
            for longest in (0, context):
                out.zero_()
                ops.flash_prefill(dev(q, dtype), pool, out, tables, dev([0], torch.int32), dev([0], torch.int32),
                                  dev([tail], torch.int32), dev(positions, torch.int32), scale, window, kernel=kernel,
                                  longest_context=longest, sink=sinks)
                ops.check_status("cuda")
                assert np.abs(out.double().cpu().numpy() - want).max() < tolerance, (kernel, longest)


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


@gpu
@pytest.mark.parametrize("name, dtype", CASES)
def test_decoding_and_portions_against_whole_prompts(folders, name, dtype):
    """The same requests as whole prompts, with their tails decoded one by one
    (over more tokens than the longest window, so that it passes over decoded
    tokens), and in portions of changing size down to two tokens (and one)."""
    from metallix_b200.engine import StepEntry
    requests = some_requests(name, 40, (75, 9, 33, 330 if name == "wide" else 50))
    reference = reference_logits(folders, name, requests)
    for schedule in (cuts.whole(requests), cuts.tail_by_one(requests, tail=45), cuts.ragged(requests),
                     cuts.ragged(requests, sizes=(2, 2, 3, 1, 2, 4, 9, 2))):
        engine = make_engine(folders, name, dtype, pages=64, max_requests=2)
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
def test_the_latent_kept_once_for_all_heads(folders, dtype):
    """The latent attention's other cache mode (one row of latent and rotated
    key part per position, shared by the heads) with its window and sinks:
    whole prompts, then tails decoded over the window's edge."""
    from metallix_b200.config import DimoraxConfig
    from metallix_b200.config.spec import PartSpec
    from metallix_b200.engine import Engine, StepEntry
    from metallix_b200.weights import load_tensors
    name = "small"
    folder, config, tensors, page = folders[name]
    typed = DimoraxConfig.from_dict(config)
    spec = typed.to_model_spec()
    layers = tuple(dataclasses.replace(layer, mixer=PartSpec(layer.mixer.kind, {**layer.mixer.params, "cache_mode": "latent"}))
                   if layer.mixer.kind == "latent_attention" else layer for layer in spec.layers)
    engine = Engine(typed, load_tensors(folder, typed, device="cuda"), dtype=dtype, page_tokens=page, num_pages=64,
                    max_requests=2, spec=dataclasses.replace(spec, layers=layers))
    assert [need.planes for need in engine.model.cache_needs()[2].flat()] == [1]
    requests = some_requests(name, 50, (60, 21))
    reference = reference_logits(folders, name, requests)
    for schedule in (cuts.whole(requests), cuts.tail_by_one(requests, tail=30)):
        _, seen = cuts.replay(engine, schedule, reference, StepEntry)
        compare_replay(name, dtype, seen, reference)


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
    assert receipt["cache_comparisons"]["logits_within_bound"]

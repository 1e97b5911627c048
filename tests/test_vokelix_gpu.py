"""The Vokelix decoder in the engine against the plain implementation (tests/plain_vokelix.py), GPU.

Every test makes its own small configuration and its own weights (numpy, rounded to bfloat16 so that
the float32 mode, the bfloat16 mode and the plain implementation see the same numbers).  Weights are
drawn so that faults show: the attention scale is large (peaked softmax: a missed or doubled key
changes the result), sinks are of the order of the scores, and the decays include values close to
one (a token far back still counts) and far from one.
"""
import json
import os
import struct
import subprocess

import numpy as np
import pytest
import plain_vokelix as pv
from util import assert_close, rel_err

from inferllm_b200 import Engine, EngineOptions, Model, ModelConfig, StepItem

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_model(folder, cfg, seed, sink_scale=2.0, norm2_always=False):
    """config.json + model.safetensors (bfloat16) with random weights; returns the float64 weights."""
    rng = np.random.default_rng(seed)
    w, blobs, header, off = {}, [], {}, 0
    for name, shape in pv.tensor_shapes(cfg, norm2_always).items():
        fan_in = shape[-1]
        if name.endswith(".sink"):
            a = rng.normal(0, sink_scale, shape)
        elif name.endswith((".q.norm", ".k.norm", "mix.norm")):
            a = 1.0 + rng.normal(0, 0.2, shape)
        elif len(shape) == 1:            # biases and norm offsets
            a = rng.normal(0, 0.3, shape)
        elif name == "embed":
            a = rng.normal(0, 1.0, shape)
        else:
            a = rng.normal(0, 1.0 / np.sqrt(fan_in), shape)      # larger gains make the stack chaotic: rounding then decides
        bits = to_bf16_bits(a)
        w[name] = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64).reshape(shape)
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + bits.nbytes]}
        blobs.append(bits.tobytes())
        off += bits.nbytes
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return w


def engine(folder, dtype, max_tokens=1024, page_size=64, max_seq_len=512, poison=False, max_batch=None):
    return Engine.from_folder(folder, EngineOptions(dtype=dtype, max_tokens=max_tokens, page_size=page_size, max_seq_len=max_seq_len,
                                                    poison_freed_pages=poison, max_batch=max_batch))


def whole(eng, ids):
    s = eng.new_sequence()
    lg = eng.step([StepItem(s, list(ids), list(range(len(ids))))]).cpu().numpy()
    eng.end_sequence(s)
    return lg


def in_portions(eng, ids, sizes):
    """The sequence in steps of the given sizes (the last size repeats)."""
    s, at, out, k = eng.new_sequence(), 0, [], 0
    while at < len(ids):
        n = min(sizes[min(k, len(sizes) - 1)], len(ids) - at)
        out.append(eng.step([StepItem(s, list(ids[at:at + n]), list(range(n)))]).cpu().numpy())
        at += n
        k += 1
    eng.end_sequence(s)
    return np.concatenate(out)


def same_or_close(a, b, dtype, what):
    """float32: the engine's kernels fix the order of every sum per row, so two ways of cutting the
    same tokens give the same bits; bfloat16: the library's products choose kernels by shape."""
    if dtype == "float32":
        assert np.array_equal(a, b), f"{what}: float32 logits differ between two cuttings (max {np.abs(a - b).max():.3e})"
    else:
        assert rel_err(a, b) <= 4e-2, what


CONFIGS = {
    # every mixer, keys and values shared by a later layer, value size != key size, partial rotations
    "mixed": lambda rng: pv.random_config(rng, ("lightning", "attention", "retention", "attention", "lightning"), share_from={3: 1},
                                          scale=1.0, ret_rot_dims=4),
    # other sizes: one kv head per query head, whole-head rotation without scaling, one linear head,
    # alpha 1, a layer without feed-forward, attention first
    "other": lambda rng: pv.random_config(rng, ("attention", "retention", "lightning", "attention"), width=40, vocab=61, heads=3, kv_heads=3,
                                          dim=24, vdim=8, rot_dims=24, scaling=None, scale=0.9, lin_heads=1, lin_dim=16, lin_vdim=8,
                                          decay=[0.97], ret_rot_dims=16, alpha=1.0, ff=48, no_mlp=[1], eps=1e-6),
    # head sizes the tensor-core kernels of other models take, one kv head for all query heads
    "wide": lambda rng: pv.random_config(rng, ("attention", "lightning", "retention"), width=64, vocab=128, heads=4, kv_heads=1, dim=64,
                                         vdim=64, rot_dims=16, scale=0.6, lin_heads=3, lin_dim=32, lin_vdim=64, decay=[0.6, 0.998, 0.9],
                                         ret_rot_dims=32, ff=96),
    # the other head size of the tensor-core kernels, two query heads per kv head, linear heads of 128 x 128
    "wide128": lambda rng: pv.random_config(rng, ("retention", "attention", "lightning", "attention"), share_from={3: 1}, width=96, vocab=150,
                                            heads=4, kv_heads=2, dim=128, vdim=128, rot_dims=64, scale=0.5, lin_heads=2, lin_dim=128,
                                            lin_vdim=128, decay=[0.9, 0.995], ret_rot_dims=64, ff=160),
}


def with_max_positions(cfg, n):
    cfg = dict(cfg)
    cfg["max_positions"] = n
    return cfg


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, make) in enumerate(CONFIGS.items()):
        rng = np.random.default_rng(100 + i)
        cfg = with_max_positions(make(rng), 1024)
        d = str(tmp_path_factory.mktemp("vk_" + name))
        out[name] = (d, cfg, write_model(d, cfg, 7 + i))
    return out


def prompt(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


# ------------------------------------------------------------------ each mechanism alone

ALONE = {
    "lightning": dict(layer_types=("lightning",)),
    "retention": dict(layer_types=("retention",), ret_rot_dims=4),
    "attention": dict(layer_types=("attention",), scale=2.0),
    "attention_plain_rotation": dict(layer_types=("attention",), scaling=None, rot_dims=16),
    "attention_shared": dict(layer_types=("attention", "attention"), share_from={1: 0}),
    "no_feed_forward": dict(layer_types=("retention",), no_mlp=[0]),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", list(ALONE))
def test_each_mechanism_alone(which, dtype, tmp_path):
    cfg = with_max_positions(pv.random_config(np.random.default_rng(1), **ALONE[which]), 256)
    w = write_model(str(tmp_path), cfg, 3)
    ids = prompt(cfg, 150, 5)
    ref = pv.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype, max_seq_len=256)
    assert_close(whole(eng, ids), ref, dtype, which)


@pytest.mark.parametrize("dtype", DTYPES)
def test_second_norm_of_a_layer_without_feed_forward(dtype, tmp_path):
    """A weight file may hold a second norm for a layer that has no feed-forward: it then norms the scaled
    stream alone.  (Without the tensor the layer ends after its first norm: `no_feed_forward` above.)"""
    cfg = with_max_positions(pv.random_config(np.random.default_rng(1), ("lightning", "attention"), no_mlp=[0, 1]), 256)
    w = write_model(str(tmp_path), cfg, 3, norm2_always=True)
    assert "l0.norm2" in w
    ids = prompt(cfg, 70, 5)
    eng = engine(str(tmp_path), dtype, max_seq_len=256)
    assert_close(in_portions(eng, ids, [66, 1]), pv.forward(cfg, w, ids), dtype, "second norm without feed-forward")


# ------------------------------------------------------------------ whole models, every way of cutting


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_and_token_by_token(name, dtype, models):
    d, cfg, w = models[name]
    eng = engine(d, dtype)
    for n, seed in ((1, 1), (2, 2), (3, 3), (130, 4)):       # the first tokens of a sequence, and past two page borders
        ids = prompt(cfg, n, seed)
        ref = pv.forward(cfg, w, ids)
        a = whole(eng, ids)
        assert_close(a, ref, dtype, f"{name} whole {n}")
        b = in_portions(eng, ids, [1])
        assert_close(b, ref, dtype, f"{name} token by token {n}")
        same_or_close(a, b, dtype, f"{name} {n}: whole against token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "other"])
def test_portions(name, dtype, models):
    d, cfg, w = models[name]
    eng = engine(d, dtype)
    ids = prompt(cfg, 200, 11)
    ref = pv.forward(cfg, w, ids)
    a = whole(eng, ids)
    for sizes in ([2], [3, 5, 7], [16, 17], [63, 1, 1, 64], [64], [65, 2], [128, 1], [100, 2, 2, 2, 94]):
        b = in_portions(eng, ids, sizes)
        assert_close(b, ref, dtype, f"{name} portions {sizes}")
        same_or_close(a, b, dtype, f"{name} portions {sizes} against whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, models):
    d, cfg, w = models["wide"]
    eng = engine(d, dtype, max_seq_len=1024)
    ids = prompt(cfg, 40 + 300, 21)
    ref = pv.forward(cfg, w, ids)
    got = in_portions(eng, ids, [40, 1])        # 300 single-token steps, replayed from a captured graph
    assert_close(got, ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "other", "wide", "wide128"])
def test_batches_of_unequal_requests_and_reuse(name, dtype, models):
    """Prompts of unequal lengths in one step, decoded together until each runs out; two batches one
    after the other on a cache that only holds one of them, freed pages poisoned: slots, pages and
    state of the first batch are used again by the second.  Each request equals itself alone."""
    d, cfg, w = models[name]
    lens = [(1, 40), (65, 33), (129, 20), (30, 70), (64, 5), (2, 64)]       # (prompt tokens, tokens decoded one by one)
    reqs = [prompt(cfg, a + b, 30 + i) for i, (a, b) in enumerate(lens)]
    eng = engine(d, dtype, max_tokens=512, poison=True, max_batch=3)
    alone = engine(d, dtype, max_tokens=512)
    got = {}
    for batch in ([0, 1, 2], [3, 4, 5]):
        slots = {r: eng.new_sequence() for r in batch}
        lg = eng.step([StepItem(slots[r], reqs[r][:lens[r][0]], list(range(lens[r][0]))) for r in batch]).cpu().numpy()
        off = 0
        for r in batch:
            got[r] = [lg[off:off + lens[r][0]]]
            off += lens[r][0]
        pos = {r: lens[r][0] for r in batch}
        live = list(batch)
        while live:
            lg = eng.step([StepItem(slots[r], [reqs[r][pos[r]]], [0]) for r in live]).cpu().numpy()
            nxt = []
            for i, r in enumerate(live):
                got[r].append(lg[i:i + 1])
                pos[r] += 1
                if pos[r] < len(reqs[r]):
                    nxt.append(r)
                else:
                    eng.end_sequence(slots[r])
            live = nxt
    eng.check_device_errors()
    for r, ids in enumerate(reqs):
        g = np.concatenate(got[r])
        assert_close(g, pv.forward(cfg, w, ids), dtype, f"{name} request {r} in a batch")
        same_or_close(in_portions(alone, ids, [lens[r][0], 1]), g, dtype, f"{name} request {r}: alone against in a batch")


# ------------------------------------------------------------------ faults that random weights would hide


def test_one_far_key_and_the_sink_decide(tmp_path):
    """One attention layer whose queries all point at one early token: the embedding of a marker token
    is large along one direction, the key projection maps that direction to a key that every query
    likes, and its value is large.  The marker stands at chosen places (first token, ends and starts
    of pages, far back), in prompts and with the tail decoded token by token.  A key that is skipped,
    read twice or taken from the wrong page changes the logits by far more than the tolerance; so does
    a sink that is left out, since the sinks are about as large as the marker's score."""
    rng = np.random.default_rng(9)
    cfg = with_max_positions(pv.random_config(rng, ("attention",), heads=2, kv_heads=1, dim=16, vdim=16, rot_dims=4, scale=1.0), 512)
    d = str(tmp_path)
    w = write_model(d, cfg, 13, sink_scale=0.0)
    # rewrite the file with crafted tensors
    D = cfg["width"]
    embed = w["embed"].copy()
    embed[0] = 0.0
    embed[0, 0] = 30.0                                   # the marker token 0
    w["embed"] = embed
    wk = w["l0.mix.k"].copy()
    wk[:, 0] = 0.0
    wk[12, 0] = 1.0                                      # marker -> key along channel 12 (not rotated)
    w["l0.mix.k"] = wk
    w["l0.mix.q.b"] = np.zeros_like(w["l0.mix.q.b"])
    w["l0.mix.q.b"][12] = 40.0                           # every query of head 0 looks along channel 12
    w["l0.mix.q.b"][16 + 12] = 40.0                      # and of head 1
    w["l0.mix.sink"] = np.array([15.0, 17.0])
    _rewrite(d, cfg, w)
    w = _reload(d, cfg)
    eng32, eng16 = engine(d, "float32"), engine(d, "bfloat16")
    for place, n in ((0, 70), (63, 140), (64, 140), (127, 200), (128, 200), (5, 300)):
        ids = np.random.default_rng(place).integers(1, cfg["vocab"], n)
        ids[place] = 0
        ids = ids.tolist()
        ref = pv.forward(cfg, w, ids)
        # the check has teeth: without the marker's key the logits are far away
        ids2 = list(ids)
        ids2[place] = 1
        assert rel_err(pv.forward(cfg, w, ids2)[place + 1:], ref[place + 1:]) > 0.05
        for eng, dtype in ((eng32, "float32"), (eng16, "bfloat16")):
            assert_close(whole(eng, ids), ref, dtype, f"marker at {place}, whole")
            assert_close(in_portions(eng, ids, [n - 40, 1]), ref, dtype, f"marker at {place}, tail decoded")
            assert_close(in_portions(eng, ids, [place + 1, 2]), ref, dtype, f"marker at {place}, cut right behind it")


def _rewrite(folder, cfg, w):
    blobs, header, off = [], {}, 0
    for name, shape in pv.tensor_shapes(cfg).items():
        bits = to_bf16_bits(w[name])
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + bits.nbytes]}
        blobs.append(bits.tobytes())
        off += bits.nbytes
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def _reload(folder, cfg):
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, rec in header.items():
        a, b = rec["data_offsets"]
        bits = np.frombuffer(data[a:b], dtype=np.uint16)
        out[name] = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64).reshape(rec["shape"])
    return out


def test_state_far_back_survives(tmp_path):
    """One linear-attention layer with decays 1 - 2^-10 and 0.5: what the first tokens wrote into the
    state still decides the output hundreds of tokens later for the slow head and not at all for the
    fast one; the state is carried through steps of every size."""
    rng = np.random.default_rng(2)
    for kind in ("lightning", "retention"):
        cfg = with_max_positions(pv.random_config(rng, (kind,), lin_heads=2, decay=[1.0 - 2.0 ** -10, 0.5], lin_dim=8, lin_vdim=16), 1024)
        d = os.path.join(str(tmp_path), kind)
        w = write_model(d, cfg, 17)
        ids = prompt(cfg, 600, 3)
        ref = pv.forward(cfg, w, ids)
        other = list(ids)
        other[:8] = prompt(cfg, 8, 4)
        assert rel_err(pv.forward(cfg, w, other)[-50:], ref[-50:]) > 1e-3        # the first tokens matter at the end
        for dtype in DTYPES:
            eng = engine(d, dtype, max_seq_len=1024, max_tokens=2048)
            assert_close(whole(eng, ids), ref, dtype, f"{kind} whole")
            assert_close(in_portions(eng, ids, [500, 2, 1]), ref, dtype, f"{kind} portions")


def test_long_prompts_in_segments(tmp_path):
    """In the bfloat16 mode a long prompt's recurrence is cut into segments that run side by side and are
    joined afterwards (the float32 mode keeps the order, bit for bit).  Prompts whose lengths leave the
    last segment short, fill only some segments, or are a single token, together in one step; then each
    goes on token by token from the state the joined segments left."""
    rng = np.random.default_rng(4)
    cfg = with_max_positions(pv.random_config(rng, ("retention", "lightning"), lin_heads=2, decay=[0.98, 0.75], lin_dim=16, lin_vdim=24,
                                              ret_rot_dims=8), 2048)
    d = str(tmp_path)
    w = write_model(d, cfg, 23)
    lens = [1500, 1, 257, 1024, 130]
    reqs = [prompt(cfg, n + 5, 70 + i) for i, n in enumerate(lens)]
    refs = [pv.forward(cfg, w, ids) for ids in reqs]
    for dtype in DTYPES:
        eng = engine(d, dtype, max_tokens=4096, max_seq_len=2048)
        slots = [eng.new_sequence() for _ in reqs]
        lg = eng.step([StepItem(s, ids[:n], list(range(n))) for s, ids, n in zip(slots, reqs, lens)]).cpu().numpy()
        off = 0
        for ids, n, ref in zip(reqs, lens, refs):
            assert_close(lg[off:off + n], ref[:n], dtype, f"prompt of {n} tokens among others")
            off += n
        for k in range(5):
            lg = eng.step([StepItem(s, [ids[n + k]], [0]) for s, ids, n in zip(slots, reqs, lens)]).cpu().numpy()
            for i, (n, ref) in enumerate(zip(lens, refs)):
                assert_close(lg[i:i + 1], ref[n + k:n + k + 1], dtype, f"token {k} behind a prompt of {n}")
        eng.check_device_errors()


# ------------------------------------------------------------------ the library's own entry point


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_greedy_generation_through_the_model_api(name, models):
    d, cfg, w = models[name]
    prompts = [prompt(cfg, n, 50 + n) for n in (3, 17, 70)]
    want = [pv.greedy_generate(cfg, w, p, 12) for p in prompts]
    m = Model(ModelConfig(compt_type="float32", nr_ctx=256, max_tokens=1024))
    m.load(d)
    m.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    got = m.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens
    assert got == want
    m16 = Model(ModelConfig(compt_type="bfloat16", nr_ctx=256, max_tokens=1024))
    m16.load(d)
    m16.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    got16 = m16.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens
    assert [g[0] for g in got16] == [x[0] for x in want]        # later tokens may turn at a near-tie in bfloat16


def test_command_line(models):
    """bin/llama on a Vokelix folder: greedy tokens of two requests, float32."""
    d, cfg, w = models["other"]
    prompts = [prompt(cfg, n, 80 + n) for n in (4, 21)]
    want = [pv.greedy_generate(cfg, w, p, 6) for p in prompts]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = [os.path.join(root, "bin", "llama"), "-m", d, "-d", "float32", "-c", "128", "-n", "6", "--temp", "0", "--top_k", "0",
            "--top_p", "1", "--repeat_penalty", "1", "-s", "1"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in ln.split(": ")[1].split(",")] for ln in r.stdout.splitlines() if ln.startswith("[")]
    assert got == want
    r = subprocess.run(args[:3] + ["--random-prompts", "5,9", "-n", "3", "-c", "64"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr        # the vocabulary size comes from the model's spec, whatever its key is called

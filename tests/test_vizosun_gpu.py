"""The Vizosun decoder in the engine against the plain implementation (tests/plain_vizosun.py), GPU.

Every test makes its own small configuration and its own weights (numpy, rounded to bfloat16 so that the
float32 mode, the bfloat16 mode and the plain implementation see the same numbers).  Weights are drawn so
that faults show: the attention scale is large (a peaked softmax: a missed or doubled key changes the
result), decay rates include values close to zero (a token far back still counts), and the routers' logits
are spread (a wrong expert changes the row).
"""
import json
import os

import numpy as np
import pytest
import plain_vizosun as pz
from util import BF16_TOL, assert_close, rel_err

from inferllm_b200 import Engine, EngineOptions, Model, ModelConfig, StepItem

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def write_model(folder, cfg, seed, edit=None, gain=0.5):
    """config.json + model.safetensors (bfloat16) with random weights; returns the weights.  `gain` scales the
    matrices: with larger ones a stack of layers amplifies rounding until bfloat16 decides the result."""
    w = pz.random_weights(cfg, seed, gain)
    for name in w:
        if name.endswith("router"):
            w[name] = pz.bf16_round(w[name] * 6.0 / gain)   # spread logits: the choice of experts is clear
        if name.endswith("A_log"):
            w[name] = pz.bf16_round(np.linspace(-6.0, 0.5, w[name].size).astype(np.float32))     # slow and fast heads
    if edit:
        edit(w)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    pz.write_safetensors(os.path.join(folder, "model.safetensors"), w)
    return w


def engine(folder, dtype, max_tokens=2048, page_size=64, max_seq_len=1024, poison=False, max_batch=None):
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


def close(got, ref, dtype, what):
    """float32: every position within the bound.  bfloat16: a router whose two best logits lie closer together than
    the rounding of its input may choose the other expert, which changes that token's row (and, less, the rows after
    it) by more than rounding: at most one position in fifty (or one) may exceed the bound, none five times the
    bound, and the others are held to it."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    if dtype == "float32" or got.ndim < 2:
        return assert_close(got, ref, dtype, what)
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    err = np.abs(got - ref).max(-1) / max(np.abs(ref).max(), 1e-30)
    over = err > BF16_TOL
    assert over.sum() <= max(1, len(err) // 50), f"{what}: {int(over.sum())} of {len(err)} positions exceed {BF16_TOL:.1e} (worst {err.max():.3e})"
    assert err.max() <= 5 * BF16_TOL, f"{what}: a position is off by {err.max():.3e}"
    if (~over).any():
        assert_close(got[~over], ref[~over], dtype, what)


def same_or_close(a, b, dtype, what):
    """float32: every kernel fixes the order of its sums per row, so two ways of cutting the same tokens give
    the same bits; bfloat16: the library's products choose kernels by shape."""
    if dtype == "float32":
        assert np.array_equal(a, b), f"{what}: float32 logits differ between two cuttings (max {np.abs(a - b).max():.3e})"
    else:
        close(a, b, dtype, what)


D, L = "channel_delta", "latent_attention"
CONFIGS = {
    # both mixers, both feed-forwards, a loop over two layers, the bigram table, a window shorter than a page
    "mixed": pz.random_config((D, L, D, L), loop=(1, 3, 2), scale=1.5),
    # no loop, no bigram table, no window, one q/k head per value head, one tap, one expert per token, a layer
    # without a feed-forward, odd sizes
    "other": pz.random_config((L, D, D), width=40, vocab=61, heads=3, kv_heads=3, dim=24, vdim=10, conv=1, a_rank=5, g_rank=3, att_heads=5,
                              att_dim=8, att_vdim=16, q_rank=16, kv_rank=24, window=0, scale=2.0, experts=3, top=1, expert_ff=20, ff=36,
                              mlps=["moe", None, "dense"], bigram=None, eps=1e-6),
    # latents of the sizes the tensor-core attention kernels take, a loop that starts at the first layer and runs three
    # times, windows across pages, key heads of 64 channels spread over two lanes
    "wide": pz.random_config((L, D, L), width=64, vocab=128, heads=2, kv_heads=1, dim=64, vdim=40, conv=4, a_rank=16, g_rank=8, att_heads=4,
                             att_dim=32, att_vdim=32, q_rank=40, kv_rank=64, window=70, scale=0.7, experts=8, top=3, expert_ff=32, ff=96,
                             mlps=["dense", "moe", "moe"], loop=(0, 2, 3), bigram=(1021, 5, 3)),
    # a latent of 128 channels with many heads, key heads of 128 channels over four lanes, all experts chosen
    "wide128": pz.random_config((D, L), width=96, vocab=150, heads=2, kv_heads=2, dim=128, vdim=16, conv=2, a_rank=8, g_rank=8, att_heads=20,
                                att_dim=16, att_vdim=8, q_rank=32, kv_rank=128, window=130, scale=0.9, experts=2, top=2, expert_ff=48, ff=80,
                                mlps=["moe", "dense"]),
    # sizes that are multiples of nothing much: low ranks of 3 and 5, a query latent of 12, a key/value latent of 40, every
    # expert chosen, a loop over all layers
    "odd": pz.random_config((D, L, D), width=56, vocab=75, heads=3, kv_heads=1, dim=20, vdim=12, conv=2, a_rank=3, g_rank=5, att_heads=7,
                            att_dim=12, att_vdim=20, q_rank=12, kv_rank=40, window=33, scale=0.8, experts=4, top=4, expert_ff=12, ff=44,
                            mlps=["moe", "dense", "moe"], loop=(0, 3, 2), bigram=(7, 3, 1)),
    # an odd width and an odd vocabulary: no row of an activation or a matrix is a whole number of 16-byte pieces
    "odd_width": pz.random_config((D, L, L), width=45, vocab=71, heads=3, kv_heads=3, dim=10, vdim=6, conv=3, a_rank=2, g_rank=2, att_heads=3,
                                  att_dim=6, att_vdim=10, q_rank=9, kv_rank=24, window=11, scale=0.9, experts=3, top=2, expert_ff=10, ff=30,
                                  mlps=["moe", "dense", None], loop=(1, 2, 2), bigram=(13, 5, 3)),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("vz_" + name))
        out[name] = (d, cfg, write_model(d, cfg, 7 + i))
    return out


def prompt(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


# ------------------------------------------------------------------ each mechanism alone

ALONE = {
    "delta": pz.random_config((D,), mlps=[None], bigram=None),
    "delta_grouped_taps": pz.random_config((D,), mlps=[None], bigram=None, heads=6, kv_heads=2, dim=8, vdim=12, conv=5),
    "latent": pz.random_config((L,), mlps=[None], bigram=None, window=0, scale=2.0),
    "latent_window": pz.random_config((L,), mlps=[None], bigram=None, window=5, scale=2.0),
    "dense": pz.random_config((L,), mlps=["dense"], bigram=None),
    "moe": pz.random_config((L,), mlps=["moe"], bigram=None, experts=7, top=3),
    "latent_odd_width": pz.random_config((L,), mlps=[None], bigram=None, window=9, scale=1.5, kv_rank=21, q_rank=7, att_heads=3),
    "latent_wide": pz.random_config((L,), mlps=[None], bigram=None, window=0, scale=0.4, kv_rank=264, att_heads=2),
    "bigram": pz.random_config((L,), mlps=[None], bigram=(17, 1000003, 999983)),
    "loop": pz.random_config((L, L), mlps=[None, None], bigram=None, loop=(0, 1, 3)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_mechanism_alone(tmp_path, name, dtype):
    cfg = ALONE[name]
    w = write_model(str(tmp_path), cfg, 3)
    ids = prompt(cfg, 41, 5)
    ref, layers = pz.forward(cfg, w, ids, return_layers=True)
    eng = engine(str(tmp_path), dtype)
    assert_close(whole(eng, ids), ref, dtype, name)
    # and token by token through the cache and the state
    assert_close(in_portions(eng, ids, [1]), ref, dtype, name + " token by token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_through_the_fused_products(tmp_path, dtype):
    """A prompt long enough, and a feed-forward wide enough, for the product kernels whose epilogue is the gate's
    activation (relu here), and for the experts' products on row tiles of 128."""
    cfg = pz.random_config((L, L), mlps=["dense", "moe"], bigram=None, width=64, ff=256, expert_ff=64, experts=4, top=2, window=50,
                           att_heads=2, att_dim=16, att_vdim=16, q_rank=16, kv_rank=64)
    w = write_model(str(tmp_path), cfg, 21)
    ids = prompt(cfg, 600, 8)
    ref = pz.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype, max_tokens=2048)
    got = whole(eng, ids)
    close(got, ref, dtype, "600 tokens in one step")
    same_or_close(in_portions(eng, ids, [520, 1]), got, dtype, "the same, its last tokens one by one")


# ------------------------------------------------------------------ whole models


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt(models, name, dtype):
    d, cfg, w = models[name]
    ids = prompt(cfg, 150, 11)
    close(whole(engine(d, dtype), ids), pz.forward(cfg, w, ids), dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_first_tokens_and_one_token(models, name, dtype):
    d, cfg, w = models[name]
    eng = engine(d, dtype)
    for n in (1, 2, 3):
        ids = prompt(cfg, n, 20 + n)
        assert_close(whole(eng, ids), pz.forward(cfg, w, ids), dtype, f"{name} {n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_and_decoding(models, name, dtype):
    """Prefill against token-by-token decoding and portions of several sizes, down to two tokens, across page borders
    and window edges."""
    d, cfg, w = models[name]
    ids = prompt(cfg, 200, 13)
    ref = pz.forward(cfg, w, ids)
    eng = engine(d, dtype)
    base = whole(eng, ids)
    close(base, ref, dtype, name)
    for sizes in ([1], [2], [63, 2, 64, 7], [128, 1], [5, 64, 3]):
        got = in_portions(eng, ids, sizes)
        close(got, ref, dtype, f"{name} portions {sizes}")
        same_or_close(got, base, dtype, f"{name} portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_unequal_batches(models, name, dtype):
    """Requests of different lengths in one batch, then decoded together while the shorter ones end, against each alone."""
    d, cfg, w = models[name]
    eng = engine(d, dtype, max_tokens=4096)
    lens, extra = [1, 37, 150, 66], [9, 30, 12, 5]
    seqs = [prompt(cfg, n + e, 40 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    refs = [pz.forward(cfg, w, s) for s in seqs]
    alone = [whole(eng, s) for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    lg = eng.step([StepItem(slots[i], seqs[i][:lens[i]], list(range(lens[i]))) for i in range(len(seqs))]).cpu().numpy()
    at, got = 0, []
    for i, n in enumerate(lens):
        got.append([lg[at:at + n]])
        at += n
    pos = list(lens)
    live = list(range(len(seqs)))
    while live:
        lg = eng.step([StepItem(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(lg[r:r + 1])
            pos[i] += 1
        for i in list(live):
            if pos[i] == len(seqs[i]):
                eng.end_sequence(slots[i])
                live.remove(i)
    for i in range(len(seqs)):
        g = np.concatenate(got[i])
        close(g, refs[i], dtype, f"{name} batch, sequence {i}")
        same_or_close(g, alone[i], dtype, f"{name} batch, sequence {i} against itself alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(models, dtype):
    """A small cache whose slots, pages and state rows go round several times, freed pages poisoned with NaN."""
    d, cfg, w = models["mixed"]
    eng = engine(d, dtype, max_tokens=320, max_batch=3, max_seq_len=256, poison=True)
    for rnd in range(4):
        seqs = [prompt(cfg, n, 70 + 10 * rnd + i) for i, n in enumerate((90 + rnd, 33, 70))]
        slots = [eng.new_sequence() for _ in seqs]
        cut = [len(s) // 2 + rnd for s in seqs]
        eng.step([StepItem(slots[i], seqs[i][:cut[i]], []) for i in range(3)])
        eng.end_sequence(slots[1])                        # its slot and pages go to the next sequence at once
        late = prompt(cfg, 40, 90 + rnd)
        s_late = eng.new_sequence()
        got_late = eng.step([StepItem(s_late, late, list(range(40)))]).cpu().numpy()
        close(got_late, pz.forward(cfg, w, late), dtype, f"round {rnd}: a sequence in a slot used before")
        for i in (0, 2):
            rest = seqs[i][cut[i]:]
            got = eng.step([StepItem(slots[i], rest, list(range(len(rest))))]).cpu().numpy()
            close(got, pz.forward(cfg, w, seqs[i])[cut[i]:], dtype, f"round {rnd}: sequence {i} continued")
            eng.end_sequence(slots[i])
        eng.end_sequence(s_late)


# ------------------------------------------------------------------ crafted cases


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 64, 65, 7])
def test_one_key_decides(tmp_path, window, dtype):
    """One far position's latent is made to dominate the scores of every later query (its token's embedding is scaled
    up and the scale is large), so whether exactly that key is seen decides the output: just inside and just outside
    the window, at a page border, in a prompt and in decoding."""
    cfg = pz.random_config((L,), mlps=[None], bigram=None, window=window, scale=4.0, vocab=50)
    far = 63                                             # the last row of the first page
    ids = prompt(cfg, 140, 3)
    ids = [t if t != 7 else 8 for t in ids]
    ids[far] = 7                                         # token 7 appears once

    def edit(w):
        w["embed"][7] = pz.bf16_round(w["embed"][7] * 3.0)

    w = write_model(str(tmp_path), cfg, 9, edit)
    ref = pz.forward(cfg, w, ids)
    eng = engine(str(tmp_path), dtype)
    assert_close(whole(eng, ids), ref, dtype, f"window {window}, prompt")
    assert_close(in_portions(eng, ids, [60, 1]), ref, dtype, f"window {window}, decoding past the key")
    assert_close(in_portions(eng, ids, [far + 1, 2]), ref, dtype, f"window {window}, portions from the key on")


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_far_back(tmp_path, dtype):
    """Decay rates near zero: what the first tokens wrote is still in the state hundreds of tokens later, through a
    prompt and through long decoding."""
    cfg = pz.random_config((D, D), mlps=[None, "dense"], bigram=(31, 3, 5), heads=2, kv_heads=1, dim=32, vdim=16)

    def edit(w):
        for name in w:
            if name.endswith("A_log"):
                w[name] = pz.bf16_round(np.full(w[name].shape, -9.0, np.float32))

    w = write_model(str(tmp_path), cfg, 4, edit)
    ids = prompt(cfg, 420, 6)
    ref = pz.forward(cfg, w, ids)
    # the oracle itself depends on the first tokens at the end: the test would not see a lost state otherwise
    other = pz.forward(cfg, w, prompt(cfg, 20, 99) + ids[20:])
    assert rel_err(other[-1], ref[-1]) > 1e-3
    eng = engine(str(tmp_path), dtype)
    assert_close(whole(eng, ids), ref, dtype, "prompt")
    assert_close(in_portions(eng, ids, [100, 1]), ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_rank_from_the_file(tmp_path, dtype):
    """A configuration that does not name the low ranks of the decay and gate projections takes them from the file."""
    cfg = pz.random_config((D,), mlps=["moe"], a_rank=6, g_rank=10)
    w = write_model(str(tmp_path), cfg, 12)
    for layer in cfg["layers"]:
        del layer["mixer"]["a_rank"], layer["mixer"]["g_rank"]
    with open(os.path.join(str(tmp_path), "config.json"), "w") as f:
        json.dump(cfg, f)
    ids = prompt(cfg, 30, 1)
    full = json.loads(json.dumps(cfg))
    assert_close(whole(engine(str(tmp_path), dtype), ids), pz.forward(full, w, ids), dtype, "ranks from the file")


# ------------------------------------------------------------------ generation


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation(models, dtype):
    """Greedy tokens through Model.generate (the scheduler, batches, the sampler) against the plain implementation."""
    d, cfg, w = models["mixed"]
    prompts = [prompt(cfg, n, 50 + n) for n in (3, 17, 70, 1)]
    m = Model(ModelConfig(compt_type=dtype, nr_ctx=256, max_tokens=1024))
    m.load(d)
    m.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    got = m.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens
    want = [pz.greedy_generate(cfg, w, p, 12) for p in prompts]
    if dtype == "float32":
        assert got == want
        return
    # bfloat16 may turn a near-tie: every token the engine chose must be (within rounding) the best continuation of what
    # it had generated so far, by the plain implementation's logits for that very sequence
    for p, g in zip(prompts, got):
        assert len(g) == 12
        lg = pz.forward(cfg, w, p + g)[len(p) - 1:-1]
        gap = lg.max(-1) - lg[np.arange(12), g]
        assert (gap <= BF16_TOL * np.abs(lg).max()).all(), (g, gap)


def test_trace_replay_program(models, tmp_path):
    """bin/trace_run on a Vizosun folder: portions, a batch, ends, and the logits files."""
    import subprocess
    d, cfg, w = models["other"]
    a, b = prompt(cfg, 9, 1), prompt(cfg, 5, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:6], "want": [0, 5]}, {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[6:7], "want": [0]}, {"id": "b", "tokens": b[4:5], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[7:], "want": [1]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    ra, rb = pz.forward(cfg, w, a), pz.forward(cfg, w, b)
    want = [np.stack([ra[0], ra[5], rb[3]]), np.stack([ra[6], rb[4]]), np.stack([ra[8]])]
    for n, ref in enumerate(want):
        got = np.fromfile(os.path.join(out, f"{n}.f32"), "<f4").reshape(ref.shape)
        assert_close(got, ref, "float32", f"step {n}")


def test_command_line(models):
    """bin/llama on a Vizosun folder: greedy tokens of two requests, float32."""
    import subprocess
    d, cfg, w = models["mixed"]
    prompts = [prompt(cfg, n, 90 + n) for n in (7, 12)]
    want = [pz.greedy_generate(cfg, w, p, 6) for p in prompts]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = [os.path.join(root, "bin", "llama"), "-m", d, "-d", "float32", "-c", "128", "-n", "6", "--temp", "0", "--top_k", "0",
            "--top_p", "1", "--repeat_penalty", "1", "-s", "1"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in ln.split(": ")[1].split(",")] for ln in r.stdout.splitlines() if ln.startswith("[")]
    assert got == want

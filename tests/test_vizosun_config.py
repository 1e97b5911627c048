"""The Vizosun configuration class and the plain implementation's own pieces, on the CPU.

What config.json says must arrive in the ModelSpec unchanged (sizes, constants, layer order, the passes of a
loop and their cache entries), the tensors the model declares must be the file's names and shapes, and a
configuration that cannot be built is refused in words.  The plain implementation's mechanisms are checked
against second, independent formulations of the same equations.
"""
import numpy as np
import pytest
import plain_vizosun as pz

from inferllm_b200 import ConfigError, VizosunConfig, config_from_dict
from inferllm_b200.weights import tensor_decls

D, L = "channel_delta", "latent_attention"


def test_spec_carries_every_size_and_constant():
    cfg = pz.random_config((D, L, L, D), width=56, vocab=77, heads=6, kv_heads=3, dim=12, vdim=20, conv=5, a_rank=7, g_rank=9, att_heads=5,
                           att_dim=10, att_vdim=14, q_rank=18, kv_rank=40, window=33, scale=0.37, experts=6, top=3, expert_ff=22, ff=72,
                           mlps=["moe", "dense", None, "moe"], loop=(1, 3, 3), bigram=(101, 13, 29), eps=2e-5)
    spec = config_from_dict(cfg).model_spec()
    assert (spec.hidden_size, spec.vocab_size) == (56, 77)
    # layers 1 and 2 run three times in a row, every pass with cache entries of its own, entered through the re-entry map
    assert [(e.layer, e.cache, e.writes, e.reenter) for e in spec.schedule] == [
        (0, 0, True, False), (1, 1, True, True), (2, 2, True, False), (1, 3, True, True), (2, 4, True, False), (1, 5, True, True),
        (2, 6, True, False), (3, 7, True, False)]
    assert spec.reentry.kind == "linear" and (spec.reentry["in_size"], spec.reentry["out_size"]) == (112, 56)
    d, a = spec.layers[0].mixer, spec.layers[1].mixer
    assert d.kind == "channel_delta" and a.kind == "latent_attention"
    assert (d["n_heads"], d["n_kv_heads"], d["head_dim"], d["v_head_dim"], d["conv"], d["a_rank"], d["g_rank"]) == (6, 3, 12, 20, 5, 7, 9)
    assert d["q_scale"] == pytest.approx(12 ** -0.5) and d["norm_eps"] == 2e-5
    assert (a["n_heads"], a["head_dim"], a["v_head_dim"], a["q_rank"], a["kv_rank"], a["window"], a["scale"]) == (5, 10, 14, 18, 40, 33, 0.37)
    assert [l.block for l in spec.layers] == ["parallel"] * 4
    assert [l.ffn.kind for l in spec.layers] == ["routed_mlp", "gated_mlp", "", "routed_mlp"]
    moe, dense = spec.layers[0].ffn, spec.layers[1].ffn
    assert (moe["experts"], moe["top"], moe["intermediate_size"], moe["activation"]) == (6, 3, 22, "silu")
    assert (dense["intermediate_size"], dense["activation"]) == (72, "relu")
    e = spec.embedding
    assert e.kind == "bigram_embedding" and (e["buckets"], e["mul_prev"], e["mul_cur"]) == (101, 13, 29)
    assert spec.head["tied"] is True
    for l in spec.layers:
        assert l.norms["norm1"]["eps"] == 2e-5 and list(l.norms) == ["norm1"]


def test_without_loop_and_bigram_nothing_of_them_exists():
    cfg = pz.random_config((L, D), bigram=None, window=0)
    spec = config_from_dict(cfg).model_spec()
    assert spec.reentry is None and not any(e.reenter for e in spec.schedule)
    assert spec.embedding.kind == "embedding"
    assert spec.layers[0].mixer["window"] == 0
    names = set(tensor_decls(config_from_dict(cfg)))
    assert "bigram" not in names and "loop.in" not in names


def test_the_python_face_is_typed_and_round_trips():
    cfg = pz.random_config((D, L), width=40)
    c = config_from_dict(cfg)
    assert isinstance(c, VizosunConfig) and c.architecture == "Vizosun"
    assert (c.width, c.vocab) == (40, cfg["vocab"]) and len(c.layers) == 2
    assert VizosunConfig.from_dict(c.to_dict()) == c


def test_declared_tensors_are_the_files_names_and_shapes():
    cfg = pz.random_config((D, L, D, L), loop=(1, 3, 2), mlps=["dense", "moe", None, "moe"], heads=6, kv_heads=2)
    decls = {name: tuple(shape) for name, (shape, _) in tensor_decls(config_from_dict(cfg)).items()}
    assert decls == {k: tuple(v[0]) for k, v in pz.tensor_shapes(cfg).items()}
    # ranks that the configuration does not name are whatever the file has
    for layer in cfg["layers"]:
        layer["mixer"].pop("a_rank", None)
        layer["mixer"].pop("g_rank", None)
    decls = {name: tuple(shape) for name, (shape, _) in tensor_decls(config_from_dict(cfg)).items()}
    assert decls["l0.mix.a1"] == (-1, cfg["width"]) and decls["l0.mix.g2"][1] == -1


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda c: c.__setitem__("loop", {"start": 1, "stop": 1, "times": 2}), "loop"),
    (lambda c: c.__setitem__("loop", {"start": 0, "stop": 5, "times": 2}), "loop"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "mlp.kind"),
    (lambda c: c["embedding"]["bigram"].__setitem__("buckets", 0), "buckets"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
])
def test_refusals_are_in_words(edit, word):
    cfg = pz.random_config((D, L))
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_keys_only_cache_entries_form_a_group_of_their_own():
    from inferllm_b200.cache import FixedState, PagedKV, SequenceCache
    c = SequenceCache({0: PagedKV(1, 40, window=33, keys_only=True), 1: PagedKV(1, 40, window=33), 2: PagedKV(1, 40, window=33, keys_only=True),
                       -1: FixedState((1,), "int32")}, 2, 8, 16, 64)
    st = c.stats()
    assert [g["entries"] for g in st["paged"]] == [[0, 2], [1]]
    assert st["paged"][0]["request"].get("keys_only") is True and "keys_only" not in st["paged"][1]["request"]
    assert st["states"][0]["entries"] == [-1] and st["states"][0]["request"]["dtype"] == "int32"


# ------------------------------------------------------------------ the plain implementation against second formulations


def test_bigram_rows():
    assert pz.bigram_rows([5, 9, 9, 0], 11, 7, 3) == [11, (5 * 7 + 9 * 3) % 11, (9 * 7 + 9 * 3) % 11, (9 * 7) % 11]


def test_causal_conv_is_a_correlation_with_zeros_in_front():
    rng = np.random.default_rng(0)
    x, taps = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y = pz.causal_conv(x, taps)
    for c in range(3):
        padded = np.concatenate([np.zeros(3), x[:, c]])
        assert np.allclose(y[:, c], np.correlate(padded, taps[c], "valid"))


def test_delta_recurrence_against_the_expanded_update():
    """S_t = (diag(g) S_{t-1}) (as a matrix acting on columns) - beta k (k^T diag(g) S_{t-1}) + beta k v^T."""
    rng = np.random.default_rng(1)
    T, H, d, dv = 7, 2, 5, 3
    q, k, g = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, d)), rng.uniform(0.5, 1.0, (T, H, d))
    v, beta = rng.standard_normal((T, H, dv)), rng.uniform(0, 1, (T, H))
    o = pz.delta_recurrence(q, k, v, g, beta)
    for h in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            A = (np.eye(d) - beta[t, h] * np.outer(k[t, h], k[t, h])) @ np.diag(g[t, h])
            S = A @ S + beta[t, h] * np.outer(k[t, h], v[t, h])
            assert np.allclose(o[t, h], q[t, h] @ S)


def test_window_attention_against_a_masked_matrix():
    rng = np.random.default_rng(2)
    T, H, d, dv, win = 12, 2, 4, 3, 5
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, d)), rng.standard_normal((T, H, dv))
    o = pz.window_softmax_attention(q, k, v, 0.7, win)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    mask = (i - j >= 0) & (i - j < win)
    for h in range(H):
        s = np.where(mask, (q[:, h] @ k[:, h].T) * 0.7, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        assert np.allclose(o[:, h], (p / p.sum(-1, keepdims=True)) @ v[:, h])
    # the last row sees exactly `win` keys: moving the key just outside changes nothing, the one just inside does
    k2 = k.copy()
    k2[T - 1 - win] += 5.0
    assert np.allclose(pz.window_softmax_attention(q, k2, v, 0.7, win)[-1], o[-1])
    k2 = k.copy()
    k2[T - win] += 5.0
    assert not np.allclose(pz.window_softmax_attention(q, k2, v, 0.7, win)[-1], o[-1])


def test_latent_attention_against_the_absorbed_form():
    """score = (U_k^T q) . c and o = U_v (sum p c): the form a cache of latents alone allows."""
    cfg = pz.random_config((L,), mlps=[None], window=4)
    m = cfg["layers"][0]["mixer"]
    w = pz.random_weights(cfg, 0)
    rng = np.random.default_rng(3)
    h = rng.standard_normal((9, cfg["width"]))
    want = pz.latent_attention(m, w, "l0.mix.", h, 1e-5)
    H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    cq = pz.rms_norm(pz.linear(h, w["l0.mix.dq"]), w["l0.mix.dq.norm"], 1e-5)
    q = pz.linear(cq, w["l0.mix.uq"]).reshape(9, H, d)
    c = pz.rms_norm(pz.linear(h, w["l0.mix.dkv"]), w["l0.mix.dkv.norm"], 1e-5)
    uk, uv = w["l0.mix.uk"].astype(np.float64).reshape(H, d, R), w["l0.mix.uv"].astype(np.float64).reshape(H, dv, R)
    qa = np.einsum("thd,hdr->thr", q, uk)
    oa = pz.window_softmax_attention(qa, np.repeat(c[:, None], H, 1), np.repeat(c[:, None], H, 1), m["scale"], 4)
    got = pz.linear(np.einsum("thr,her->the", oa, uv).reshape(9, H * dv), w["l0.mix.o"])
    assert np.allclose(got, want)


def test_routed_ff_against_all_experts_masked():
    cfg = pz.random_config((L,), mlps=["moe"], experts=6, top=2)
    mlp = cfg["layers"][0]["mlp"]
    w = pz.random_weights(cfg, 1)
    h = np.random.default_rng(4).standard_normal((8, cfg["width"]))
    want = pz.routed_ff(mlp, w, "l0.mlp.", h)
    z = pz.linear(h, w["l0.mlp.router"], w["l0.mlp.router.b"])
    kth = np.sort(z, -1)[:, -2][:, None]
    p = np.where(z >= kth, np.exp(z - z.max(-1, keepdims=True)), 0.0)
    p /= p.sum(-1, keepdims=True)
    got = sum(p[:, [e]] * pz.linear(pz.silu(pz.linear(h, w[f"l0.mlp.e{e}.gate"])) * pz.linear(h, w[f"l0.mlp.e{e}.up"]), w[f"l0.mlp.e{e}.down"])
              for e in range(6))
    assert np.allclose(got, want)


def test_loop_runs_layers_in_passes():
    cfg = pz.random_config((D, L, D), loop=(1, 3, 2))
    assert pz.layer_runs(cfg) == [(0, False), (1, True), (2, False), (1, True), (2, False)]
    cfg = pz.random_config((D, L, D), loop=(0, 1, 3))
    assert pz.layer_runs(cfg) == [(0, True), (0, True), (0, True), (1, False), (2, False)]


def test_a_random_model_needs_the_ranks_named(tmp_path):
    from inferllm_b200 import write_random_model
    from inferllm_b200.binding import WeightError
    cfg = pz.random_config((D,))
    write_random_model(config_from_dict(cfg), str(tmp_path / "named"), 1)
    del cfg["layers"][0]["mixer"]["a_rank"]
    with pytest.raises(WeightError) as e:
        write_random_model(config_from_dict(cfg), str(tmp_path / "open"), 1)
    assert "a1" in str(e.value)

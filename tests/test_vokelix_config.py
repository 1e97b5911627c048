"""The Vokelix configuration class and the plain implementation's own pieces, on the CPU.

What config.json says must arrive in the ModelSpec unchanged (sizes, constants, layer order, which
cache entry a layer reads), the tensors the model declares must be the file's names and shapes, and
a configuration that cannot be built is refused in words.  The plain implementation's mechanisms are
checked against second, independent formulations of the same equations.
"""
import numpy as np
import pytest
import plain_vokelix as pv

from inferllm_b200 import ConfigError, VokelixConfig, config_from_dict
from inferllm_b200.weights import tensor_decls


def cfg_of(**kw):
    return pv.random_config(np.random.default_rng(0), **kw)


def test_spec_carries_every_size_and_constant():
    cfg = cfg_of(layer_types=("retention", "attention", "lightning", "attention"), share_from={3: 1}, width=56, vocab=77, heads=6, kv_heads=3,
                 dim=12, vdim=20, rot_dims=6, scale=0.37, base=777.0, lin_heads=2, lin_dim=4, lin_vdim=12, decay=[0.25, 0.875],
                 ret_rot_dims=2, ret_base=99.0, alpha=3.5, eps=2e-5, ff=72, no_mlp=[2])
    spec = config_from_dict(cfg).model_spec()
    assert (spec.hidden_size, spec.vocab_size) == (56, 77)
    assert [(e.layer, e.cache, e.writes) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False)]
    ret, att, lig, shared = [l.mixer for l in spec.layers]
    assert ret.kind == lig.kind == "decay_linear_attention" and att.kind == shared.kind == "attention"
    assert (att["n_heads"], att["n_kv_heads"], att["head_dim"], att["v_head_dim"], att["scale"]) == (6, 3, 12, 20, 0.37)
    assert att["qkv_bias"] and att["sink"] and att["qk_norm"] == "projection" and att["out_gate"] == "head_sigmoid"
    pos = att["position"]
    assert pos.kind == "rope_pairs" and (pos["rot_dim"], pos["theta"]) == (6, 777.0)
    assert pos["scaling"] == cfg["layers"][1]["mixer"]["rot"]["scaling"]
    assert shared["own_kv"] is False and att.get("own_kv", True) is True
    assert (ret["n_heads"], ret["head_dim"], ret["v_head_dim"], ret["decay"]) == (2, 4, 12, [0.25, 0.875])
    assert ret["position"].kind == "rope_half" and (ret["position"]["rot_dim"], ret["position"]["theta"]) == (2, 99.0)
    assert ret["k_scale"] == pytest.approx(0.5) and ret["out_norm"] == "per_head" and ret["gate_activation"] == "silu"
    assert lig["qk_activation"] == lig["v_activation"] == "silu" and lig["out_norm"] == "joint" and lig["gate_activation"] == "sigmoid"
    assert lig.get("position") is None
    assert [l.block for l in spec.layers] == ["postnorm", "postnorm", "postnorm_mixer", "postnorm"]
    for l in spec.layers:
        n = l.norms["norm1"]
        assert (n["eps"], n["weight_offset"], n["residual_scale"]) == (2e-5, 1.0, 3.5)
    assert spec.layers[0].ffn["intermediate_size"] == 72 and spec.layers[2].ffn.kind == ""
    assert spec.final_norm["weight_offset"] == 1.0


def test_the_python_face_is_typed_and_round_trips():
    cfg = cfg_of(layer_types=("lightning", "attention"), width=40)
    c = config_from_dict(cfg)
    assert isinstance(c, VokelixConfig) and c.architecture == "Vokelix"
    assert (c.width, c.vocab, c.postln_alpha) == (40, cfg["vocab"], cfg["postln_alpha"]) and len(c.layers) == 2
    assert VokelixConfig.from_dict(c.to_dict()) == c


def test_declared_tensors_are_the_files_names_and_shapes():
    cfg = cfg_of(layer_types=("lightning", "attention", "retention", "attention"), share_from={3: 1}, no_mlp=[2], vdim=40)
    decls = {name: tuple(shape) for name, (shape, _) in tensor_decls(config_from_dict(cfg)).items()}
    assert decls == {k: tuple(v) for k, v in pv.tensor_shapes(cfg).items()}


@pytest.mark.parametrize("change, words", [
    (lambda c: c["layers"][0].update(type="mamba"), "unknown type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=0), "attention layer"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "not supported"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.update(layers=[]), "at least one layer"),
])
def test_configurations_that_cannot_be_built_are_refused(change, words):
    cfg = cfg_of(layer_types=("lightning", "attention", "attention"))
    change(cfg)
    with pytest.raises(ConfigError, match=words):
        config_from_dict(cfg)


def test_shared_keys_need_equal_head_geometry():
    cfg = cfg_of(layer_types=("attention", "attention"), share_from={1: 0})
    cfg["layers"][1]["mixer"] = dict(cfg["layers"][1]["mixer"], kv_heads=1)
    with pytest.raises(ConfigError, match="same head count"):
        config_from_dict(cfg)


# ------------------------------------------------------------------ the plain implementation against second formulations


def test_state_scan_equals_the_explicit_double_sum():
    rng = np.random.default_rng(1)
    T, H, d, dv = 9, 2, 3, 4
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, H, d)), rng.normal(size=(T, H, dv))
    decay = [0.5, 0.9]
    want = np.zeros((T, H, dv))
    for h in range(H):
        for t in range(T):
            for s in range(t + 1):
                want[t, h] += decay[h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h]
    assert np.allclose(pv.decayed_state_scan(q, k, v, decay), want, atol=1e-12)


def test_sink_softmax_equals_a_softmax_with_one_more_key_of_zero_value():
    rng = np.random.default_rng(2)
    T, H, G, d, dv = 6, 4, 2, 5, 3
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, G, d)), rng.normal(size=(T, G, dv))
    sink = rng.normal(size=H)
    got = pv.sink_softmax_attention(q, k, v, 0.7, sink)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            scores = np.concatenate([(k[:t + 1, g] @ q[t, h]) * 0.7, [sink[h]]])
            w = np.exp(scores - scores.max())
            w /= w.sum()
            assert np.allclose(got[t, h], w[:-1] @ v[:t + 1, g], atol=1e-12)


def test_rotations_are_rotations_and_depend_on_the_distance_only():
    rng = np.random.default_rng(3)
    x, y = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    f, mag = pv.yarn_frequencies(100.0, 6, dict(factor=4.0, original=32, fast=8.0, slow=1.0))
    assert mag == pytest.approx(0.1 * np.log(4.0) + 1.0)
    plain = pv.base_frequencies(100.0, 6)
    assert f[0] == plain[0] and f[-1] == pytest.approx(plain[-1] / 4.0)      # the fastest pair is kept, the slowest stretched
    for layout in ("pairs", "half"):
        a = pv.rotate(x, [5], f, 1.0, 6, layout)
        assert np.allclose(a[..., 6:], x[..., 6:]) and np.allclose((a ** 2).sum(), (x ** 2).sum())
        dots = [float((pv.rotate(x, [p + 3], f, 1.0, 6, layout) * pv.rotate(y, [p], f, 1.0, 6, layout)).sum()) for p in (0, 4, 11)]
        assert np.allclose(dots, dots[0])
    assert np.allclose(pv.rotate(x, [2], f, mag, 6, "pairs")[..., :6], mag * pv.rotate(x, [2], f, 1.0, 6, "pairs")[..., :6])

"""Lasapel without a GPU: the configuration reader, the description the model is built from, the
frequency rule against the plain restatement, and the plain restatement against itself."""

import copy
import math

import numpy as np
import pytest

from tests import lasapel_util as U
from tests.plain import lasapel_plain as P


def test_describe_names_every_tensor_and_the_cache_plan():
    import torch
    from rust_llm_inference_server_b200.models.model import build_model
    for which, cfg in U.CONFIGS.items():
        m = build_model(cfg, "float32", "cpu")
        assert m.architecture == "Lasapel"
        assert {k: tuple(v) for k, v in m.tensors().items()} == U.tensor_shapes(cfg), which
    m = build_model(U.CONFIGS["X"], "bfloat16", "cpu")
    # layer 2 reads layer 0's slot and writes none; lightning layers have a state and no cache
    assert [(c.layer, c.cache, c.writes_cache) for c in m.calls] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    assert m.cache_slot_specs[0].head_dim == 40 and m.cache_slot_specs[0].values is False
    assert m.cache_slot_specs[1] is None and m.cache_slot_specs[3] is None
    assert [None if s is None else tuple(s.shape) for s in m.call_state_specs] == [None, (2, 40, 24), None, (3, 16, 16)]
    assert all(s is None or s.dtype == torch.float32 for s in m.call_state_specs)


def test_single_plane_groups_take_half_the_bytes():
    from rust_llm_inference_server_b200.cache import plan_groups
    from rust_llm_inference_server_b200.parts import KVCacheSpec
    g1, g2 = plan_groups([KVCacheSpec(1, 40, None, values=False), None, KVCacheSpec(1, 40)], 16)
    assert g1.planes == 1 and g2.planes == 2 and 2 * g1.bytes_per_page(2) == g2.bytes_per_page(2)


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "kv_from"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "mlp"),
])
def test_bad_configurations_are_refused(change, message):
    from rust_llm_inference_server_b200.config import ConfigError, LasapelConfig
    cfg = copy.deepcopy(U.CONFIGS["X"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        LasapelConfig.from_dict(cfg)


def test_registry_reads_the_single_name():
    from rust_llm_inference_server_b200.config import ConfigError, architecture_name, lookup_architecture
    assert architecture_name({"architecture": "Lasapel"}) == "Lasapel"
    assert architecture_name({}) == "LlamaForCausalLM"
    with pytest.raises(ConfigError):
        lookup_architecture({"architecture": "Nobody"})


@pytest.mark.parametrize("rot", [
    {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}},
    {"dims": 64, "base": 500000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
    {"dims": 6, "base": 100.0},
])
def test_frequencies_follow_the_plain_rule(rot):
    from rust_llm_inference_server_b200.parts.position import yarn_inverse_frequencies
    sc = rot.get("scaling") or {}
    f, mag = yarn_inverse_frequencies(rot["dims"], rot["base"], sc.get("factor"), sc.get("original", 0.0),
                                      sc.get("fast", 0.0), sc.get("slow", 0.0))
    cos, sin = P.rotary_table(rot, 3)
    # position 1 holds the frequencies themselves
    np.testing.assert_allclose(np.arctan2(sin[1], cos[1]), np.float64(f), rtol=1e-6)
    np.testing.assert_allclose(np.hypot(cos[1], sin[1]), mag, rtol=1e-12)
    if sc:
        assert mag == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)
        plain = rot["base"] ** (-2.0 * np.arange(rot["dims"] // 2) / rot["dims"])
        assert np.all(f <= plain * (1 + 1e-6)) and np.all(f >= plain / sc["factor"] * (1 - 1e-6))


def test_plain_lightning_equals_the_explicit_sum():
    rng = np.random.default_rng(0)
    T, W, mx = 9, 12, {"heads": 2, "dim": 3, "vdim": 4, "decay": [0.8, 0.3]}
    Wt = {"q": rng.standard_normal((6, W)), "k": rng.standard_normal((6, W)), "v": rng.standard_normal((8, W)),
          "g": rng.standard_normal((8, W)), "o": np.eye(8), "norm": np.ones(8)}
    h = rng.standard_normal((T, W))
    q, k, v = (P.silu(h @ Wt[n].T) for n in "qkv")
    o = np.zeros((T, 8))
    for hd in range(2):
        for t in range(T):
            for j in range(t + 1):
                o[t, 4 * hd:4 * hd + 4] += mx["decay"][hd] ** (t - j) * (q[t, 3 * hd:3 * hd + 3] @ k[j, 3 * hd:3 * hd + 3]) * v[j, 4 * hd:4 * hd + 4]
    want = P.plain_norm(o, np.ones(8), 1e-6) * P.sigmoid(h @ Wt["g"].T)
    np.testing.assert_allclose(P.lightning(Wt, "", mx, h, 1e-6), want, rtol=1e-9, atol=1e-12)


def test_plain_sink_only_enters_the_denominator():
    """With one token the attention weight is 1 / (1 + exp(sink - score)); a very low sink is no sink."""
    rng = np.random.default_rng(1)
    mx = U.latent(2, 4, 2, 3, 5, 6, 0.7)
    W = {"dq": rng.standard_normal((5, 8)), "dq.norm": np.ones(5), "uq": rng.standard_normal((12, 5)),
         "dkv": rng.standard_normal((8, 8)), "dkv.norm": np.ones(6), "uk": rng.standard_normal((8, 6)),
         "uv": rng.standard_normal((6, 6)), "o": np.eye(6), "sink": np.array([-50.0, 0.3])}
    h = rng.standard_normal((1, 8))
    kv = P.latent_kv(W, "", mx, h, 1e-6)
    out = P.latent_attention(W, "", mx, h, 1e-6, kv)[0]
    v = (kv[0] @ W["uv"].T)[0]
    np.testing.assert_allclose(out[:3], v[:3], rtol=1e-9)
    cq = P.plain_norm(h @ W["dq"].T, W["dq.norm"], 1e-6)
    q = (cq @ W["uq"].T).reshape(2, 6)
    score = (q[1, :4] @ (kv[0] @ W["uk"].T)[0, 4:] + q[1, 4:] @ kv[1][0]) * 0.7   # position 0: no rotation
    np.testing.assert_allclose(out[3:], v[3:] / (1 + math.exp(0.3 - score)), rtol=1e-9)


def test_a_lost_state_a_missing_sink_or_a_key_one_off_would_show(model_root):
    """The weights of these tests make such faults large: the plain restatement with the fault
    built in differs from the right one by far more than 0.045, the widest tolerance (a position's root-mean-square error) of the GPU tests."""
    d = U.make_dir(model_root, "X")
    cfg, w = U.read_config(d), U.plain_weights(d)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], size=120).tolist()
    right = P.forward(cfg, w, toks)
    no_sink = {k: (v - 40.0 if k.endswith("sink") else v) for k, v in w.items()}
    rms = lambda d: np.sqrt(np.mean(d * d, axis=-1)).max()
    assert rms(P.forward(cfg, no_sink, toks) - right) > 4 * 0.045
    lost = P.forward(cfg, w, toks[60:])                     # the state and the keys of the first 60 tokens are gone
    assert rms(lost - right[60:]) > 4 * 0.045
    dropped = P.forward(cfg, w, toks[:30] + toks[31:])      # one key missing, later positions one off
    assert rms(dropped[30:] - right[31:]) > 4 * 0.045

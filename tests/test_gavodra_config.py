"""Gavodra without a GPU: the configuration reader and what it refuses, the description against an
independent list of tensors, the bucket rule, the plain restatement against closed forms, and that the
test models' logits move far beyond the tolerances when a mechanism is left out."""

import copy
import math

import numpy as np
import pytest

from tests import gavodra_util as U
from tests.plain import gavodra_plain as P


def test_reader_takes_every_size_and_constant_from_the_file():
    from rust_llm_inference_server_b200.config import ConfigError, GavodraConfig
    cfg = GavodraConfig.from_dict(U.CONFIGS["A"])
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.residual_mult, cfg.embedding_scale, cfg.logit_scale, cfg.logit_softcap) == \
        (211, 96, 1e-5, 0.7, 3.0, 0.8, 9.0)
    m = cfg.layers[2].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.bias_max, m.v_mix) == (6, 2, 16, 16, 0.35, 25.0, True)
    assert cfg.layers[2].mlp is None and cfg.layers[0].mlp.kind == "dense" and cfg.layers[0].mlp.limit == 1.5
    x = cfg.layers[1].mlp
    assert (x.experts, x.top, x.scale, x.expert.ff, x.expert.limit, x.shared.ff, x.shared.limit) == (5, 2, 1.7, 24, 0.8, 40, 2.5)
    assert cfg.layers[3].mlp.shared is None
    b = GavodraConfig.from_dict(U.CONFIGS["B"])        # none of the optional constants
    assert (b.residual_mult, b.embedding_scale, b.logit_scale, b.logit_softcap) == (1.0, 1.0, 1.0, None)

    def broken(edit):
        c = copy.deepcopy(U.CONFIGS["A"])
        edit(c)
        with pytest.raises(ConfigError):
            GavodraConfig.from_dict(c)
    broken(lambda c: c["layers"][0]["mixer"].update(heads=3))                    # not a multiple of kv_heads
    broken(lambda c: c["layers"][0].update(type="convolution"))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=9))
    broken(lambda c: c["layers"][0]["mlp"].update(limit=0))
    broken(lambda c: c["layers"][2]["mixer"].update(vdim=24))                    # mixing layers must share the values' shape
    broken(lambda c: c.pop("norm"))
    broken(lambda c: c.update(logit_softcap=-1.0))
    broken(lambda c: c["layers"][1]["mlp"].update(kind="sparse"))


@pytest.mark.parametrize("which", sorted(U.CONFIGS))
def test_description_lists_the_tensors(which):
    from rust_llm_inference_server_b200.models.model import build_model
    model = build_model(U.CONFIGS[which], "float32", "cpu")
    want = U.tensor_shapes(U.CONFIGS[which], U.BIAS_ROWS[which])
    got = model.tensors()
    unread = set(model.spec.ignorable)
    assert set(got) | unread == set(want) and not (set(got) & unread)
    for name, shape in got.items():
        assert all(a is None or a == b for a, b in zip(shape, want[name])) and len(shape) == len(want[name]), name
    layers = U.CONFIGS[which]["layers"]
    first = next(i for i, l in enumerate(layers) if l["mixer"]["v_mix"])
    for i, l in enumerate(layers):                       # who mixes, who is the source
        s = model.spec.layers[i].mixer
        assert s.value_source == (i == first)
        assert (s.value_mix is not None) == (l["mixer"]["v_mix"] and i != first)
        assert (f"l{i}.mix.vmix" in unread) == (s.value_mix is None)
    assert model.graph_safe
    # keys and values of different widths live in pools of their own
    specs = model.cache_slot_specs
    assert all((sp.v_head_dim or sp.head_dim) == l["mixer"]["vdim"] and sp.head_dim == l["mixer"]["dim"]
               for sp, l in zip(specs, layers))


def test_bucket_rule():
    from rust_llm_inference_server_b200.parts.biased_attention import bias_by_distance, log_bucket
    import torch
    for rows, far in ((12, 40.0), (9, 30.5), (6, 7.0), (32, 1000.0), (16, 17.0)):
        half = rows // 2
        seen = [P.distance_bucket(n, rows, far) for n in range(int(far) + 50)]
        assert seen == [log_bucket(n, rows, far) for n in range(int(far) + 50)]
        assert seen[:half] == list(range(half))                      # one row a distance at first
        assert all(a <= b for a, b in zip(seen, seen[1:]))           # never back
        assert seen[half] == half and seen[-1] == rows - 1
        assert all(b == rows - 1 for n, b in enumerate(seen) if n >= far)
        edges = [n for n in range(1, len(seen)) if seen[n] != seen[n - 1]]
        for n in edges[half:]:                                       # an edge lies where the logarithm says
            k = seen[n] - half
            assert (n - 1) < half * (far / half) ** (k / (rows - half)) <= n + 1e-9
        table = torch.arange(rows * 3, dtype=torch.float32).reshape(rows, 3)
        by = bias_by_distance(table, far)
        assert by.shape[0] >= math.ceil(far) and float(by[-1, 0]) == float(table[-1, 0])
        assert [int(v) // 3 for v in by[:, 0].tolist()] == seen[:by.shape[0]]
    with pytest.raises(ValueError):
        bias_by_distance(torch.zeros((8, 2)), 3.0)                  # reach inside the one-row-a-distance part


def test_plain_functions_against_closed_forms():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 8))
    w = rng.standard_normal(8)
    y = P.rms_norm(x, w, 1e-3)
    assert np.allclose(y[1], x[1] / math.sqrt(float(np.mean(x[1] ** 2)) + 1e-3) * w)
    # the gated unit: gate cut from above only, linear branch clipped on both sides, then shifted by one
    eye = np.eye(4)
    h = np.array([[5.0, -5.0, 0.5, -0.5]])
    out = P.clipped_glu(h, eye, eye, eye, 2.0)[0]
    g = np.array([2.0, -5.0, 0.5, -0.5])
    u = np.array([2.0, -2.0, 0.5, -0.5])
    assert np.allclose(out, g / (1 + np.exp(-1.702 * g)) * (u + 1))
    # the router: the correction picks, the plain score weighs
    wr = np.array([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0]])
    idx, wts = P.route(np.array([[2.0, 1.0]]), wr, np.array([0.0, 0.0, 5.0]), 2, 3.0)
    assert idx.tolist() == [[2, 0]]
    assert np.allclose(wts, [[3.0 / (1 + math.e ** 2), 3.0 / (1 + math.e ** -2)]])


def _logits(which, edit=None, root=None, cfg_edit=None):
    cfg = copy.deepcopy(U.CONFIGS[which])
    if cfg_edit:
        cfg_edit(cfg)
    w = {k: v.double().numpy() for k, v in U.draw_weights(U.CONFIGS[which], U.SEEDS[which], U.BIAS_ROWS[which]).items()}
    if edit:
        edit(w)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=70).tolist()
    return P.forward(w, cfg, toks)


@pytest.mark.parametrize("which", ["A", "B"])
def test_a_missing_mechanism_shows_in_the_logits(which):
    base = _logits(which)

    def moved(**kw):
        d = _logits(which, **kw) - base
        return float(np.sqrt(np.mean(d * d, axis=-1)).max())
    mixing = [i for i, l in enumerate(U.CONFIGS[which]["layers"]) if l["mixer"]["v_mix"]]
    routed = [i for i, l in enumerate(U.CONFIGS[which]["layers"]) if l["mlp"] and l["mlp"]["kind"] == "moe"]
    # no bias by distance; a table read one row off; no value mixing; no gate; no correction; no shared expert's gate
    assert moved(edit=lambda w: [w.__setitem__(k, v * 0) for k, v in list(w.items()) if k.endswith(".rel")]) > 0.2
    assert moved(edit=lambda w: [w.__setitem__(k, np.roll(v, 1, axis=0)) for k, v in list(w.items()) if k.endswith(".rel")]) > 0.2
    assert moved(edit=lambda w: w.__setitem__(f"l{mixing[1]}.mix.vmix", np.asarray(0.0))) > 0.1
    assert moved(edit=lambda w: [w.__setitem__(k, v * 0) for k, v in list(w.items()) if k.endswith("mix.g")]) > 0.2
    assert moved(edit=lambda w: w.__setitem__(f"l{routed[0]}.mlp.correction", w[f"l{routed[0]}.mlp.correction"] * 0)) > 0.05
    assert moved(edit=lambda w: w.__setitem__(f"l{routed[0]}.mlp.shared.sg", w[f"l{routed[0]}.mlp.shared.sg"] * 0)) > 0.02
    # a limit that is not applied; a wrong scale
    assert moved(cfg_edit=lambda c: [l["mlp"].update(limit=50.0) for l in c["layers"] if l["mlp"] and l["mlp"]["kind"] == "dense"]) > 0.05
    assert moved(cfg_edit=lambda c: c["layers"][0]["mixer"].update(scale=c["layers"][0]["mixer"]["scale"] * 2)) > 0.2


def test_value_rows_of_their_own_width_get_a_pool_of_their_own():
    """Sizing counts key and value rows by their own widths, and equal specs still share a group."""
    from rust_llm_inference_server_b200.cache.storage import plan_groups, size_groups
    from rust_llm_inference_server_b200.parts.base import KVCacheSpec
    narrow = KVCacheSpec(2, 64, None, v_head_dim=16)
    same = KVCacheSpec(2, 64, None)
    groups = plan_groups([narrow, same, narrow, None, same], 8)
    assert [g.slots for g in groups] == [[0, 2], [1, 4]]
    assert groups[0].bytes_per_page(2) == 2 * 2 * 8 * (64 + 16) * 2 and groups[0].v_head_dim == 16
    assert groups[1].bytes_per_page(2) == 2 * 2 * 8 * (64 + 64) * 2 and groups[1].v_head_dim == 64
    size_groups(groups, 10 * (groups[0].bytes_per_page(2) + groups[1].bytes_per_page(2)), 2)
    assert [g.num_pages for g in groups] == [10, 10]


def test_a_checkpoint_may_decide_an_open_extent():
    import torch
    from rust_llm_inference_server_b200.weights.loader import WeightError, check_checkpoint
    from rust_llm_inference_server_b200.weights.safetensors_io import Checkpoint
    ckpt = Checkpoint(tensors={"t": torch.zeros(7, 3), "u": torch.zeros(2)})
    check_checkpoint({"t": (None, 3), "u": (2,)}, ckpt)
    with pytest.raises(WeightError):
        check_checkpoint({"t": (None, 4), "u": (2,)}, ckpt)
    with pytest.raises(WeightError):
        check_checkpoint({"t": (None,), "u": (2,)}, ckpt)

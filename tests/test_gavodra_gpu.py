"""Gavodra on the GPU against the plain restatement: every kernel alone (keys far back made to carry a
head's weight, table rows and page borders one position off, first tokens, gates, mixing, routing with
crowded and empty experts), every kind of layer alone in a small model, whole prompts against portions,
single tokens and mixed batches in pools so small that pages are used again, long decoding, and greedy
generation through the entry point and the command line."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from tests import gavodra_util as U
from tests import replay_util as R
from tests.plain import gavodra_plain as P

pytestmark = pytest.mark.gpu

# A position's error is the root mean square, over the vocabulary, of the difference of its logits, as a
# part of the spread of the logits there (1 to 2 in these models).  float32: sums in another order than
# the plain float64 ones.  bfloat16: every product's inputs are rounded to 8 bits and attention here is
# peaked, which amplifies it.
TOL = {"float32": 5e-5, "bfloat16": 0.06}
TOL_BETWEEN = {"float32": 1e-5, "bfloat16": 0.06}


def position_error(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    d = a - b
    e = float(np.sqrt(np.mean(d * d)) / max(float(np.std(b)), 0.5))
    return e if np.isfinite(e) else float("inf")


def dev(x, dtype=torch.float32):
    return torch.as_tensor(np.asarray(x)).to(device="cuda", dtype=dtype).contiguous()


def host(t):
    return t.detach().to("cpu", torch.float64).numpy()


def requests_for(cfg, lens, seed=1):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab"], size=n).tolist() for i, n in enumerate(lens)}


def plain_logits(model_dir, reqs):
    cfg, w = U.read_config(model_dir), U.plain_weights(model_dir)
    return {name: P.forward(w, cfg, toks) for name, toks in reqs.items()}


def session(model_dir, dtype, max_tokens, page=16, max_live=4):
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    return ReplaySession(model_dir, dtype, max_tokens, page, max_live=max_live)


def worst_difference(got, ref):
    worst, where = 0.0, None
    for (name, pos), row in got.items():
        d = position_error(row, ref[name][pos])
        if d >= worst:
            worst, where = d, (name, pos)
    return worst, where


def model_dir(root, which, dtype, cfg=None, seed=None):
    """The model folder of a run: the bfloat16 runs take weights whose routing does not hang on close scores."""
    if dtype == "bfloat16":
        return U.make_dir(root, which + "_settled", cfg or U.CONFIGS[which], U.SEEDS.get(which, 0) if seed is None else seed,
                          U.BIAS_ROWS.get(which), edit=U.settle_routing)
    return U.make_dir(root, which, cfg, seed)


# ---- the kernels, one by one -------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [40, 96, 1030])
def test_scaled_join_and_copy_of_the_stream(dtype, hidden):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(hidden)
    T = 5
    sub, resid = dev(rng.standard_normal((T, hidden)) * 3, dtype), dev(rng.standard_normal((T, hidden)))
    w = dev(1 + 0.3 * rng.standard_normal(hidden))
    want = host(resid) + 0.37 * P.rms_norm(host(sub), host(w), 1e-4)
    out = torch.empty((T, hidden), dtype=dtype, device="cuda")
    assert ops.post_norm_residual(sub, resid, w, 1e-4, mult=0.37, out=out) is out
    np.testing.assert_allclose(host(resid), want, rtol=0, atol=3e-6)                  # float32 whatever the type
    assert torch.equal(out, resid.to(dtype))                                         # the stream, rounded once
    before = resid.clone()
    ops.post_norm_residual(sub, resid, w, 1e-4, mult=-1.5)                             # no copy asked for
    np.testing.assert_allclose(host(resid), host(before) - 1.5 * P.rms_norm(host(sub), host(w), 1e-4), rtol=0, atol=5e-6)
    out.zero_()
    before = resid.clone()
    ops.post_norm_residual(None, resid, None, 0.0, out=out)                           # only the copy
    assert torch.equal(resid, before) and torch.equal(out, resid.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clipped_gating(dtype):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(1)
    gu = dev(rng.standard_normal((7, 2 * 36)) * 3, dtype)
    out = torch.empty((7, 36), dtype=dtype, device="cuda")
    for slope, limit, shift in ((1.702, 1.25, 1.0), (1.0, None, 0.0), (0.5, 0.3, -2.0)):
        ops.glu_act(gu, out, slope, limit, shift)
        g, u = host(gu)[:, :36], host(gu)[:, 36:]
        if limit is not None:
            g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
        want = g * P.sigmoid(slope * g) * (u + shift)
        np.testing.assert_allclose(host(out), want, rtol=0, atol=1e-5 if dtype == torch.float32 else 0.04)


def hand_step(ctx_lens, q_lens, page, n_pages, rng, tile=64):
    """A step made by hand: request b has ctx_lens[b] tokens of which the last q_lens[b] are the step's;
    pages are dealt out in a shuffled order, so neighbours in a request are not neighbours in the pool."""
    B = len(ctx_lens)
    need = [-(-c // page) for c in ctx_lens]
    assert sum(need) <= n_pages
    perm = rng.permutation(n_pages)
    max_blocks = max(need) + 1
    tables = -np.ones((B, max_blocks), dtype=np.int32)
    k = 0
    for b in range(B):
        tables[b, :need[b]] = perm[k:k + need[b]]
        k += need[b]
    pos, seq, slots = [], [], []
    for b in range(B):
        for p in range(ctx_lens[b] - q_lens[b], ctx_lens[b]):
            pos.append(p)
            seq.append(b)
            slots.append(tables[b, p // page] * page + p % page)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    dec = [b for b in range(B) if q_lens[b] == 1]
    tiles = sorted(((b, t0) for b in range(B) if q_lens[b] > 1 for t0 in range(0, q_lens[b], tile)),
                   key=lambda bt: -(ctx_lens[bt[0]] - q_lens[bt[0]] + bt[1]))
    bufs = {}

    def buffer(name, shape, dtype):
        n = int(np.prod(shape))
        if name not in bufs or bufs[name].numel() < n or bufs[name].dtype != dtype:
            bufs[name] = torch.empty((max(n, 1),), dtype=dtype, device="cuda")
        return bufs[name][:n].view(*shape)
    i32 = lambda a: dev(np.asarray(a, dtype=np.int32), torch.int32)
    pf_rows = [r for b in range(B) if q_lens[b] > 1 for r in range(cu[b], cu[b + 1])]
    return SimpleNamespace(
        n_tokens=len(pos), n_seqs=B, positions=i32(pos), seq_of_token=i32(seq), slots=[i32(slots)],
        block_tables=[i32(tables)], ctx_lens=i32(ctx_lens), cu_seqlens=i32(cu), q_lens=list(q_lens),
        n_decode=len(dec), dec_rows=i32([cu[b] for b in dec]) if dec else None, dec_seqs=i32(dec) if dec else None,
        max_decode_ctx=max([ctx_lens[b] for b in dec], default=0), n_prefill_tokens=len(pf_rows),
        prefill_rows=i32(pf_rows) if pf_rows and dec else None, n_prefill_tiles=len(tiles),
        prefill_tiles=i32(tiles).view(-1, 2) if tiles else None, max_ctx_len=max(ctx_lens), all_decode=not tiles,
        buffer=buffer, host_pos=pos, host_seq=seq, host_tables=tables)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 32, 16), (3, 3, 8, 24), (2, 1, 80, 40)])
def test_norms_mixing_and_the_paged_write(dtype, H, G, d, dv):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(d)
    page, n_pages = 8, 12
    st = hand_step([19, 5, 30], [7, 1, 30], page, n_pages, rng)
    T = st.n_tokens
    lead = 8                                            # the sections start at a column offset, as in a stacked projection
    N = lead + H * d + G * d + G * dv + H
    proj = dev(rng.standard_normal((T, N)) * 2, dtype)
    other = dev(rng.standard_normal((T, G * dv + 5)), dtype)[:, 3:3 + G * dv]
    qw, kw = dev(1 + 0.5 * rng.standard_normal(d)), dev(1 + 0.5 * rng.standard_normal(d))
    kc = torch.full((n_pages, G, page, d), 7.0, dtype=dtype, device="cuda")
    vc = torch.full((n_pages, G, page, dv), 7.0, dtype=dtype, device="cuda")
    q_out = torch.empty((T, H * d), dtype=dtype, device="cuda")
    q_off, k_off, v_off = lead, lead + H * d, lead + H * d + G * d
    tol = 1e-5 if dtype == torch.float32 else 0.05
    x = host(proj)
    want_q = P.rms_norm(x[:, q_off:k_off].reshape(T, H, d), host(qw), 1e-5).reshape(T, -1)
    want_k = P.rms_norm(x[:, k_off:v_off].reshape(T, G, d), host(kw), 1e-5)
    for lam, oth in ((0.0, None), (0.3, other)):
        ops.qk_norm_store(proj, q_off, k_off, v_off, qw, kw, 1e-5, oth, lam, q_out, kc, vc, st.slots[0], H, G, d, dv, page)
        want_v = x[:, v_off:v_off + G * dv].reshape(T, G, dv)
        if oth is not None:
            want_v = (1 - lam) * want_v + lam * host(oth).reshape(T, G, dv)
        np.testing.assert_allclose(host(q_out), want_q, rtol=0, atol=tol)
        touched = np.zeros((n_pages, page), dtype=bool)
        for t in range(T):
            pg = st.host_tables[st.host_seq[t], st.host_pos[t] // page]
            touched[pg, st.host_pos[t] % page] = True
            np.testing.assert_allclose(host(kc[pg, :, st.host_pos[t] % page]), want_k[t], rtol=0, atol=tol)
            np.testing.assert_allclose(host(vc[pg, :, st.host_pos[t] % page]), want_v[t], rtol=0, atol=tol)
        # nothing else of the pools was written
        assert float((kc.float().permute(0, 2, 1, 3)[~torch.from_numpy(touched).cuda()] - 7.0).abs().max()) == 0.0
        assert float((vc.float().permute(0, 2, 1, 3)[~torch.from_numpy(touched).cuda()] - 7.0).abs().max()) == 0.0
    # no norm weights, nothing stored
    kc.fill_(7.0)
    ops.qk_norm_store(proj, q_off, k_off, v_off, None, None, 1e-5, None, 0.0, q_out, kc, vc, None, H, G, d, dv, page)
    np.testing.assert_allclose(host(q_out), x[:, q_off:k_off], rtol=0, atol=0)
    assert float((kc.float() - 7.0).abs().max()) == 0.0


def plain_attention_rows(q, keys, vals, bias, gate, scale, st, H, G, window=0):
    """q [T, H, d]; keys/vals: per request the whole context [ctx, G, d | dv]; bias [n_dist, H]."""
    T = q.shape[0]
    out = np.zeros((T, H, vals[0].shape[-1]))
    for t in range(T):
        b, pos = st.host_seq[t], st.host_pos[t]
        lo = max(0, pos - window + 1) if window else 0
        for h in range(H):
            g = h // (H // G)
            dist = pos - np.arange(lo, pos + 1)
            s = keys[b][lo:pos + 1, g] @ q[t, h] * scale
            if bias is not None:
                s = s + bias[np.minimum(dist, bias.shape[0] - 1), h]
            w = np.exp(s - s.max())
            out[t, h] = (w / w.sum()) @ vals[b][lo:pos + 1, g]
            if gate is not None:
                out[t, h] *= P.sigmoid(gate[t, h])
    return out


def fill_pools(st, keys, vals, page, n_pages, dtype):
    G, d, dv = keys[0].shape[1], keys[0].shape[2], vals[0].shape[2]
    kc = torch.full((n_pages, G, page, d), 50.0, dtype=dtype, device="cuda")      # what is never written must never be read
    vc = torch.full((n_pages, G, page, dv), 50.0, dtype=dtype, device="cuda")
    for b, (k, v) in enumerate(zip(keys, vals)):
        for p in range(k.shape[0]):
            pg = st.host_tables[b, p // page]
            kc[pg, :, p % page] = dev(k[p], dtype)
            vc[pg, :, p % page] = dev(v[p], dtype)
    return kc, vc


ATTN_SHAPES = [(4, 2, 32, 16, 8), (3, 3, 8, 24, 16), (2, 1, 80, 40, 32), (6, 2, 64, 64, 16), (2, 1, 128, 32, 8),
               (8, 4, 64, 32, 16), (4, 4, 128, 128, 16), (4, 2, 128, 64, 16), (2, 2, 64, 128, 32), (16, 1, 64, 64, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,page", ATTN_SHAPES)
def test_attention_far_keys_table_rows_page_borders_and_gates(dtype, H, G, d, dv, page):
    """Whole prompts, portions that start in the middle of a page, and single tokens in one launch.  Per head
    one key far back is made to carry the weight (query and key scaled), so a lost key, a wrong page or a
    wrong table row shows; the bias table is large where it is read and larger one row further."""
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.parts.biased_attention import bias_by_distance
    rng = np.random.default_rng(H * 100 + d)
    ctx = [333, 70, 129, 1, 2, 1100, 65]               # the single token of 1,100 is cut into pieces by the split kernel
    qn = [333, 1, 37, 1, 2, 1, 64]
    n_pages = sum(-(-c // page) for c in ctx) + 3
    st = hand_step(ctx, qn, page, n_pages, rng)
    T = st.n_tokens
    rows, far = 14, 90.0
    table = rng.standard_normal((rows, H)) * 2.0
    bias = bias_by_distance(dev(table), far)
    assert np.allclose(host(bias), P.distance_bias(table.astype(np.float32).astype(np.float64), far, bias.shape[0]))
    keys = [rng.standard_normal((c, G, d)) for c in ctx]
    vals = [rng.standard_normal((c, G, dv)) for c in ctx]
    q = rng.standard_normal((T, H, d))
    scale = 0.9 / np.sqrt(d)
    # the last token of request 0 and the single token of request 5 look at one far key each, per head
    # another: at position 0 (the first token), at a page's last and first slot, and right where the
    # bias table changes rows
    edges = [n for n in range(1, 120) if P.distance_bucket(n, rows, far) != P.distance_bucket(n - 1, rows, far)]
    t_last0, t5 = qn[0] - 1, sum(qn[:5])
    for t, c in ((t_last0, ctx[0]), (t5, ctx[5])):
        pos = c - 1
        targets = [0, page - 1, page, pos - edges[-1], pos - edges[-1] + 1, pos - edges[len(edges) // 2], 3 * page, pos - 1]
        for h in range(H):
            j = targets[h % len(targets)]
            g = h // (H // G)
            q[t, h] = keys[st.host_seq[t]][j, g] * (9.0 / scale / float(keys[st.host_seq[t]][j, g] @ keys[st.host_seq[t]][j, g]))
    gate = rng.standard_normal((T, H)) * 2
    qd, gd = dev(q.reshape(T, -1), dtype), dev(np.concatenate([np.zeros((T, 3)), gate], 1), dtype)[:, 3:]
    keys = [host(dev(k, dtype)) for k in keys]
    vals = [host(dev(v, dtype)) for v in vals]
    kc, vc = fill_pools(st, keys, vals, page, n_pages, dtype)
    out = torch.empty((T, H * dv), dtype=dtype, device="cuda")
    tol = 2e-5 if dtype == torch.float32 else 0.03
    for use_bias, use_gate, window in ((True, True, 0), (False, False, 0), (True, False, 100)):
        out.fill_(float("nan"))
        ops.attention_biased(qd, kc, vc, out, bias if use_bias else None, gd if use_gate else None, st, 0, H, G, d, dv,
                             page, scale, window)
        want = plain_attention_rows(host(qd).reshape(T, H, d), keys, vals, host(bias) if use_bias else None,
                                    host(gd) if use_gate else None, scale, st, H, G, window)
        got = host(out).reshape(T, H, dv)
        err = np.abs(got - want).max(axis=(1, 2))
        assert np.isfinite(got).all() and err.max() <= tol, f"row {int(err.argmax())}: {err.max()}"
    if dtype == torch.bfloat16 and ops.biased_attention_takes_mma(dtype, H, G, d, dv):
        assert ops.launches_by_kernel.get("attention_bias.decode.mma.split") and ops.launches_by_kernel.get("attention_bias.prefill.mma")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,W,I", [(1, 3, 1, 40, 24), (37, 5, 2, 96, 40), (150, 9, 3, 64, 72), (64, 4, 4, 32, 16),
                                          (300, 3, 2, 64, 48),          # wide tiles of the sort
                                          (600, 3, 2, 256, 128)])       # ... and sizes the grouped tcgen05 product takes
def test_routing_choice_sort_and_experts(dtype, T, E, top, W, I):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(T)
    x = dev(rng.standard_normal((T, W)), dtype)
    wr = dev(np.concatenate([rng.standard_normal((E, W)) * 2 / np.sqrt(W), rng.standard_normal((1, W)) / np.sqrt(W)]))
    corr = rng.standard_normal(E) * 0.5
    corr[0] += 3.0                                      # a crowded expert, whose rows fill more than one tile
    corr = dev(corr)
    st = SimpleNamespace(buffer=hand_step([1], [1], 8, 1, rng).buffer)
    plan = ops.moe_route(x, wr, corr, E, top, 1.3, True, st)
    idx, wts = P.route(host(x), host(wr)[:E], host(corr), top, 1.3)
    assert np.array_equal(plan.top_idx.view(T, top).cpu().numpy(), idx)
    np.testing.assert_allclose(host(plan.top_w).reshape(T, top), wts, rtol=0, atol=1e-5)
    np.testing.assert_allclose(host(plan.shared_gate), P.sigmoid(host(x) @ host(wr)[E]), rtol=0, atol=1e-5)
    # the sort: every pair sits in exactly one slot, of a tile of its expert
    sp, ps, te = plan.sorted_pair.cpu().numpy(), plan.pair_slot.cpu().numpy(), plan.tile_expert.cpu().numpy()
    assert sorted(sp[sp >= 0].tolist()) == list(range(T * top))
    assert plan.tile == (128 if T >= 300 else 32)
    for pair in range(T * top):
        assert sp[ps[pair]] == pair and te[ps[pair] // plan.tile] == idx.reshape(-1)[pair]
    wg, wu = (dev(rng.standard_normal((E, I, W)) / np.sqrt(W), dtype) for _ in range(2))
    wd = dev(rng.standard_normal((E, W, I)) / np.sqrt(I), dtype)
    # both branches in one stack: in blocks of 4 rows, and gate rows first
    stacks = {4: torch.stack([wg.view(E, -1, 4, W), wu.view(E, -1, 4, W)], dim=2).reshape(E, 2 * I, W).contiguous(),
              0: torch.cat([wg, wu], dim=1).contiguous()}
    ops.launches_by_kernel.clear()
    acts = {il: ops.moe_up(x, stack, plan, 1.702, 0.9, 1.0, st, il).clone() for il, stack in stacks.items()}
    real = plan.sorted_pair >= 0
    assert float((acts[4][real].float() - acts[0][real].float()).abs().max()) <= (0.0 if dtype == torch.float32 else 0.05)
    act = acts[4]
    y = ops.moe_down(act, wd, plan, st)
    grouped = dtype == torch.bfloat16 and T == 600
    assert ops.launches_by_kernel.get("gemm_tcgen05.grouped.glu4", 0) == (1 if grouped else 0)
    assert ops.launches_by_kernel.get("gemm_tcgen05.grouped", 0) == (2 if grouped else 0)
    shared = dev(rng.standard_normal((T, W)), dtype)
    out = torch.empty((T, W), dtype=dtype, device="cuda")
    ops.moe_combine(y, plan, shared, out)
    want = np.zeros((T, W))
    for t in range(T):
        for e, wt in zip(idx[t], wts[t]):
            want[t] += wt * P.clipped_glu(host(x)[t:t + 1], host(wg)[e], host(wu)[e], host(wd)[e], 0.9)[0]
    want += P.sigmoid(host(x) @ host(wr)[E])[:, None] * host(shared)
    np.testing.assert_allclose(host(out), want, rtol=0, atol=3e-5 if dtype == torch.float32 else 0.06)
    ops.check_device_errors()
    # without a shared expert and without a correction
    plan = ops.moe_route(x, wr[:E].contiguous(), None, E, top, 1.0, False, st)
    assert plan.shared_gate is None
    assert np.array_equal(plan.top_idx.view(T, top).cpu().numpy(), P.route(host(x), host(wr)[:E], np.zeros(E), top, 1.0)[0])


def test_gated_product_with_clipping_in_its_epilogue():
    """The tcgen05 gate|up product with the clipped gating on its accumulators against the plain form, one
    tile of rows (one SM a tile) and several (two SMs a tile), and the gating kernel on the same layout."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(2)
    K, I = 96, 256
    wg, wu = rng.standard_normal((I, K)) / np.sqrt(K) * 2, rng.standard_normal((I, K)) / np.sqrt(K) * 2
    w = torch.stack([dev(wg, torch.bfloat16).view(-1, 4, K), dev(wu, torch.bfloat16).view(-1, 4, K)], dim=1).reshape(2 * I, K).contiguous()
    for M in (128, 300):
        x = dev(rng.standard_normal((M, K)), torch.bfloat16)
        for slope, limit, shift in ((1.702, 0.8, 1.0), (1.0, None, 0.0)):
            got = ops.gemm_tcgen05(x, w, "glu4", glu=(slope, limit, shift))
            g, u = host(x) @ host(dev(wg, torch.bfloat16)).T, host(x) @ host(dev(wu, torch.bfloat16)).T
            if limit is not None:
                g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
            want = g * P.sigmoid(slope * g) * (u + shift)
            np.testing.assert_allclose(host(got), want, rtol=0.01, atol=0.02)     # one rounding to bfloat16
            gu = ops.linear(x, w)
            out = torch.empty((M, I), dtype=torch.bfloat16, device="cuda")
            ops.glu_act(gu, out, slope, limit, shift, 4)
            np.testing.assert_allclose(host(out), want, rtol=0.02, atol=0.03)     # the sums are rounded before the gating here
    ops.check_device_errors()


# ---- whole models ------------------------------------------------------------------------------

ALONE = {
    "attention_only": U.model(61, 48, 1e-5, [U.layer(U.attn(3, 1, 16, 8, 0.3, 20.0))], residual_mult=0.6, emb_scale=2.0),
    "with_dense": U.model(61, 48, 1e-5, [U.layer(U.attn(2, 2, 24, 16, 0.25, 12.0, v_mix=False), U.dense(56, 1.1))], softcap=5.0),
    "with_routed": U.model(61, 48, 1e-5, [U.layer(U.attn(2, 1, 8, 8, 0.5, 33.0), U.moe(4, 2, 16, 0.7, 2.0, shared=(24, 1.3)))],
                           logit_scale=1.4),
    "two_mixing": U.model(61, 48, 1e-5, [U.layer(U.attn(2, 1, 8, 24, 0.5, 33.0)), U.layer(U.attn(4, 1, 16, 24, 0.2, 9.0))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_kind_of_layer_alone(model_root, which, dtype):
    d = model_dir(model_root, which, dtype, ALONE[which], seed=11)
    reqs = requests_for(ALONE[which], [1, 2, 37, 90])
    ref = plain_logits(d, reqs)
    for fam, steps in (("whole", R.whole_trace(reqs)), ("decode", R.decode_trace(reqs, tail=20)),
                       ("chunks", R.chunk_trace(reqs, seed=2))):
        s = session(d, dtype, R.live_token_peak(steps), 8)
        worst, where = worst_difference(R.collect(s.step, steps), ref)
        assert worst <= TOL[dtype], f"{which} {dtype} {fam}: {worst} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,page,lens", [("A", 16, [1, 50, 97, 200, 64, 17, 2]), ("A", 8, [130, 33, 2, 71, 40]),
                                             ("B", 16, [3, 150, 40, 2, 129, 1]), ("B", 32, [260, 31, 5, 90]),
                                             ("C", 16, [1, 70, 333, 2, 129, 64, 65]), ("C", 8, [200, 31, 5, 400]),
                                             ("D", 16, [90, 1, 33, 150, 2]), ("E", 16, [420, 3, 200, 77])])
def test_all_ways_of_cutting_give_the_plain_logits(model_root, which, page, lens, dtype):
    from rust_llm_inference_server_b200 import ops
    ops.launches_by_kernel.clear()
    d = model_dir(model_root, which, dtype)
    reqs = requests_for(U.CONFIGS[which], lens, seed=page)
    ref = plain_logits(d, reqs)
    families = {
        "whole": (R.whole_trace(reqs), 4),
        "decode": (R.decode_trace(reqs, tail=40), 4),
        "chunks": (R.chunk_trace(reqs, seed=3), 4),
        "mixed": (R.mixed_trace(reqs, seed=4), 4),
        "mixed2": (R.mixed_trace(dict(reversed(list(reqs.items()))), seed=5, max_live=2), 2),
    }
    results = {}
    for fam, (steps, live) in families.items():
        s = session(d, dtype, R.live_token_peak(steps, max(64, page)), page, max_live=live)
        for pool in s.storage.pools:                         # whatever a page held before must not matter
            for t in (pool if isinstance(pool, tuple) else (pool,)):
                t.fill_(30.0)
        results[fam] = R.collect(s.step, steps)
        assert s.cache.check_invariants() == ""
        assert s.cache.num_free_pages(0) == s.cache.group(0).num_pages, fam
        worst, where = worst_difference(results[fam], ref)
        assert worst <= TOL[dtype], f"{which} {dtype} {fam} vs plain: {worst} at {where}"
    for fam in ("decode", "chunks", "mixed", "mixed2"):
        whole = {}
        for (name, pos), row in results["whole"].items():
            whole.setdefault(name, {})[pos] = row
        worst, where = worst_difference(results[fam], whole)
        assert worst <= TOL_BETWEEN[dtype], f"{which} {dtype}: {fam} differs from whole by {worst} at {where}"
    fast = dtype == "bfloat16" and which in ("C", "E")
    if dtype == "bfloat16" and which == "E":     # prompts of 200 and 420 tokens: 96 pairs an expert and more
        assert ops.launches_by_kernel.get("gemm_tcgen05.grouped.glu4") and ops.launches_by_kernel.get("gemm_tcgen05.grouped")
    for k in (("attention_bias.decode.mma", "attention_bias.prefill.mma", "gemm_tcgen05.glu4") if fast else ("attention_bias",)) + \
            (("moe_gemm.mma.glu", "moe_gemm.mma.down") if dtype == "bfloat16" and which != "D" else ("moe_gemm.glu", "moe_gemm.down")) + \
            ("qk_norm_store", "qk_norm_store.mix", "post_norm_residual", "post_norm_residual.copy" if dtype == "bfloat16" else
              "post_norm_residual", "glu_act", "moe_route", "moe_align", "moe_combine"):
        assert ops.launches_by_kernel.get(k), f"never launched {k}; launched {sorted(ops.launches_by_kernel)}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_reach_of_the_bias_table(model_root, dtype):
    d = model_dir(model_root, "B", dtype)
    reqs = requests_for(U.CONFIGS["B"], [230], seed=9)
    ref = plain_logits(d, reqs)
    steps = R.decode_trace(reqs, tail=215)              # decoded tokens pass every row of the tables, and a page border every 8
    s = session(d, dtype, R.live_token_peak(steps), 8)
    worst, where = worst_difference(R.collect(s.step, steps), ref)
    assert worst <= TOL[dtype], f"{worst} at {where}"


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(P.forward(w, cfg, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(model_root, dtype):
    """Prompts of unequal length batched by the scheduler, portions of 16 tokens, decode steps from CUDA
    graphs and launched ahead; two seats, so the later prompts wait for the earlier ones to end."""
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    d = model_dir(model_root, "A", dtype)
    cfg, w = U.read_config(d), U.plain_weights(d)
    prompts = list(requests_for(cfg, [1, 9, 40, 23, 3], seed=12).values())
    llm = LLM(d, dtype=dtype, max_seq_len=128, num_blocks=40, block_size=8, max_num_seqs=2, max_batched_tokens=16)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12))
    for p, o in zip(prompts, outs):
        want = plain_greedy(cfg, w, p, 12)
        assert o.finish_reason == "length" and len(o.token_ids) == 12
        if o.token_ids != want:
            i = next(k for k, (a, b) in enumerate(zip(o.token_ids, want)) if a != b)
            lg = P.forward(w, cfg, p + want[:i])[-1]
            gap = lg[want[i]] - lg[o.token_ids[i]]
            assert dtype == "bfloat16" and gap < 0.15, f"parted at token {i} with a gap of {gap}"


def test_command_line_serves_the_design(tmp_path):
    """random-weights and generate of the command line with a Gavodra folder."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def rlis(*args):
        return subprocess.run([sys.executable, os.path.join(root, "bin", "rlis"), *args], capture_output=True,
                              text=True, timeout=600)

    cfg = json.loads(json.dumps(U.CONFIGS["A"]))
    cfg["layers"][2]["mixer"]["bias_rows"] = 7          # how many rows the random tables get (the default otherwise)
    cfg_file = tmp_path / "c.json"
    cfg_file.write_text(json.dumps(cfg))
    d = str(tmp_path / "m")
    r = rlis("random-weights", "--config", str(cfg_file), "--seed", "21", "--out", d)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = U.read_config(d), U.plain_weights(d)
    assert cfg["architecture"] == "Gavodra" and w["l2.mix.rel"].shape == (7, 6) and w["l0.mix.rel"].shape[1] == 4
    assert set(w) == set(U.tensor_shapes(cfg, [w[f"l{i}.mix.rel"].shape[0] for i in range(4)]))
    prompt = [5, 9, 200, 31, 7]
    r = rlis("generate", "--model", d, "--dtype", "f32", "--prompt-ids", ",".join(map(str, prompt)),
             "--max-tokens", "8", "--max-seq-len", "64", "--kv-cache-gb", "0.001", "--block-size", "8",
             "--max-num-seqs", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == plain_greedy(cfg, w, prompt, 8)

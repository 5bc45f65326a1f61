"""Lasapel on the GPU against the plain restatement: every kernel alone, every mixer alone in a
one-layer model, whole prompts against portions, single tokens and mixed batches in pools so small
that pages and state slots are used again, far keys and sinks made to stand out, long decoding, and
greedy generation through the entry point."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from tests import lasapel_util as U
from tests import replay_util as R
from tests.plain import lasapel_plain as P

pytestmark = pytest.mark.gpu

# A position's error is the root mean square, over the vocabulary, of the difference of its logits
# (which are about 1 in size).  float32: sums in another order than the plain float64 ones.  bfloat16:
# every product's inputs are rounded to 8 bits, and attention here is peaked, which amplifies it: over
# all positions the error is about 0.007, at the worst position about 0.03 with every kernel.
TOL = {"float32": 2e-5, "bfloat16": 0.045}
TOL_BETWEEN = {"float32": 1e-5, "bfloat16": 0.045}


def position_error(a, b):
    d = np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64)
    e = float(np.sqrt(np.mean(d * d)))
    return e if np.isfinite(e) else float("inf")


def dev(x, dtype=torch.float32):
    return torch.as_tensor(np.asarray(x)).to(device="cuda", dtype=dtype).contiguous()


def requests_for(cfg, lens, seed=1):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab"], size=n).tolist() for i, n in enumerate(lens)}


def plain_logits(model_dir, reqs):
    cfg, w = U.read_config(model_dir), U.plain_weights(model_dir)
    return {name: P.forward(cfg, w, toks) for name, toks in reqs.items()}


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


# ---- the kernels, one by one -------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [40, 96, 1000])
def test_post_norm_residual(dtype, hidden):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(hidden)
    T = 5
    sub, resid = dev(rng.standard_normal((T, hidden)), dtype), dev(rng.standard_normal((T, hidden)))
    wp, sc, b, wn = (dev(1 + 0.3 * rng.standard_normal(hidden)) for _ in range(4))
    y = sub.double().cpu().numpy() + b.double().cpu().numpy()
    want_resid = resid.double().cpu().numpy() + sc.double().cpu().numpy() * P.plain_norm(y, wp.double().cpu().numpy(), 1e-5)
    want_out = P.plain_norm(want_resid, wn.double().cpu().numpy(), 1e-6)
    out = torch.empty((T, hidden), dtype=dtype, device="cuda")
    ops.post_norm_residual(sub, resid, wp, 1e-5, sc, bias=b, w_next=wn, eps_next=1e-6, out=out)
    np.testing.assert_allclose(resid.cpu().numpy(), want_resid, rtol=0, atol=2e-6)       # float32 whatever the type
    np.testing.assert_allclose(out.float().cpu().numpy(), want_out, rtol=0, atol=2e-6 if dtype == torch.float32 else 2e-2)
    # without scale, bias and next norm
    resid2 = dev(rng.standard_normal((T, hidden)))
    want2 = resid2.double().cpu().numpy() + P.plain_norm(sub.double().cpu().numpy(), wp.double().cpu().numpy(), 1e-5)
    assert ops.post_norm_residual(sub, resid2, wp, 1e-5) is None
    np.testing.assert_allclose(resid2.cpu().numpy(), want2, rtol=0, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_act_norm_with_gate_and_bias_act(dtype):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(2)
    T, W = 7, 72
    wide = dev(rng.standard_normal((T, 3 * W)), dtype)
    x32 = dev(rng.standard_normal((T, W)) * 3)
    w = dev(1 + 0.3 * rng.standard_normal(W))
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    out = torch.empty((T, W), dtype=dtype, device="cuda")
    ops.act_norm(x32, w, 1e-5, out, gate=wide[:, 2 * W:])                   # float32 rows, gate a column slice
    g = wide[:, 2 * W:].double().cpu().numpy()
    want = P.plain_norm(x32.double().cpu().numpy(), w.double().cpu().numpy(), 1e-5) * P.sigmoid(g)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=0, atol=tol)
    ops.act_norm(wide[:, W:2 * W], w, 1e-5, out)                             # rows in the activation type, a slice
    want = P.plain_norm(wide[:, W:2 * W].double().cpu().numpy(), w.double().cpu().numpy(), 1e-5)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=0, atol=tol)
    b = dev(rng.standard_normal(W))
    xa = wide[:, :W].contiguous()
    got = ops.bias_act(xa, b, torch.empty_like(xa), "relu2")
    want = P.relu_squared(xa.double().cpu().numpy() + b.double().cpu().numpy())
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-6)
    got = ops.bias_act(xa, b, torch.empty_like(xa), "none")
    np.testing.assert_allclose(got.float().cpu().numpy(), xa.double().cpu().numpy() + b.double().cpu().numpy(),
                               rtol=2e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_head_linear_on_slices(dtype):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(4)
    T, H, K, N, extra = 70, 3, 24, 40, 8
    a = dev(rng.standard_normal((T, H, K + extra)), dtype)
    w = dev(rng.standard_normal((H, N, K)) / 5, dtype)
    out = torch.zeros((T, H, N + extra), dtype=torch.float32, device="cuda")
    ops.per_head_linear(a[:, :, :K], w, out[:, :, :N])
    want = np.einsum("thk,hnk->thn", a[:, :, :K].double().cpu().numpy(), w.double().cpu().numpy())
    np.testing.assert_allclose(out[:, :, :N].cpu().numpy(), want, rtol=0, atol=1e-4)
    assert float(out[:, :, N:].abs().max()) == 0.0                            # nothing written beside the slice


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot,dims", [(32, 8, 8), (10, 4, 2), (24, 16, 16)])
def test_latent_rows_are_normed_rotated_and_stored(dtype, rank, rot, dims):
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.parts.position import yarn_inverse_frequencies
    rng = np.random.default_rng(rank)
    rcfg = {"dims": dims, "base": 1000.0, "scaling": {"factor": 3.0, "original": 50, "fast": 6.0, "slow": 1.5}}
    f, mag = yarn_inverse_frequencies(dims, 1000.0, 3.0, 50, 6.0, 1.5)
    T, page, lead = 6, 4, 5
    positions = np.array([0, 1, 2, 700, 701, 33], dtype=np.int32)
    slots = np.array([8, 9, 10, 3, 0, 21], dtype=np.int32)
    z = dev(rng.standard_normal((T, lead + rank + rot)), dtype)
    w = dev(1 + 0.3 * rng.standard_normal(rank))
    cache = torch.zeros((6, 1, page, rank + rot), dtype=dtype, device="cuda")
    wq = dev(1 + 0.3 * rng.standard_normal(lead))
    cq = torch.empty((T, lead), dtype=dtype, device="cuda")
    ops.latent_kv_store(z[:, lead:], w, 1e-5, dev(f), dims, mag, dev(positions, torch.int32), dev(slots, torch.int32),
                        cache, rank, page, q_latent=z[:, :lead], q_weight=wq, q_out=cq)    # the leading columns as a query latent
    np.testing.assert_allclose(cq.float().cpu().numpy(),
                               P.plain_norm(z[:, :lead].double().cpu().numpy(), wq.double().cpu().numpy(), 1e-5),
                               rtol=0, atol=3e-5 if dtype == torch.float32 else 3e-2)
    zz = z[:, lead:].double().cpu().numpy()
    cos, sin = P.rotary_table(rcfg, 702)
    want = np.concatenate([P.plain_norm(zz[:, :rank], w.double().cpu().numpy(), 1e-5),
                           P.rotate(zz[:, rank:], cos[positions], sin[positions], dims)], axis=1)
    rows = cache.view(-1, rank + rot)[torch.as_tensor(slots, device="cuda").long()].float().cpu().numpy()
    np.testing.assert_allclose(rows, want, rtol=0, atol=3e-4 if dtype == torch.float32 else 3e-2)
    untouched = np.setdiff1d(np.arange(24), slots)
    assert float(cache.view(-1, rank + rot)[untouched].abs().max()) == 0.0
    # the query's rotated part, by the same rule, in float32
    H, d = 2, 6
    q = dev(rng.standard_normal((T, H * (d + rot))), dtype)
    qa = torch.zeros((T, H * (rank + rot)), dtype=torch.float32, device="cuda")
    ops.latent_q_rope(q, qa, dev(f), dims, mag, dev(positions, torch.int32), H, d, rot, rank)
    qq = q.double().cpu().numpy().reshape(T, H, d + rot)[..., d:]
    np.testing.assert_allclose(qa.view(T, H, rank + rot)[..., rank:].cpu().numpy(),
                               P.rotate(qq, cos[positions], sin[positions], dims), rtol=0, atol=3e-4)


def latent_step(ctx_positions, page, n_pages, rng):
    """One request whose tokens sit in shuffled pages; queries at `ctx_positions`."""
    table = rng.permutation(n_pages).astype(np.int32)
    return SimpleNamespace(block_tables=[dev(table[None, :], torch.int32)],
                           seq_of_token=dev(np.zeros(len(ctx_positions)), torch.int32),
                           positions=dev(ctx_positions, torch.int32)), table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_over_latents_far_keys_sinks_and_windows(dtype):
    """One key far back is made to carry almost all the weight; queries sit at the first positions,
    at page borders and far out; a window is checked one key inside and one outside."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(7)
    H, rank, rot, page, n_pages = 3, 24, 8, 8, 90
    dk, n_keys, far = rank + rot, 700, 5
    rows = rng.standard_normal((n_keys, dk)) * 0.3
    rows[far] = rng.standard_normal(dk) * 1.5
    q_pos = np.array([0, 1, far, 7, 8, 15, 16, 17, 31, 32, 63, 64, 300, 511, 512, 699], dtype=np.int32)
    qa = rng.standard_normal((len(q_pos), H, dk)) * 0.3
    qa[:, 1] = rows[far] * 3.0                                   # head 1 looks for the far key
    sinks = np.array([-1.0, 4.0, 30.0])
    step, table = latent_step(q_pos, page, n_pages, rng)
    cache = torch.zeros((n_pages, 1, page, dk), dtype=dtype, device="cuda")
    stored = dev(rows, dtype)
    for j in range(n_keys):
        cache[int(table[j // page]), 0, j % page] = stored[j]
    kk = stored.double().cpu().numpy()

    def plain(window, use_sinks):
        out = np.zeros((len(q_pos), H, rank))
        for i, p in enumerate(q_pos):
            lo = max(0, p - window + 1) if window else 0
            for h in range(H):
                s = (kk[lo:p + 1] @ qa[i, h]) * 0.4
                m = max(s.max(), sinks[h]) if use_sinks else s.max()
                e = np.exp(s - m)
                out[i, h] = e @ kk[lo:p + 1, :rank] / (e.sum() + (np.exp(sinks[h] - m) if use_sinks else 0.0))
        return out

    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for window, use_sinks in ((0, True), (0, False), (far + 1, True), (64, False)):
        out = torch.empty((len(q_pos), H * rank), dtype=dtype, device="cuda")
        ops.attention_latent(dev(qa.reshape(len(q_pos), -1)), cache, out, step, 0, H, rank, page, 0.4,
                             dev(sinks) if use_sinks else None, window)
        np.testing.assert_allclose(out.float().cpu().numpy().reshape(len(q_pos), H, rank), plain(window, use_sinks),
                                   rtol=0, atol=tol, err_msg=f"window {window} sinks {use_sinks}")
    # the far key matters: head 1 at the last position puts most of its weight there when the sink is left out
    w_far = plain(0, False)[-1, 1]
    assert np.abs(w_far - kk[far, :rank]).max() < 0.05
    # and a window that ends one key after it sees something else entirely
    a, b = plain(700 - far, False)[-1, 1], plain(700 - far - 1, False)[-1, 1]
    assert np.abs(a - b).max() > 0.3


class FakeStep:
    """The arrays of a step that the attention kernels read, for requests (tokens cached before, tokens now)."""

    def __init__(self, reqs, tables, tile=64):
        lens = [n for _, n in reqs]
        cu = np.cumsum([0] + lens)
        self.n_tokens, self.n_seqs = int(cu[-1]), len(reqs)
        self.block_tables = [dev(tables, torch.int32)]
        self.positions = dev(np.concatenate([np.arange(s, s + n) for s, n in reqs]), torch.int32)
        self.seq_of_token = dev(np.concatenate([np.full(n, b) for b, (_, n) in enumerate(reqs)]), torch.int32)
        self.cu_seqlens, self.ctx_lens = dev(cu, torch.int32), dev([s + n for s, n in reqs], torch.int32)
        dec = [b for b, (_, n) in enumerate(reqs) if n == 1]
        self.n_decode = len(dec)
        self.dec_seqs, self.dec_rows = dev(dec, torch.int32), dev([cu[b] for b in dec], torch.int32)
        self.max_decode_ctx = max([reqs[b][0] + 1 for b in dec], default=0)
        tiles = [(b, t0) for b, (_, n) in enumerate(reqs) if n > 1 for t0 in range(0, n, tile)]
        self.n_prefill_tiles, self.n_prefill_tokens = len(tiles), sum(n for _, n in reqs if n > 1)
        self.prefill_tiles = dev(np.asarray(tiles).reshape(-1, 2), torch.int32) if tiles else None
        self._bufs = {}

    def buffer(self, name, shape, dtype):
        return self._bufs.setdefault((name, tuple(shape)), torch.empty(shape, dtype=dtype, device="cuda"))


@pytest.mark.parametrize("H,rank,rot", [(5, 64, 32), (18, 128, 16), (16, 256, 64)])
@pytest.mark.parametrize("window,use_sinks", [(0, True), (0, False), (100, True)])
def test_tensor_core_attention_over_latents(H, rank, rot, window, use_sinks):
    """Portions that start in the middle of a page and of a tile, single tokens at short, page-border
    and long contexts (cut into pieces), one far key that carries the weight of a head."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(H)
    dk, page, far = rank + rot, 16, 3
    reqs = [(0, 1), (0, 70), (37, 129), (15, 1), (16, 1), (63, 1), (64, 1), (1500, 1), (700, 2), (255, 1)]
    n_pages = sum(-(-(s + n) // page) for s, n in reqs)
    perm = rng.permutation(n_pages)
    tables = np.full((len(reqs), max(-(-(s + n) // page) for s, n in reqs)), -1, dtype=np.int32)
    cache = torch.zeros((n_pages, 1, page, dk), dtype=torch.bfloat16, device="cuda")
    rows, k = [], 0
    for b, (s, n) in enumerate(reqs):
        r = rng.standard_normal((s + n, dk)) * 0.4
        if s + n > far:
            r[far] = rng.standard_normal(dk)
        r = dev(r, torch.bfloat16)
        rows.append(r.double().cpu().numpy())
        for j in range(-(-(s + n) // page)):
            tables[b, j] = perm[k]
            chunk = r[j * page:(j + 1) * page]
            cache[int(perm[k]), 0, :chunk.shape[0]] = chunk
            k += 1
    step = FakeStep(reqs, tables)
    qa = rng.standard_normal((step.n_tokens, H, dk)) * 0.4
    sinks = rng.standard_normal(H) * 2
    want = np.zeros((step.n_tokens, H, rank))
    t = 0
    for b, (s, n) in enumerate(reqs):
        qa[t:t + n, 1] = rows[b][min(far, s + n - 1)] * 1.5
        for i in range(n):
            p = s + i
            lo = max(0, p - window + 1) if window else 0
            qq = dev(qa[t], torch.bfloat16).double().cpu().numpy()          # the kernel rounds queries once
            for h in range(H):
                sc = (rows[b][lo:p + 1] @ qq[h]) * 0.3
                m = max(sc.max(), sinks[h]) if use_sinks else sc.max()
                e = np.exp(sc - m)
                want[t, h] = e @ rows[b][lo:p + 1, :rank] / (e.sum() + (np.exp(sinks[h] - m) if use_sinks else 0.0))
            t += 1
    ops.launches_by_kernel.clear()
    out = torch.full((step.n_tokens, H * rank), 9.0, dtype=torch.bfloat16, device="cuda")
    ops.attention_latent(dev(qa.reshape(step.n_tokens, -1)), cache, out, step, 0, H, rank, page, 0.3,
                         dev(sinks) if use_sinks else None, window)
    assert ops.launches_by_kernel.get("attention_latent.decode.mma.split") and ops.launches_by_kernel.get("attention_latent.prefill.mma")
    np.testing.assert_allclose(out.float().cpu().numpy().reshape(step.n_tokens, H, rank), want, rtol=0, atol=2e-2)
    # queries that are bfloat16 already (as the mixer hands them over) are copied as they are
    assert ops.latent_attention_queries_dtype(step, torch.bfloat16, dk, rank) == torch.bfloat16
    out.fill_(9.0)
    ops.attention_latent(dev(qa.reshape(step.n_tokens, -1), torch.bfloat16), cache, out, step, 0, H, rank, page, 0.3,
                         dev(sinks) if use_sinks else None, window)
    np.testing.assert_allclose(out.float().cpu().numpy().reshape(step.n_tokens, H, rank), want, rtol=0, atol=2e-2)
    # short contexts alone are not cut into pieces
    short = [(15, 1), (16, 1), (0, 1)]
    step2 = FakeStep(short, tables[[3, 4, 0]])
    idx = [int(np.cumsum([0] + [n for _, n in reqs])[b]) for b in (3, 4, 0)]
    out2 = torch.empty((3, H * rank), dtype=torch.bfloat16, device="cuda")
    ops.attention_latent(dev(qa[idx].reshape(3, -1)), cache, out2, step2, 0, H, rank, page, 0.3,
                         dev(sinks) if use_sinks else None, window)
    assert ops.launches_by_kernel.get("attention_latent.decode.mma")
    np.testing.assert_allclose(out2.float().cpu().numpy().reshape(3, H, rank), want[idx], rtol=0, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dv", [(2, 24, 40), (1, 8, 48), (3, 128, 16), (2, 200, 8), (1, 320, 24)])
def test_decayed_recurrence_carries_its_state(dtype, H, d, dv):
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(d)
    decay = np.array([0.9, 1.0, 0.4][:H])
    lead, width = 3, 2 * H * d + H * dv
    lens = {0: [5, 1, 1, 19, 2], 1: [1, 70, 1, 1, 4]}             # two requests in portions (one step is long enough for
    bufs = {}                                                     # the pass that applies silu once for all CTAs)
    toks = {b: rng.standard_normal((sum(l), lead + width)) for b, l in lens.items()}
    state = torch.full((4, H, dv, d), 7.0, device="cuda")           # S is kept transposed        # slots hold leftovers of earlier requests
    slots, done, got = {0: 2, 1: 0}, {0: 0, 1: 0}, {0: [], 1: []}
    for k in range(5):
        order = [0, 1] if k % 2 == 0 else [1, 0]
        rows = [toks[b][done[b]:done[b] + lens[b][k]] for b in order]
        proj = dev(np.concatenate(rows), dtype)
        cu = np.cumsum([0] + [len(r) for r in rows]).astype(np.int32)
        step = SimpleNamespace(cu_seqlens=dev(cu, torch.int32), n_seqs=2,
                               buffer=lambda name, shape, dt: bufs.setdefault((name, tuple(shape)), torch.empty(shape, dtype=dt, device="cuda")),
                               ctx_lens=dev([done[b] + lens[b][k] for b in order], torch.int32),
                               state_slots=dev([slots[b] for b in order], torch.int32))
        out = torch.empty((proj.shape[0], H * dv), dtype=torch.float32, device="cuda")
        # (the pass needs q to start at column 0: every other step gets such a view)
        view, off = (proj, lead) if k % 2 else (proj[:, lead:], 0)
        if off == 0:
            view = view.contiguous()
        ops.lightning_scan(view, off, off + H * d, off + 2 * H * d, out, state, dev(decay), step, H, d, dv)
        o = out.cpu().numpy()
        for i, b in enumerate(order):
            got[b].append(o[cu[i]:cu[i + 1]])
            done[b] += lens[b][k]
    for b in (0, 1):
        x = dev(toks[b], dtype).double().cpu().numpy()[:, lead:]
        q, k_, v = (P.silu(x[:, a:z]).reshape(-1, H, n) for a, z, n in
                    ((0, H * d, d), (H * d, 2 * H * d, d), (2 * H * d, width, dv)))
        want = np.zeros((x.shape[0], H, dv))
        for h in range(H):
            S = np.zeros((d, dv))
            for t in range(x.shape[0]):
                S = decay[h] * S + np.outer(k_[t, h], v[t, h])
                want[t, h] = S.T @ q[t, h]
        np.testing.assert_allclose(np.concatenate(got[b]).reshape(-1, H, dv), want, rtol=2e-5, atol=2e-4)
        # the state left in the slot is the last S, in float32
        np.testing.assert_allclose(state[slots[b], H - 1].cpu().numpy(), S.T, rtol=2e-5, atol=2e-4)
    assert float((state[1] - 7.0).abs().max()) == 0.0 and float((state[3] - 7.0).abs().max()) == 0.0


# ---- whole models ------------------------------------------------------------------------------

ALONE = {
    "lightning_only": {"architecture": "Lasapel", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "layers": [
        U.layer("lightning", {"heads": 3, "dim": 16, "vdim": 8, "decay": [0.95, 0.6, 0.8]})]},
    "latent_only": {"architecture": "Lasapel", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "layers": [
        U.layer("latent_attention", U.latent(2, 8, 16, 12, 24, 16, 0.35, scaling=(8.0, 16, 4.0, 1.0)))]},
    "latent_with_ff": {"architecture": "Lasapel", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "layers": [
        U.layer("latent_attention", U.latent(2, 8, 16, 12, 24, 16, 0.35), 56)]},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mixer_alone(model_root, which, dtype):
    d = U.make_dir(model_root, which, ALONE[which], seed=11)
    reqs = requests_for(ALONE[which], [1, 2, 37, 90])
    ref = plain_logits(d, reqs)
    for fam, steps in (("whole", R.whole_trace(reqs)), ("decode", R.decode_trace(reqs, tail=20)),
                       ("chunks", R.chunk_trace(reqs, seed=2))):
        s = session(d, dtype, R.live_token_peak(steps), 8)
        worst, where = worst_difference(R.collect(s.step, steps), ref)
        assert worst <= TOL[dtype], f"{which} {dtype} {fam}: {worst} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,page,lens", [("X", 16, [1, 50, 97, 200, 64, 17, 2]), ("X", 8, [130, 33, 2, 71, 40]),
                                             ("Y", 16, [3, 150, 40, 2, 129, 1]), ("Y", 32, [260, 31, 5, 90]),
                                             ("Z", 16, [1, 70, 333, 2, 129, 64, 65]), ("Z", 8, [200, 31, 5, 640])])
def test_all_ways_of_cutting_give_the_plain_logits(model_root, which, page, lens, dtype):
    from rust_llm_inference_server_b200 import ops
    ops.launches_by_kernel.clear()
    d = U.make_dir(model_root, which)
    reqs = requests_for(U.CONFIGS[which], lens, seed=page)
    ref = plain_logits(d, reqs)
    families = {
        "whole": (R.whole_trace(reqs), 4),
        "decode": (R.decode_trace(reqs, tail=40), 4),
        "chunks": (R.chunk_trace(reqs, seed=3), 4),
        "mixed": (R.mixed_trace(reqs, seed=4), 4),
        "mixed2": (R.mixed_trace(dict(reversed(list(reqs.items()))), seed=5, max_live=2), 2),   # two state slots for all
    }
    results = {}
    for fam, (steps, live) in families.items():
        s = session(d, dtype, R.live_token_peak(steps, max(64, page)), page, max_live=live)
        for state in s.storage.states:                       # whatever a slot held before must not matter
            if state is not None:
                state.fill_(3.0)
        results[fam] = R.collect(s.step, steps)
        assert s.cache.check_invariants() == ""
        assert s.cache.num_free_pages(0) == s.cache.group(0).num_pages, fam
        assert s.cache.num_free_state_slots() == live, fam
        worst, where = worst_difference(results[fam], ref)
        assert worst <= TOL[dtype], f"{which} {dtype} {fam} vs plain: {worst} at {where}"
    for fam in ("decode", "chunks", "mixed", "mixed2"):
        worst = max(position_error(v, results["whole"][k]) for k, v in results[fam].items())
        assert worst <= TOL_BETWEEN[dtype], f"{which} {dtype}: {fam} differs from whole by {worst}"
    fast = dtype == "bfloat16" and which == "Z"
    reads_other = any("kv_from" in l["mixer"] for l in U.CONFIGS[which]["layers"])
    for k in (("attention_latent.decode.mma", "attention_latent.prefill.mma") if fast else ("attention_latent",)) + \
            (("act_norm",) if reads_other else ()) + \
            ("lightning_scan", "lightning_scan.silu_pass", "latent_kv_store.q_norm", "latent_q_rope", "post_norm_residual",
             "post_norm_residual.next", "act_norm.gate", "bias_act.relu2"):
        assert ops.launches_by_kernel.get(k), f"never launched {k}; launched {sorted(ops.launches_by_kernel)}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_pages(model_root, dtype):
    d = U.make_dir(model_root, "Y")
    reqs = requests_for(U.CONFIGS["Y"], [230], seed=9)
    ref = plain_logits(d, reqs)
    steps = R.decode_trace(reqs, tail=200)
    s = session(d, dtype, R.live_token_peak(steps), 8)
    worst, where = worst_difference(R.collect(s.step, steps), ref)
    assert worst <= TOL[dtype], f"{worst} at {where}"


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(P.forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(model_root, dtype):
    """Prompts of unequal length batched by the scheduler, portions of 16 tokens, decode steps from
    CUDA graphs and launched ahead; two seats, so the later prompts take over state slots."""
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    d = U.make_dir(model_root, "X")
    cfg, w = U.read_config(d), U.plain_weights(d)
    prompts = list(requests_for(cfg, [1, 9, 40, 23, 3], seed=12).values())
    llm = LLM(d, dtype=dtype, max_seq_len=128, num_blocks=40, block_size=8, max_num_seqs=2, max_batched_tokens=16)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12))
    for p, o in zip(prompts, outs):
        want = plain_greedy(cfg, w, p, 12)
        assert o.finish_reason == "length" and len(o.token_ids) == 12
        if o.token_ids != want:
            i = next(k for k, (a, b) in enumerate(zip(o.token_ids, want)) if a != b)
            lg = P.forward(cfg, w, p + want[:i])[-1]
            gap = lg[want[i]] - lg[o.token_ids[i]]
            assert dtype == "bfloat16" and gap < 0.1, f"parted at token {i} with a gap of {gap}"
    assert llm.engine.cache.check_invariants() == "" if hasattr(llm.engine, "cache") else True


def test_command_line_serves_the_design(tmp_path):
    """random-weights, generate and perplexity of the command line with a Lasapel folder."""
    import json
    import math
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def rlis(*args):
        return subprocess.run([sys.executable, os.path.join(root, "bin", "rlis"), *args], capture_output=True,
                              text=True, timeout=600)

    cfg_file = tmp_path / "c.json"
    cfg_file.write_text(json.dumps(U.CONFIGS["X"]))
    d = str(tmp_path / "m")
    r = rlis("random-weights", "--config", str(cfg_file), "--seed", "21", "--out", d)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = U.read_config(d), U.plain_weights(d)
    assert cfg["architecture"] == "Lasapel" and set(w) == set(U.tensor_shapes(cfg))
    prompt = [5, 9, 200, 31, 7]
    r = rlis("generate", "--model", d, "--dtype", "f32", "--prompt-ids", ",".join(map(str, prompt)),
             "--max-tokens", "8", "--max-seq-len", "64", "--kv-cache-gb", "0.001", "--block-size", "8",
             "--max-num-seqs", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == plain_greedy(cfg, w, prompt, 8)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], size=2 * 32 + 5).tolist()
    f = tmp_path / "toks.txt"
    f.write_text(" ".join(map(str, toks)))
    r = rlis("perplexity", "--model", d, "--dtype", "f32", "--token-file", str(f), "--ctx", "32")
    assert r.returncode == 0, r.stderr[-2000:]
    rep = json.loads(r.stdout.strip().splitlines()[-1])
    nll = []
    for wdw in range(2):
        chunk = toks[wdw * 32:(wdw + 1) * 32]
        chunk[0] = toks[0]
        lg = P.forward(cfg, w, chunk)
        lp = lg - np.log(np.exp(lg - lg.max(-1, keepdims=True)).sum(-1, keepdims=True)) - lg.max(-1, keepdims=True)
        nll += [-float(lp[i, chunk[i + 1]]) for i in range(16, 31)]
    assert rep["windows"] == 2 and abs(rep["mean_nll"] - np.mean(nll)) < 1e-4
    assert abs(rep["ppl"] - math.exp(np.mean(nll))) < 1e-2

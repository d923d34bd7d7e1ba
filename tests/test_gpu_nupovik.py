"""Nupovik family on the GPU against the float64 oracle (oracle/nupovik_oracle.py): every mechanism alone
through its operator, then whole models through the serving path (ScheduleBatch → worker → kernels, decode
through the captured CUDA graphs) under every way of cutting and batching the same tokens, then greedy
generation through the semi-PD engine."""
import math

import pytest
import torch

from oracle import nupovik_oracle as N
from tests import nupovik_helpers as C
from tests import rimidra_helpers as H

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _close(got, want, dtype, what="", tol32=2e-5):
    tol = tol32 if dtype == torch.float32 else 3e-2
    err = (got.double().cpu() - want.double().cpu()).abs().max().item()
    ref = want.double().abs().max().item() + 1e-9
    assert err <= tol * ref, f"{what}: max abs err {err:.3e} vs ref max {ref:.3e}"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def i64(x):
    return torch.tensor(x, dtype=torch.int64, device=DEV)


# =================================================================================================
# mechanisms alone
# =================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [36, 64, 7])
def test_embedding_with_positions(dtype, width):
    from semi_pd_b200 import ops
    from semi_pd_b200.nupovik import _sinusoid_frequencies
    g = torch.Generator().manual_seed(width)
    table = torch.randn(20, width, generator=g).to(DT[dtype])
    pos = [0, 1, 2, 63, 64, 1000, 4097, 70001, 1 << 20]
    ids = torch.randint(0, 20, (len(pos),), generator=g)
    hi, lo = _sinusoid_frequencies(width, DEV)
    got = ops.embed_sincos(table.to(DEV), ids.to(DEV), i64(pos), hi, lo)
    want = table.double()[ids]
    pv = N.position_vector(pos, width)
    assert (got.double().cpu() - (want + pv)).abs().max().item() < 3e-7 * 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_norms_of_one_row(dtype):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(1)
    for dim in (36, 256, 1000):
        x = torch.randn(5, dim, generator=g) * 3
        a, b = torch.randn(5, dim, generator=g).to(dt), torch.randn(5, dim, generator=g).to(dt)
        w1, w2 = (1 + 0.2 * torch.randn(dim, generator=g)).to(dt), torch.randn(dim, generator=g).to(dt)
        xd = x.to(DEV)
        o1, o2 = ops.residual_rmsnorm2(xd, w1.to(DEV), w2.to(DEV), 1e-6, a=a.to(DEV), b=b.to(DEV))
        ref = x.double() + (a.double() + b.double())
        _close(xd, ref, torch.float32, "residual")
        _close(o1, N.rms_norm(ref, w1, 1e-6), dt, "first norm")
        _close(o2, N.rms_norm(ref, w2, 1e-6), dt, "second norm")
        o1, o2 = ops.residual_rmsnorm2(xd, w1.to(DEV), None, 1e-6)
        assert o2 is None
        _close(o1, N.rms_norm(ref, w1, 1e-6), dt, "norm only")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_operators(dtype):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(7, 52, generator=g) * 2).to(dt)
    xd = x.double()
    for act, fn in (("relu2", N.relu_sq), ("tanh", torch.tanh), ("silu", N.silu)):
        _close(ops.activation(x.to(DEV), act), fn(xd), dt, act)
    _close(ops.activation(x.to(DEV)[:, 4:20], "relu2"), N.relu_sq(xd[:, 4:20]), dt, "strided view")
    # per-head sigmoid gate, gate columns inside a wider row
    o, gate = (torch.randn(7, 3 * 10, generator=g)).to(dt), torch.randn(7, 8, generator=g).to(dt)
    got = ops.head_gate_sigmoid(o.to(DEV), gate.to(DEV)[:, 2:5], 3, 10)
    _close(got, (o.double().view(7, 3, 10) * torch.sigmoid(gate.double()[:, 2:5]).unsqueeze(-1)).reshape(7, 30), dt, "head gate")
    # per-head norm with a weight shared by the heads / a weight per channel, times a SiLU gate
    of = torch.randn(7, 3 * 10, generator=g) * 4
    gt = torch.randn(7, 30, generator=g).to(dt)
    for wn in (10, 30):
        w = (1 + 0.3 * torch.randn(wn, generator=g)).to(dt)
        got = ops.headnorm_gate(of.to(DEV), gt.to(DEV), 3, 10, 1e-5, weight=w.to(DEV))
        want = N.rms_norm(of.double().view(7, 3, 10), None, 1e-5) * w.double().view(-1, 10) * N.silu(gt.double()).view(7, 3, 10)
        _close(got, want.reshape(7, 30), dt, f"head norm, weight of {wn}")
    # norm of a slice written into pool rows
    pool = torch.zeros(12, 1, 20, dtype=dt, device=DEV)
    wide = (torch.randn(4, 44, generator=g) * 2).to(dt)
    w = (1 + 0.3 * torch.randn(20, generator=g)).to(dt)
    out = ops.rmsnorm_store(wide.to(DEV)[:, 8:28], w.to(DEV), 1e-6, pool=pool.view(12, 20), loc=i64([3, 11, 0, 7]), want_out=True)
    want = N.rms_norm(wide.double()[:, 8:28], w, 1e-6)
    _close(out, want, dt, "normed slice")
    _close(pool.view(12, 20)[[3, 11, 0, 7]], want, dt, "pool rows")
    assert pool.view(12, 20)[[1, 2, 4, 5, 6, 8, 9, 10]].abs().max().item() == 0
    # two fp32 streams as one operand; scale in place
    a, b = torch.randn(3, 36, generator=g), torch.randn(3, 36, generator=g)
    _close(ops.cast_concat(a.to(DEV), b.to(DEV), dt), torch.cat([a, b], -1), dt, "concat")
    z = torch.randn(5, 9, generator=g).to(DEV)
    want = z.double().cpu() * 0.37
    _close(ops.scale_f32_(z, 0.37), want, torch.float32, "scale")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(5, 3, 10, 12), (70, 4, 64, 128), (130, 2, 128, 64)])
def test_block_diagonal_products(dtype, shape):
    """Per-head products of the absorbed latent attention, shapes on and off the tensor-core tiles."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    M, G, k, n = shape
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, G * k + 8, generator=g).to(dt)
    w = (torch.randn(G * n, k, generator=g) / math.sqrt(k)).to(dt)
    got = ops.linear_block_diag_any(x.to(DEV)[:, : G * k], w.to(DEV), G, k, n)
    want = torch.einsum("mgk,gnk->mgn", x.double()[:, : G * k].view(M, G, k), w.double().view(G, n, k)).reshape(M, G * n)
    _close(got, want, dt, f"block diagonal {shape}")


@pytest.mark.parametrize("experts,top,groups,keep", [(20, 4, 5, 3), (8, 2, 4, 2), (6, 3, 3, 2), (2, 1, 1, 1), (12, 5, 12, 7),
                                                     (64, 8, 8, 4), (9, 3, 1, 1)])
def test_grouped_routing(experts, top, groups, keep):
    """Choice by score + correction inside the kept groups (negative choice scores included), weights from the
    scores alone, renormalised."""
    from semi_pd_b200 import ops
    g = torch.Generator().manual_seed(experts * 31 + top)
    z = torch.randn(200, experts + 3, generator=g) * 2
    corr = torch.randn(experts, generator=g) * 1.5 - 1.0  # mostly negative choice scores
    ids, w = ops.moe_route_scores(z.to(DEV)[:, :experts], experts, top, "sigmoid", renormalize=True,
                                  correction=corr.to(DEV), num_groups=groups, keep_groups=keep)
    r = {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}
    want_ids, want_w = N.route_logits(z.double()[:, :experts], corr.double(), r)
    got = {(t, int(e)): float(x) for t in range(200) for e, x in zip(ids[t].cpu(), w[t].cpu())}
    for t in range(200):
        assert sorted(int(e) for e in ids[t].cpu()) == sorted(int(e) for e in want_ids[t]), f"token {t}"
        for e, x in zip(want_ids[t], want_w[t]):
            assert abs(got[(t, int(e))] - float(x)) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,rank", [(5, 128), (16, 64), (3, 24), (20, 32), (40, 64), (2, 320)])
def test_attention_over_latent_pool(dtype, heads, rank):
    """Every query head against ONE latent row per token that serves as key and as value (one buffer): requests
    of unequal length whose slots are interleaved in the pool, decoded in one launch and extended in portions;
    in the long request one far key is made to win a head's softmax, so a missed key shows."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(heads * 100 + rank)
    lens = [700, 129, 1, 64, 257]
    scale = 0.25
    total = sum(lens)
    perm = (torch.randperm(total, generator=g) + 1).tolist()
    pool = torch.zeros(total + 1, 1, rank, dtype=dt)
    r2t = torch.zeros(len(lens) + 1, max(lens) + 8, dtype=torch.int32)
    lat, qs, at = [], [], 0
    for i, L in enumerate(lens):
        c = torch.randn(L, rank, generator=g).to(dt)
        q = (torch.randn(L, heads * rank, generator=g) * 0.5).to(dt)
        if L > 600:  # head 1 of the last queries looks at key 5, far back
            c[5] = (4.0 * c[5] / c[5].float().norm()).to(dt)
            q[-40:, rank:2 * rank] = (8.0 * c[5].float()).to(dt)
        slots = perm[at:at + L]
        at += L
        pool[slots, 0] = c
        r2t[i, :L] = torch.tensor(slots, dtype=torch.int32)
        lat.append(c)
        qs.append(q)

    def want(i, lo, hi):
        c = lat[i].double()
        q = qs[i].double()[lo:hi].view(hi - lo, heads, rank)
        s = torch.einsum("thd,jd->thj", q, c) * scale
        j = torch.arange(c.shape[0]).view(1, 1, -1)
        s = s.masked_fill(j > torch.arange(lo, hi).view(-1, 1, 1), -math.inf)
        return torch.einsum("thj,jd->thd", torch.softmax(s, -1), c).reshape(hi - lo, heads * rank)

    poold, r2d = pool.to(DEV), r2t.to(DEV)
    kw = dict(num_q_heads=heads, num_kv_heads=1, head_dim=rank, v_dim=rank, sm_scale=scale)
    rpi = i64(list(range(len(lens))))
    # decode: every request's last position in one launch
    q = torch.stack([qs[i][-1] for i in range(len(lens))]).to(DEV)
    got = ops.attn_general(q, poold, poold, r2d, rpi, seq_lens=i64(lens), **kw)
    _close(got, torch.cat([want(i, L - 1, L) for i, L in enumerate(lens)]), dt, "decode")
    # extend: the last n positions of every request as one ragged batch (n = 1 .. 40)
    ns = [40, 2, 1, 17, 33]
    q = torch.cat([qs[i][L - n:] for i, (L, n) in enumerate(zip(lens, ns))]).to(DEV)
    starts = [sum(ns[:i]) for i in range(len(ns))]
    got = ops.attn_general(q, poold, poold, r2d, rpi, prefix_lens=i32([L - n for L, n in zip(lens, ns)]),
                           extend_lens=i32(ns), extend_start_loc=i32(starts), max_extend_len=max(ns), **kw)
    ref = torch.cat([want(i, L - n, L) for i, (L, n) in enumerate(zip(lens, ns))])
    _close(got, ref, dt, "extend")
    far = want(0, lens[0] - 1, lens[0])[0, rank:2 * rank]
    assert (far - lat[0][5].double()).abs().max() < 0.05 * lat[0][5].double().abs().max(), "the far key does not win"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_shift(dtype):
    """Portions of unequal requests, then decoding with a padded row; a slot used again starts from zeros."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(5)
    W, n_mix, T = 40, 5, 75
    mu = torch.rand(n_mix, W, generator=g).to(dt)
    seqs = [torch.randn(T, W, generator=g).to(dt) for _ in range(2)]
    want = [N.token_shift(s.double(), torch.zeros(W, dtype=torch.float64), mu.double()) for s in seqs]
    state = torch.full((6, W), 9.0, device=DEV)  # stale content that position 0 must ignore
    rpi = i64([3, 1])
    at = [0, 0]
    for n0, n1 in ((1, 2), (33, 2), (2, 40), (1, 1)):
        h = torch.cat([seqs[0][at[0]:at[0] + n0], seqs[1][at[1]:at[1] + n1]]).to(DEV)
        out = ops.token_shift_mix(h, mu.to(DEV), state, rpi, prefix_lens=i32(at), extend_lens=i32([n0, n1]),
                                  extend_start_loc=i32([0, n0]), max_extend_len=max(n0, n1))
        ref = torch.cat([want[0][:, at[0]:at[0] + n0], want[1][:, at[1]:at[1] + n1]], 1)
        _close(out, ref, dt, f"portions {(n0, n1)}")
        at = [at[0] + n0, at[1] + n1]
    before = state[4].clone()
    while max(at) < T:
        h = torch.cat([seqs[0][at[0]:at[0] + 1], seqs[1][at[1]:at[1] + 1], seqs[0][:1]]).to(DEV)
        out = ops.token_shift_mix(h, mu.to(DEV), state, i64([3, 1, 4]), seq_lens=i64([at[0] + 1, at[1] + 1, 1]),
                                  out_cache_loc=i64([5, 6, 0]))
        _close(out[:, :2], torch.cat([want[0][:, at[0]:at[0] + 1], want[1][:, at[1]:at[1] + 1]], 1), dt, f"decode {at}")
        at = [at[0] + 1, at[1] + 1]
    assert torch.equal(state[4], before)
    _close(state[3], seqs[0][at[0] - 1], dt, "kept row")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("form", ["sigmoid_pow", "double_exp"])
@pytest.mark.parametrize("shape", [(2, 16, 16), (1, 8, 40), (3, 64, 32), (1, 100, 12), (2, 160, 64)])
def test_gated_recurrence(dtype, form, shape):
    """Both forms: portions of two unequal requests against the token-by-token recurrence, then decoding with a
    padded row; a decay close to 1 keeps the first tokens in the state."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    H_, dk, dv = shape
    T = 70
    g = torch.Generator().manual_seed(dk * 7 + dv)
    tau, q_scale = 4.0, dk ** -0.5 if form == "sigmoid_pow" else 1.0
    bias = (torch.randn(H_ * dk, generator=g) + (4.0 if form == "sigmoid_pow" else -4.0))
    u = torch.randn(H_ * dk, generator=g) * 0.5 if form == "double_exp" else None
    seqs = []
    for _ in range(2):
        q, k, z = (torch.randn(T, H_ * dk, generator=g).to(dt) for _ in range(3))
        v = torch.randn(T, H_ * dv, generator=g).to(dt)
        zz = z.double() + bias.double()
        w = N.sigmoid_pow_decay(zz, tau) if form == "sigmoid_pow" else N.double_exp_decay(zz)
        S0 = torch.zeros(H_, dk, dv, dtype=torch.float64)
        args = (q.double().view(T, H_, dk) * q_scale, k.double().view(T, H_, dk), v.double().view(T, H_, dv), w.view(T, H_, dk))
        o, S = N.decay_recurrence(*args, S0) if form == "sigmoid_pow" else \
            N.bonus_recurrence(*args, u.double().view(H_, dk), S0)
        seqs.append((q, k, v, z, o.reshape(T, H_ * dv), S))
    state = torch.full((6, H_, dk, dv), 5.0, device=DEV)
    kw = dict(num_heads=H_, head_dim=dk, v_dim=dv, form=form, q_scale=q_scale, tau=tau, z_bias=bias.to(DEV),
              bonus=u.to(DEV) if u is not None else None)
    at = [0, 0]
    for n0, n1 in ((1, 2), (17, 2), (2, 33), (16, 1)):
        parts = [(at[0], n0), (at[1], n1)]
        cat = lambda j: torch.cat([seqs[r][j][a:a + n] for r, (a, n) in enumerate(parts)]).to(DEV)
        o = ops.gated_recurrence(cat(0), cat(1), cat(2), cat(3), state, i64([3, 1]), prefix_lens=i32(at),
                                 extend_lens=i32([n0, n1]), extend_start_loc=i32([0, n0]), **kw)
        _close(o, torch.cat([seqs[r][4][a:a + n] for r, (a, n) in enumerate(parts)]), dt, f"portions {parts}", tol32=5e-5)
        at = [at[0] + n0, at[1] + n1]
    before = state[4].clone()
    while max(at) < T:
        rows = [(0, at[0]), (1, at[1])]
        cat = lambda j: torch.cat([seqs[r][j][a:a + 1] for r, a in rows] + [seqs[0][j][:1]]).to(DEV)
        o = ops.gated_recurrence(cat(0), cat(1), cat(2), cat(3), state, i64([3, 1, 4]),
                                 seq_lens=i64([at[0] + 1, at[1] + 1, 1]), out_cache_loc=i64([7, 9, 0]), **kw)
        _close(o[:2], torch.cat([seqs[r][4][a:a + 1] for r, a in rows]), dt, f"decode {rows}", tol32=5e-5)
        at = [at[0] + 1, at[1] + 1]
    assert torch.equal(state[4], before)
    _close(state[1], seqs[1][5], dt, "final state", tol32=5e-5)


# =================================================================================================
# whole models through the serving path
# =================================================================================================
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, make in C.CONFIGS.items():
        cfg = make()
        weights = N.make_weights(cfg, seed=C.SEEDS[name], low_rank=8 if name != "ones" else 5, slow_decay=name == "far")
        folder = H.write_model(tmp_path_factory.mktemp(name), cfg, weights)
        out[name] = (cfg, weights, folder)
    return out


_oracle_cache = {}


def _oracle(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _oracle_cache:
        cfg, weights, _ = models[name]
        _oracle_cache[key] = N.forward(cfg, weights, list(tokens))
    return _oracle_cache[key]


def _check(got, want, dtype, what):
    err = H.rel_err(got, want)
    if dtype == "float32":
        assert err.max().item() < H.TOL[dtype], f"{what}: worst relative error {err.max().item():.3e} at row {int(err.argmax())}"
    else:  # 16-bit: a routing decision on a near tie may differ from float64 for a few tokens
        assert err.median().item() < H.TOL[dtype] / 2, f"{what}: median {err.median().item():.3e}"
        assert (err > H.TOL[dtype]).float().mean().item() <= 0.05, f"{what}: {(err > H.TOL[dtype]).sum()} rows off"


def test_config_reader_and_layer_runs(models):
    from semi_pd_b200.configs import get_model_config
    for name, (cfg, _, folder) in models.items():
        mc = get_model_config(folder)
        runs = N.layer_runs(cfg)
        assert mc.model_type == "nupovik" and mc.num_hidden_layers == len(runs)
        assert [(s["layer"], s["opens_pass"]) for s in mc.layer_specs] == runs
        assert mc.logit_scale == cfg.get("logit_scale", 1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_residual_after_every_layer_run(models, dtype):
    """The residual stream after every layer run of a short prompt (looped layers count each time)."""
    cfg, weights, folder = models["mixed"]
    s = H.open_session(folder, dtype, max_tokens=256, max_requests=2, cuda_graph=False)
    model = s.worker.model_runner.model
    got = {}
    model._layer_hook = lambda i, x: got.__setitem__(i, x.double().cpu())
    toks = H.prompt(19, cfg["vocab"], 19)
    s.step([{"id": "a", "tokens": toks, "want": []}])
    model._layer_hook = None
    want = []
    N.forward(cfg, weights, toks, want)
    assert len(got) == len(want)
    for r, ref in enumerate(want):
        rel = ((got[r] - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
        assert rel < (1e-5 if dtype == "float32" else 2e-2), f"layer run {r}: relative RMS error {rel:.3e}"


LENGTHS = (1, 2, 13, 150)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_model_every_schedule(models, name, dtype):
    """Whole prompts, prompt + token-by-token decoding, portions of changing size down to two tokens, and mixed
    batches of unequal requests — each position against the whole-sequence oracle; all of it in one small pool,
    so request slots, state slots and cache runs are reused throughout."""
    cfg, _, folder = models[name]
    s = H.open_session(folder, dtype, max_tokens=640, max_requests=4)
    V = cfg["vocab"]
    prompts = {n: H.prompt(n, V, seed=n) for n in LENGTHS}
    full = lambda n: list(range(n))
    for n, toks in prompts.items():
        got = s.step([{"id": f"w{n}", "tokens": toks, "want": full(n)}])
        s.end([f"w{n}"])
        _check(got, _oracle(models, name, toks), dtype, f"{name} whole {n}")
    for n in (13, 150):
        toks, want = prompts[n], _oracle(models, name, prompts[n])
        cut = n - 9
        rows = [s.step([{"id": "d", "tokens": toks[:cut], "want": full(cut)}])]
        for p in range(cut, n):
            rows.append(s.step([{"id": "d", "tokens": [toks[p]], "want": [0]}]))
        s.end(["d"])
        _check(torch.cat(rows), want, dtype, f"{name} decode {n}")
    toks, want = prompts[150], _oracle(models, name, prompts[150])
    rows, at = [], 0
    for size in (2, 3, 64, 2, 5, 1, 1, 40, 2, 30):
        rows.append(s.step([{"id": "c", "tokens": toks[at:at + size], "want": full(size)}]))
        at += size
    assert at == 150
    s.end(["c"])
    _check(torch.cat(rows), want, dtype, f"{name} portions")
    plan = {"a": prompts[150], "b": prompts[13], "c": prompts[2], "d": H.prompt(70, V, 70), "e": H.prompt(31, V, 31)}
    cuts = {"a": [64, 2, 1, 1, 50, 1, 31], "b": [1, 1, 1, 5, 5], "c": [2], "d": [3, 60, 1, 1, 1, 1, 1, 1, 1],
            "e": [30, 1]}
    order = [["a", "b", "c", "d"], ["a", "b", "d"], ["a", "b", "d", "e"], ["a", "b", "d", "e"], ["a", "b", "d"],
             ["a", "d"], ["a", "d"], ["d"], ["d"]]
    at = {k: 0 for k in plan}
    idx = {k: 0 for k in plan}
    got = {k: [] for k in plan}
    for live in order:
        entries, ends = [], []
        for r in live:
            n = cuts[r][idx[r]]
            entries.append({"id": r, "tokens": plan[r][at[r]:at[r] + n], "want": full(n)})
            at[r] += n
            idx[r] += 1
            if at[r] == len(plan[r]):
                ends.append(r)
        out = s.step(entries)
        o = 0
        for e in entries:
            got[e["id"]].append(out[o:o + len(e["tokens"])])
            o += len(e["tokens"])
        s.end(ends)
    for r, toks in plan.items():
        assert at[r] == len(toks)
        _check(torch.cat(got[r]), _oracle(models, name, toks), dtype, f"{name} mixed {r}")


def test_long_decoding_and_far_tokens(models):
    """330 tokens, 320 of them decoded one by one, with sharp attention and slow decays; and a change of the
    FIRST token still moves the last logits by what the oracle says."""
    cfg, _, folder = models["far"]
    s = H.open_session(folder, "float32", max_tokens=768, max_requests=2)
    V = cfg["vocab"]
    toks = H.prompt(330, V, 9)
    other = [(toks[0] + 1) % V] + toks[1:]
    last = {}
    for rid, seq in (("x", toks), ("y", other)):
        s.step([{"id": rid, "tokens": seq[:10], "want": []}])
        for p in range(10, 329):
            s.step([{"id": rid, "tokens": [seq[p]], "want": []}])
        last[rid] = s.step([{"id": rid, "tokens": [seq[329]], "want": [0]}])[0].cpu().double()
        s.end([rid])
    wx, wy = _oracle(models, "far", toks)[329], _oracle(models, "far", other)[329]
    assert H.rel_err(last["x"][None], wx[None]).item() < 2 * H.TOL["float32"]
    assert H.rel_err(last["y"][None], wy[None]).item() < 2 * H.TOL["float32"]
    moved, want_moved = last["x"] - last["y"], wx - wy
    assert want_moved.abs().max() > 1e-3, "the test's weights do not carry the first token this far"
    assert (moved - want_moved).abs().max() < 0.05 * want_moved.abs().max() + 2e-5


def test_sharp_attention_sees_every_key(models):
    """With the sharp scale each query's output is one far key's value: every row of a 300-token prompt must
    match, as a whole and when the tail is fed in portions and single tokens across the run border of the pool."""
    cfg, _, folder = models["far"]
    s = H.open_session(folder, "float32", max_tokens=512, max_requests=2)
    toks = H.prompt(300, cfg["vocab"], 3)
    want = _oracle(models, "far", toks)
    got = s.step([{"id": "w", "tokens": toks, "want": list(range(300))}])
    s.end(["w"])
    _check(got, want, "float32", "sharp whole")
    rows, at = [], 0
    for size in [120, 7, 1, 1, 2, 125] + [1] * 10 + [34]:
        rows.append(s.step([{"id": "p", "tokens": toks[at:at + size], "want": list(range(size))}]))
        at += size
    assert at == 300
    _check(torch.cat(rows), want, "float32", "sharp portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_greedy_generation(models, dtype):
    from semi_pd_b200.configs import ServerArgs
    from semi_pd_b200.semi_pd_scheduler import SemiPDEngine
    cfg, weights, folder = models["mixed"]
    V, n_new = cfg["vocab"], 24
    sa = ServerArgs(model_path=folder, dtype=dtype, load_format="auto", max_total_tokens=4096,
                    max_running_requests=8, context_length=512, enable_semi_pd=True, cuda_graph_bs=[1, 2, 4, 8],
                    chunked_prefill_size=48, max_prefill_tokens=256)
    eng = SemiPDEngine(sa, gpu_id=0, prefill_sm_percent=50, decode_sm_percent=50)
    try:
        prompts = [H.prompt(n, V, seed=100 + n) for n in (5, 33, 120, 61, 2, 77)]
        rids = [eng.submit(p, n_new) for p in prompts]
        done = {r.rid: r for r in eng.wait(len(rids), timeout=120)}
    finally:
        eng.shutdown()
    margin_floor = 1e-3 if dtype == "float32" else 0.3
    for rid, p in zip(rids, prompts):
        out = done[rid].output_ids
        assert len(out) == n_new
        stepper = N.Stepper(cfg, weights)
        logits = stepper.feed(list(p))[-1]
        for t, tok in enumerate(out):
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < margin_floor:
                break  # a near tie: either token is a correct greedy choice; stop comparing this request
            assert tok == int(logits.argmax()), f"{rid}: token {t} differs from the oracle's greedy choice"
            logits = stepper.feed([tok])[-1]

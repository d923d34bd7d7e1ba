"""Rimidra family on the GPU against the float64 oracle (oracle/rimidra_oracle.py): every mechanism
alone through its operator, then whole models through the serving path (ScheduleBatch → worker →
kernels, decode through the captured CUDA graphs) under every way of cutting and batching the same
tokens, then greedy generation through the semi-PD engine."""
import math

import pytest
import torch

from oracle import rimidra_oracle as R
from tests import rimidra_helpers as H

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _close(got, want, dtype, what=""):
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = (got.double().cpu() - want.double().cpu()).abs().max().item()
    ref = want.double().abs().max().item() + 1e-9
    assert err <= tol * ref, f"{what}: max abs err {err:.3e} vs ref max {ref:.3e}"


# =================================================================================================
# mechanisms alone
# =================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [40, 64, 1000])
def test_residual_rmsnorm(dtype, dim):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(7, dim, generator=g)
    a = torch.randn(7, dim, generator=g).to(dt)
    b = torch.randn(7, dim, generator=g).to(dt)
    w = (torch.randn(dim, generator=g) * 0.3).to(dt)
    xd = x.to(DEV)
    out = ops.residual_rmsnorm(xd, w.to(DEV), 1e-5, a=a.to(DEV), b=b.to(DEV), weight_offset=1.0)
    x_ref = x.double() + (a.double() + b.double())
    _close(xd, x_ref, torch.float32, "residual")
    _close(out, R.offset_rms_norm(x_ref, w.double(), 1e-5), dt, "norm")
    # norm only, and add only
    x2 = x.to(DEV)
    out2 = ops.residual_rmsnorm(x2, w.to(DEV), 1e-5, weight_offset=1.0)
    _close(out2, R.offset_rms_norm(x.double(), w.double(), 1e-5), dt, "norm only")
    assert ops.residual_rmsnorm(x2, None, 1e-5, a=a.to(DEV)) is None
    _close(x2, x.double() + a.double(), torch.float32, "add only")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_activations_and_head_norm(dtype):
    from semi_pd_b200 import ops
    dt = DT[dtype]
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(9, 2 * 52, generator=g) * 3).to(dt)
    for act, fn in (("silu", R.silu), ("gelu_tanh", R.gelu_tanh)):
        got = ops.act_and_mul(x.to(DEV), act)
        xd = x.double()
        _close(got, fn(xd[:, :52]) * xd[:, 52:], dt, act)
    heads, vdim = 3, 24
    o = torch.randn(5, heads * vdim, generator=g)
    wide = torch.randn(5, 100 + heads * vdim, generator=g).to(dt)  # the gate is a strided slice of a wider row
    gate = wide[:, 100:]
    got = ops.headnorm_gate(o.to(DEV), wide.to(DEV)[:, 100:], heads, vdim, 1e-6)
    want = (R.unit_rms(o.double().view(5, heads, vdim), 1e-6).reshape(5, -1)) * R.silu(gate.double())
    _close(got, want, dt, "headnorm_gate")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 50, 40), (5, 17, 9), (70, 130, 33), (129, 64, 256)])
def test_linear_simt(dtype, shape):
    from semi_pd_b200 import ops
    M, N, K = shape
    dt = DT[dtype]
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(dt)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(dt)
    want = x.double() @ w.double().T
    _close(ops.linear_simt(x.to(DEV), w.to(DEV)), want, dt)
    _close(ops.linear_simt(x.to(DEV), w.to(DEV), out_f32=True), want, torch.float32)
    # the same row gives the same bits whatever else is in the batch
    one = ops.linear_simt(x[:1].to(DEV), w.to(DEV), out_f32=True)
    assert torch.equal(one, ops.linear_simt(x.to(DEV), w.to(DEV), out_f32=True)[:1])


@pytest.mark.parametrize("shape", [(1, 64, 256), (3, 24, 40), (33, 136, 96), (300, 96, 64), (40, 8, 72)])
def test_linear_any_tensor_core_route_matches(shape):
    """16-bit aligned shapes take the tcgen05 GEMMs; they must agree with the CUDA-core GEMM."""
    from semi_pd_b200 import ops
    M, N, K = shape
    g = torch.Generator().manual_seed(N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    assert ops._tc_gemm_ok(x, w, N)
    a, b = ops.linear_any(x, w, out_f32=True), ops.linear_simt(x, w, out_f32=True)
    _close(a, b.cpu(), torch.float32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top", [(4, 2), (5, 3), (2, 1), (16, 1)])
def test_moe_pieces(dtype, experts, top):
    """sigmoid top-k routing without renormalisation, experts that weight their input, grouped GEMMs
    over expert-aligned tiles, gated shared expert — against the per-token loop."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    T, Wd, ff = 37, 48, 24
    g = torch.Generator().manual_seed(experts * 10 + top)
    u = torch.randn(T, Wd, generator=g).to(dt)
    router = (torch.randn(experts + 1, Wd, generator=g) * 4 / math.sqrt(Wd)).to(dt)
    wgu = (torch.randn(experts * 2 * ff, Wd, generator=g) / math.sqrt(Wd)).to(dt)
    wdn = (torch.randn(experts * Wd, ff, generator=g) / math.sqrt(ff)).to(dt)
    shared = torch.randn(T, Wd, generator=g).to(dt)
    z = ops.linear_simt(u.to(DEV), router.to(DEV), out_f32=True)
    ids, w = ops.moe_route_scores(z, experts, top, "sigmoid")
    want_ids, want_w = R.sigmoid_topk_routing(u.double(), router.double()[:experts], top)
    assert torch.equal(ids.cpu().long(), want_ids)
    _close(w, want_w, torch.float32, "routing weights")
    row_token, inv_pos, tile_group = ops.moe_align(ids, experts)
    xs = ops.moe_gather_scaled(u.to(DEV), row_token, inv_pos, w)
    act = ops.act_and_mul(ops.linear_grouped_any(xs, wgu.to(DEV), tile_group, experts, 2 * ff), "silu")
    y = ops.linear_grouped_any(act, wdn.to(DEV), tile_group, experts, Wd)
    got = ops.moe_combine_gated(y, inv_pos, T, top, shared=shared.to(DEV), shared_gate=z[:, experts:])
    want = torch.zeros(T, Wd, dtype=torch.float64)
    ud = u.double()
    for t in range(T):
        for j in range(top):
            e = int(want_ids[t, j])
            gu = wgu.double()[e * 2 * ff:(e + 1) * 2 * ff]
            xin = want_w[t, j] * ud[t]
            want[t] += (R.silu(gu[:ff] @ xin) * (gu[ff:] @ xin)) @ wdn.double()[e * Wd:(e + 1) * Wd].T
    want += shared.double() * torch.sigmoid(ud @ router.double()[experts:].T)
    _close(got, want, dt, "moe output")


@pytest.mark.parametrize("ff", [24, 96, 128, 200, 704])
def test_silu_mul_in_the_gemm_epilogue(ff):
    """silu(gate) * up applied by the tensor-core GEMMs to their accumulators — grouped (experts) and
    plain (a shared expert at prefill size) — against float64, for widths on and off the 128-row tile."""
    from semi_pd_b200 import ops
    dt, Wd, E, T = torch.bfloat16, 128, 3, 300
    g = torch.Generator().manual_seed(ff)
    x = torch.randn(T, Wd, generator=g).to(dt)
    wgu = (torch.randn(E * 2 * ff, Wd, generator=g) / Wd ** 0.5).to(dt)
    ids = torch.randint(0, E, (T, 1), generator=g).int()
    row_token, inv_pos, tile_group = ops.moe_align(ids.to(DEV), E)
    xs = ops.moe_gather_scaled(x.to(DEV), row_token, inv_pos, None)
    got = ops.linear_grouped_any(xs, wgu.to(DEV), tile_group, E, ff, silu_mul=True)
    pos = inv_pos.cpu().long().reshape(T)
    for t in range(0, T, 7):
        e = int(ids[t, 0])
        gu = wgu.double()[e * 2 * ff:(e + 1) * 2 * ff] @ x[t].double()
        _close(got[pos[t]], R.silu(gu[:ff]) * gu[ff:], dt, f"expert row {t}")
    gu = x.double() @ wgu.double()[:2 * ff].T
    _close(ops.linear_silu_mul_any(x.to(DEV), wgu[:2 * ff].to(DEV)), R.silu(gu[:, :ff]) * gu[:, ff:], dt, "plain")


def _paged(seq_k, seq_v, dtype, extra_slots=37, seed=0):
    """Scatter a sequence's K / V rows over a pool in a random slot order; → pools, page table row."""
    T = seq_k.shape[0]
    g = torch.Generator().manual_seed(seed)
    slots = torch.randperm(T + extra_slots, generator=g)[:T] + 1
    kp = torch.randn(T + extra_slots + 1, *seq_k.shape[1:], generator=g).to(dtype)
    vp = torch.randn(T + extra_slots + 1, *seq_v.shape[1:], generator=g).to(dtype)
    kp[slots], vp[slots] = seq_k.to(dtype), seq_v.to(dtype)
    return kp.to(DEV), vp.to(DEV), slots.int()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [
    dict(H=4, G=2, dk=16, dv=8, window=12, sink=True, slopes=True, qt=(0.4, 16)),
    dict(H=1, G=1, dk=8, dv=8, window=1, sink=True, slopes=False, qt=None),
    dict(H=8, G=2, dk=64, dv=64, window=130, sink=True, slopes=True, qt=(0.3, 128)),
    dict(H=3, G=3, dk=24, dv=40, window=-1, sink=False, slopes=True, qt=(0.2, 5)),
    # shapes of the grouped decode kernel: 3, 8 and 1 query heads per key/value head, every value width
    dict(H=6, G=2, dk=32, dv=128, window=33, sink=True, slopes=True, qt=(0.3, 7)),
    dict(H=16, G=2, dk=16, dv=32, window=200, sink=True, slopes=True, qt=None),
    dict(H=2, G=2, dk=128, dv=256, window=-1, sink=True, slopes=True, qt=(0.1, 64)),
    # head sizes of the tensor-core kernels: 4, 12 and 1 query heads per key/value head
    dict(H=8, G=2, dk=128, dv=128, window=100, sink=True, slopes=True, qt=(0.3, 128)),
    dict(H=12, G=1, dk=64, dv=128, window=-1, sink=True, slopes=True, qt=(0.2, 9)),
    dict(H=3, G=3, dk=128, dv=64, window=31, sink=False, slopes=True, qt=None),
])
def test_attention_kernel_prefill_chunks_and_decode(dtype, case):
    """One sequence of 300 tokens over scattered slots: a portion with a prefix, a portion from the
    start, and single decoded tokens — all against the whole-sequence oracle."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    T = 300
    Hh, G, dk, dv = case["H"], case["G"], case["dk"], case["dv"]
    g = torch.Generator().manual_seed(Hh * 100 + dk)
    q = torch.randn(T, Hh, dk, generator=g).to(dt)
    k = torch.randn(T, G, dk, generator=g).to(dt)
    v = torch.randn(T, G, dv, generator=g).to(dt)
    sinks = torch.randn(Hh, generator=g) if case["sink"] else None
    slopes = R.distance_slopes(Hh) if case["slopes"] else None
    want = R.windowed_sink_attention(q.double(), k.double(), v.double(), 0.2, case["window"], sinks, slopes,
                                     case["qt"]).reshape(T, Hh * dv)
    kp, vp, slots = _paged(k, v, dt)
    r2t = torch.zeros(3, 512, dtype=torch.int32)
    r2t[2, :T] = slots
    r2t = r2t.to(DEV)
    rpi = torch.tensor([2], dtype=torch.int64, device=DEV)
    kw = dict(num_q_heads=Hh, num_kv_heads=G, head_dim=dk, v_dim=dv, sm_scale=0.2, window=case["window"],
              sinks=sinks.to(DEV) if sinks is not None else None,
              slopes=slopes.float().to(DEV) if slopes is not None else None,
              qtemp_coef=case["qt"][0] if case["qt"] else 0.0, qtemp_every=case["qt"][1] if case["qt"] else 0)
    qd = q.reshape(T, Hh * dk).to(DEV)
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32, device=DEV)
    for pre, n in ((0, T), (0, 1), (5, 2), (127, 3), (100, 157)):
        got = ops.attn_general(qd[pre:pre + n].contiguous(), kp, vp, r2t, rpi, prefix_lens=i32(pre), extend_lens=i32(n),
                               extend_start_loc=i32(0), **kw)
        _close(got, want[pre:pre + n], dt, f"extend {pre}+{n}")
    for pos in (0, 1, 11, 12, 13, 127, 128, 129, 130, 131, 299):
        got = ops.attn_general(qd[pos:pos + 1].contiguous(), kp, vp, r2t, rpi,
                               seq_lens=torch.tensor([pos + 1], dtype=torch.int64, device=DEV), **kw)
        _close(got, want[pos:pos + 1], dt, f"decode at {pos}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(H=8, G=2, dk=64, dv=64), dict(H=4, G=4, dk=32, dv=32), dict(H=5, G=1, dk=16, dv=24),
                                   dict(H=16, G=1, dk=128, dv=128), dict(H=6, G=3, dk=64, dv=128)])
def test_attention_decode_batch_of_unequal_requests(dtype, shape):
    """Five requests of unequal length decode in one launch (slots interleaved in one pool, request
    rows out of order): every row equals the whole-sequence oracle of its own request."""
    from semi_pd_b200 import ops
    dt = DT[dtype]
    Hh, G, dk, dv = shape["H"], shape["G"], shape["dk"], shape["dv"]
    window, lens = 70, [1, 69, 70, 71, 260]
    g = torch.Generator().manual_seed(11)
    total = sum(lens)
    perm = torch.randperm(total + 50, generator=g)[:total] + 1
    kp = torch.randn(total + 51, G, dk, generator=g).to(dt)
    vp = torch.randn(total + 51, G, dv, generator=g).to(dt)
    r2t = torch.zeros(8, 320, dtype=torch.int32)
    sinks, slopes = torch.randn(Hh, generator=g), R.distance_slopes(Hh)
    rows, qs, wants, at = [7, 2, 5, 0, 3], [], [], 0
    for n, row in zip(lens, rows):
        q = torch.randn(n, Hh, dk, generator=g).to(dt)
        k = torch.randn(n, G, dk, generator=g).to(dt)
        v = torch.randn(n, G, dv, generator=g).to(dt)
        sl = perm[at:at + n]
        at += n
        kp[sl], vp[sl] = k, v
        r2t[row, :n] = sl.int()
        wants.append(R.windowed_sink_attention(q.double(), k.double(), v.double(), 0.25, window, sinks, slopes,
                                               (0.3, 32)).reshape(n, Hh * dv)[-1])
        qs.append(q[-1].reshape(Hh * dk))
    got = ops.attn_general(torch.stack(qs).to(DEV), kp.to(DEV), vp.to(DEV), r2t.to(DEV),
                           torch.tensor(rows, dtype=torch.int64, device=DEV), num_q_heads=Hh, num_kv_heads=G, head_dim=dk,
                           v_dim=dv, sm_scale=0.25, window=window, sinks=sinks.to(DEV), slopes=slopes.float().to(DEV),
                           qtemp_coef=0.3, qtemp_every=32, seq_lens=torch.tensor(lens, dtype=torch.int64, device=DEV))
    _close(got, torch.stack(wants), dt, "batched decode")


@pytest.mark.parametrize("mode", ["extend", "decode"])
def test_attention_window_edge_and_sink_show(mode):
    """Inputs made so that one score stands out.  The key just inside the window carries the output;
    the same spike one position further back, just outside, must not be seen; and a large sink must
    drain the weight of ordinary keys (a missing sink would leave the output at O(1))."""
    from semi_pd_b200 import ops
    T, window, dk, dv = 200, 9, 16, 16
    g = torch.Generator().manual_seed(5)
    q = torch.randn(T, 1, dk, generator=g) * 0.1
    k = torch.randn(T, 1, dk, generator=g) * 0.1
    v = torch.randn(T, 1, dv, generator=g)
    i = 150
    e = torch.zeros(dk)
    e[3] = 1.0
    q[i, 0] = 30.0 * e
    k[i - window + 1, 0] = 30.0 * e      # last visible key
    k[i - window, 0] = 60.0 * e          # first invisible key: a larger spike
    kp, vp, slots = _paged(k, v, torch.float32)
    r2t = torch.zeros(1, 256, dtype=torch.int32)
    r2t[0, :T] = slots
    r2t = r2t.to(DEV)
    rpi = torch.zeros(1, dtype=torch.int64, device=DEV)
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32, device=DEV)

    def run(sinks):
        kw = dict(num_q_heads=1, num_kv_heads=1, head_dim=dk, v_dim=dv, sm_scale=1.0, window=window, sinks=sinks)
        if mode == "decode":
            return ops.attn_general(q[i].reshape(1, dk).to(DEV), kp, vp, r2t, rpi,
                                    seq_lens=torch.tensor([i + 1], dtype=torch.int64, device=DEV), **kw).cpu()[0]
        out = ops.attn_general(q[i - 20:i + 1].reshape(21, dk).to(DEV), kp, vp, r2t, rpi, prefix_lens=i32(i - 20),
                               extend_lens=i32(21), extend_start_loc=i32(0), **kw)
        return out.cpu()[20]

    out = run(torch.zeros(1, device=DEV))
    assert (out - v[i - window + 1, 0]).abs().max() < 1e-3, "the last key of the window was not seen"
    drained = run(torch.full((1,), 2000.0, device=DEV))
    assert drained.abs().max() < 1e-3, "the sink did not enter the denominator"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [dict(H=2, dk=16, dv=32, rot=8), dict(H=1, dk=8, dv=8, rot=8),
                                  dict(H=3, dk=64, dv=72, rot=32), dict(H=2, dk=128, dv=40, rot=0)])
def test_retention_kernel(dtype, case):
    """Portions of several sizes (down to one token), decoding, two requests in one launch, a state
    slot that held another request before, and a padded decode row."""
    from semi_pd_b200 import ops
    from semi_pd_b200.rimidra import _rotary_table
    dt = DT[dtype]
    Hh, dk, dv, rot = case["H"], case["dk"], case["dv"], case["rot"]
    T = 90
    g = torch.Generator().manual_seed(dk + dv)
    decay = [1.0 - 2.0 ** (-3 - h) for h in range(Hh)]
    seqs = []
    for _ in range(2):
        q = torch.randn(T, Hh, dk, generator=g).to(dt)
        k = torch.randn(T, Hh, dk, generator=g).to(dt)
        v = torch.randn(T, Hh, dv, generator=g).to(dt)
        pos = torch.arange(T)
        qr = R.rotate_half_partial(q.double(), pos, rot, 1000.0)
        kr = R.rotate_half_partial(k.double(), pos, rot, 1000.0) * dk ** -0.5
        want, final = R.retention_recurrence(qr, kr, v.double(), decay)
        seqs.append((q, k, v, want.reshape(T, Hh * dv), final))
    state = torch.randn(5, Hh, dk, dv, generator=g).to(DEV)  # stale contents: slots were "used before"
    table = _rotary_table(rot, 1000.0, 128, DEV)
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    kw = dict(num_heads=Hh, head_dim=dk, v_dim=dv, decay=dec, cos_sin=table, rot_dims=rot, k_scale=dk ** -0.5)
    rpi = torch.tensor([3, 1], dtype=torch.int64, device=DEV)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    flat = lambda t, a, b: t[a:b].reshape(b - a, -1)
    at = [0, 0]
    # unequal portions of the two requests side by side
    for n0, n1 in ((1, 17), (2, 16), (33, 2), (16, 1), (5, 31)):
        parts = [(at[0], n0), (at[1], n1)]
        q = torch.cat([flat(seqs[r][0], a, a + n) for r, (a, n) in enumerate(parts)]).to(DEV)
        k = torch.cat([flat(seqs[r][1], a, a + n) for r, (a, n) in enumerate(parts)]).to(DEV)
        v = torch.cat([flat(seqs[r][2], a, a + n) for r, (a, n) in enumerate(parts)]).to(DEV)
        o = ops.retention(q, k, v, state, rpi, prefix_lens=i32([at[0], at[1]]), extend_lens=i32([n0, n1]),
                          extend_start_loc=i32([0, n0]), **kw)
        want = torch.cat([seqs[r][3][a:a + n] for r, (a, n) in enumerate(parts)])
        _close(o, want, dt, f"portions {parts}")
        at = [at[0] + n0, at[1] + n1]
    # decode both, with a padded third row (out_cache_loc 0) that must leave slot 4 alone
    before = state[4].clone()
    while at[0] < T and at[1] < T:
        rows = [(0, at[0]), (1, at[1])]
        q = torch.cat([flat(seqs[r][0], a, a + 1) for r, a in rows] + [flat(seqs[0][0], 0, 1)]).to(DEV)
        k = torch.cat([flat(seqs[r][1], a, a + 1) for r, a in rows] + [flat(seqs[0][1], 0, 1)]).to(DEV)
        v = torch.cat([flat(seqs[r][2], a, a + 1) for r, a in rows] + [flat(seqs[0][2], 0, 1)]).to(DEV)
        o = ops.retention(q, k, v, state, torch.tensor([3, 1, 4], dtype=torch.int64, device=DEV),
                          seq_lens=torch.tensor([at[0] + 1, at[1] + 1, 1], dtype=torch.int64, device=DEV),
                          out_cache_loc=torch.tensor([7, 9, 0], dtype=torch.int64, device=DEV), **kw)
        _close(o[:2], torch.cat([seqs[r][3][a:a + 1] for r, a in rows]), dt, f"decode {rows}")
        at = [at[0] + 1, at[1] + 1]
    assert torch.equal(state[4], before)
    _close(state[1], seqs[1][4], dt, "final state")


# =================================================================================================
# whole models through the serving path
# =================================================================================================
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, make in H.CONFIGS.items():
        cfg = make()
        weights = R.make_weights(cfg, seed=len(name))
        folder = H.write_model(tmp_path_factory.mktemp(name), cfg, weights)
        out[name] = (cfg, weights, folder)
    return out


_oracle_cache = {}


def _oracle(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _oracle_cache:
        cfg, weights, _ = models[name]
        _oracle_cache[key] = R.forward(cfg, weights, list(tokens))
    return _oracle_cache[key]


def _check(got, want, dtype, what):
    err = H.rel_err(got, want)
    if dtype == "float32":
        assert err.max().item() < H.TOL[dtype], f"{what}: worst relative error {err.max().item():.3e} at row {int(err.argmax())}"
    else:  # 16-bit: a routing decision on a near tie may differ from float64 for a few tokens
        assert err.median().item() < H.TOL[dtype] / 2, f"{what}: median {err.median().item():.3e}"
        assert (err > H.TOL[dtype]).float().mean().item() <= 0.05, f"{what}: {(err > H.TOL[dtype]).sum()} rows off"


LENGTHS = (1, 2, 13, 150)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(H.CONFIGS))
def test_model_every_schedule(models, name, dtype):
    """Whole prompts, prompt + token-by-token decoding, portions of changing size down to two
    tokens, and mixed batches of unequal requests — each position against the whole-sequence oracle;
    all of it in one small pool, so request slots, state slots and KV runs are reused throughout."""
    cfg, _, folder = models[name]
    s = H.open_session(folder, dtype, max_tokens=640, max_requests=4)
    V = cfg["vocab"]
    prompts = {n: H.prompt(n, V, seed=n) for n in LENGTHS}
    full = lambda n: list(range(n))
    # whole
    for n, toks in prompts.items():
        got = s.step([{"id": f"w{n}", "tokens": toks, "want": full(n)}])
        s.end([f"w{n}"])
        _check(got, _oracle(models, name, toks), dtype, f"{name} whole {n}")
    # most of it at once, the tail token by token (through the decode graphs)
    for n in (13, 150):
        toks, want = prompts[n], _oracle(models, name, prompts[n])
        cut = n - 9
        rows = [s.step([{"id": "d", "tokens": toks[:cut], "want": full(cut)}])]
        for p in range(cut, n):
            rows.append(s.step([{"id": "d", "tokens": [toks[p]], "want": [0]}]))
        s.end(["d"])
        _check(torch.cat(rows), want, dtype, f"{name} decode {n}")
    # portions
    toks, want = prompts[150], _oracle(models, name, prompts[150])
    rows, at = [], 0
    for size in (2, 3, 64, 2, 5, 1, 1, 40, 2, 30):
        rows.append(s.step([{"id": "c", "tokens": toks[at:at + size], "want": full(size)}]))
        at += size
    assert at == 150
    s.end(["c"])
    _check(torch.cat(rows), want, dtype, f"{name} portions")
    # mixed: four live requests, portions beside single tokens; a finished one's slot is taken by the next
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
    """330 tokens, 320 of them decoded one by one: the recurrent state and the window keep up; and a
    change of the FIRST token still moves the last logits by what the oracle says (nothing but the
    recurrent state can carry it that far)."""
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
    assert H.rel_err(last["x"][None], wx[None]).item() < H.TOL["float32"]
    assert H.rel_err(last["y"][None], wy[None]).item() < H.TOL["float32"]
    moved, want_moved = last["x"] - last["y"], wx - wy
    assert want_moved.abs().max() > 1e-3, "the test's weights do not carry the first token this far"
    assert (moved - want_moved).abs().max() < 0.05 * want_moved.abs().max() + 2e-5


def test_float32_refused_for_16bit_families():
    from semi_pd_b200.configs import ServerArgs, get_model_config
    from semi_pd_b200.model_runner import ModelRunner
    sa = ServerArgs(model_path="tiny-llama-test", dtype="float32", enable_semi_pd=True, max_total_tokens=256)
    with pytest.raises(ValueError):
        ModelRunner(get_model_config("tiny-llama-test"), 0.5, 0, 0, 1, 0, sa)


# =================================================================================================
# greedy generation through the engine (prefill and decode workers, chunked prefill, CUDA graphs)
# =================================================================================================
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
        seq = list(p)
        for t, tok in enumerate(out):
            logits = R.forward(cfg, weights, seq)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < margin_floor:
                break  # a near tie: either token is a correct greedy choice; stop comparing this request
            assert tok == int(logits.argmax()), f"{rid}: token {t} differs from the oracle's greedy choice"
            seq.append(tok)

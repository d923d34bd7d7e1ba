"""Nupovik beside Llama and Rimidra (the closest family: recurrent mixers, fp32 stream, routed experts) at equal
size: whole-model prefill / decode throughput through the worker (ScheduleBatch → TpModelWorker, decode through
the captured CUDA graphs) and the per-kernel times of the mechanisms the family adds, each beside the like
kernel of the existing paths, with the fraction of the measured roofline.  Random weights, synthetic tokens.
`bench.py --family nupovik` runs this; stand-alone: python scripts/bench_nupovik.py [--sizes s,m] [--out FILE]."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import bench_rimidra as BR  # noqa: E402  (sizes, timing helpers, the two models set beside this one)

SIZES = {
    # the Rimidra / Llama shape of the same name, plus this family's own sizes: latent rank, recurrent heads
    "s": dict(BR.SIZES["s"], rank=128, wkv_heads=16, wkv_dim=64, low_rank=64, groups=4, keep=2),
    "m": dict(BR.SIZES["m"], rank=128, wkv_heads=32, wkv_dim=64, low_rank=64, groups=4, keep=2),
    "l": dict(BR.SIZES["l"], rank=128, wkv_heads=64, wkv_dim=64, low_rank=128, groups=4, keep=2),
}
VOCAB = BR.VOCAB


def nupovik_config(z, moe):
    """Eight layer runs: latent attention, two passes over (token-shift mixer, gated linear attention), then gated
    linear attention, token-shift mixer, gated linear attention."""
    from semi_pd_b200.configs import _nupovik_config
    mlp = ({"kind": "moe", "expert": {"ff": z["eff"]},
            "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"], "keep": z["keep"]}}}
           if moe else {"kind": "dense", "ff": z["ff"]})
    gla = {"type": "gla", "mlp": mlp, "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["dim"], "tau": 16.0}}
    wkv = {"type": "wkv", "mlp": mlp, "mixer": {"heads": z["wkv_heads"], "dim": z["wkv_dim"]}}
    layers = [
        {"type": "latent_attention", "mlp": mlp,
         "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["dim"], "kv_rank": z["rank"], "scale": z["dim"] ** -0.5}},
        wkv, gla, gla, wkv, gla]
    cfg = {"architecture": "Nupovik", "vocab": VOCAB, "width": z["width"], "norm": {"eps": 1e-6}, "layers": layers,
           "loop": {"start": 1, "stop": 3, "times": 2}, "logit_scale": 0.25, "context": 8192}
    return _nupovik_config("nupovik-bench", cfg)


def kernel_table(z, flush):
    """Per-kernel time of this family's mechanisms and of the like kernels of the existing paths."""
    from semi_pd_b200 import ops
    from semi_pd_b200.nupovik import _sinusoid_frequencies
    from semi_pd_b200.rimidra import _rotary_table
    hbm, tf, _ = BR.peaks()
    dev, bf = "cuda", torch.bfloat16
    H, D, Wd, R = z["heads"], z["dim"], z["width"], z["rank"]
    n_req, L, B = 4, 2048, 64
    T = n_req * L
    rows = []

    def add(name, like, ms, flops=None, bytes_=None, peak_tf=None):
        r = {"kernel": name, "like": like, "ms": ms}
        if flops is not None:
            r["tflops"] = flops / ms / 1e9
            r["frac_of_peak"] = r["tflops"] / (peak_tf or tf)
            r["peak"] = "cuda-core fp32" if peak_tf else "bf16 tensor (measured)"
        if bytes_ is not None:
            r["gbs"] = bytes_ / ms / 1e6
            r["frac_of_peak"] = r["gbs"] / hbm
            r["peak"] = "hbm (measured)"
        rows.append(r)

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    rpi = torch.arange(n_req, device=dev, dtype=torch.int64)
    pre, ext, start = i32([0] * n_req), i32([L] * n_req), i32([r * L for r in range(n_req)])
    rpd = torch.arange(B, device=dev, dtype=torch.int64)
    sl = torch.full((B,), L, dtype=torch.int64, device=dev)
    loc = torch.ones(B, dtype=torch.int64, device=dev)
    ev = lambda fn: BR.event_ms(fn, flush=flush)
    # ---- the two recurrences, beside retention ------------------------------------------------------
    for form, heads, dk in (("sigmoid_pow", H, D), ("double_exp", z["wkv_heads"], z["wkv_dim"])):
        state = torch.zeros(B + 1, heads, dk, dk, device=dev)
        x = torch.randn(T, 4 * heads * dk, device=dev, dtype=bf)
        q, k, v, zz = x.split(heads * dk, dim=-1)
        bias = torch.full((heads * dk,), 3.0 if form == "sigmoid_pow" else -3.0, device=dev)
        u = torch.zeros(heads * dk, device=dev) if form == "double_exp" else None
        kw = dict(num_heads=heads, head_dim=dk, v_dim=dk, form=form, q_scale=dk ** -0.5, tau=16.0, z_bias=bias, bonus=u)
        ms = ev(lambda: ops.gated_recurrence(q, k, v, zz, state, rpi, prefix_lens=pre, extend_lens=ext,
                                             extend_start_loc=start, **kw))
        add(f"gated_recurrence {form} prefill {n_req}x{L} ({heads}x{dk})", "", ms, flops=4.0 * heads * dk * dk * T,
            peak_tf=BR.FP32_CORE_TFLOPS)
        xd = torch.randn(B, 4 * heads * dk, device=dev, dtype=bf)
        qd, kd, vd, zd = xd.split(heads * dk, dim=-1)
        ms = ev(lambda: ops.gated_recurrence(qd, kd, vd, zd, state, rpd, seq_lens=sl, out_cache_loc=loc, **kw))
        add(f"gated_recurrence {form} decode B={B} ({heads}x{dk})", "", ms, bytes_=B * heads * dk * dk * 4 * 2)
    state = torch.zeros(B + 1, H, D, D, device=dev)
    qkv = torch.randn(T, 3 * H * D, device=dev, dtype=bf)
    dec = torch.full((H,), 0.97, device=dev)
    table = _rotary_table(D // 2, 1e6, L + 64, dev)
    rq, rk, rv = qkv.split(H * D, dim=-1)
    ms = ev(lambda: ops.retention(rq, rk, rv, state, rpi, H, D, D, dec, table, D // 2, D ** -0.5, prefix_lens=pre,
                                  extend_lens=ext, extend_start_loc=start))
    add(f"retention prefill {n_req}x{L} ({H}x{D})", "like: recurrence prefill", ms, flops=4.0 * H * D * D * T,
        peak_tf=BR.FP32_CORE_TFLOPS)
    qkvd = torch.randn(B, 3 * H * D, device=dev, dtype=bf)
    ms = ev(lambda: ops.retention(*qkvd.split(H * D, dim=-1), state, rpd, H, D, D, dec, table, D // 2, D ** -0.5,
                                  seq_lens=sl, out_cache_loc=loc))
    add(f"retention decode B={B} ({H}x{D})", "like: recurrence decode", ms, bytes_=B * H * D * D * 4 * 2)
    # ---- latent attention: every head against one latent row, beside the grouped attention of Rimidra ---------------
    slots = T + 256
    cp = torch.randn(slots, 1, R, device=dev, dtype=bf)
    r2t = torch.zeros(n_req + 64, L + 64, dtype=torch.int32, device=dev)
    for r in range(n_req):
        r2t[r, :L] = torch.arange(1 + r * L, 1 + (r + 1) * L, device=dev, dtype=torch.int32)
    ql = torch.randn(T, H * R, device=dev, dtype=bf)
    full = sum(i + 1 for i in range(L)) * n_req
    ms = ev(lambda: ops.attn_general(ql, cp, cp, r2t, rpi, H, 1, R, R, D ** -0.5, prefix_lens=pre, extend_lens=ext,
                                     extend_start_loc=start, max_extend_len=L))
    add(f"attn_general over the latent pool, prefill {n_req}x{L} ({H} heads, rank {R})", "", ms, flops=4.0 * H * R * full)
    G = z["kv_heads"]
    kp, vp = torch.randn(slots, G, D, device=dev, dtype=bf), torch.randn(slots, G, D, device=dev, dtype=bf)
    qa = torch.randn(T, H * D, device=dev, dtype=bf)
    ms = ev(lambda: ops.attn_general(qa, kp, vp, r2t, rpi, H, G, D, D, D ** -0.5, prefix_lens=pre, extend_lens=ext,
                                     extend_start_loc=start, max_extend_len=L))
    add(f"attn_general grouped heads, prefill {n_req}x{L} ({H}/{G}x{D}, no window)", "like: prefill attention", ms,
        flops=4.0 * H * D * full)
    r2d = torch.randint(1, slots, (B + 1, L + 64), device=dev, dtype=torch.int32)
    qd = torch.randn(B, H * R, device=dev, dtype=bf)
    ms = ev(lambda: ops.attn_general(qd, cp, cp, r2d, rpd, H, 1, R, R, D ** -0.5, seq_lens=sl))
    add(f"attn_general over the latent pool, decode B={B} ctx {L}", "", ms, bytes_=B * L * R * 2)
    qd2 = torch.randn(B, H * D, device=dev, dtype=bf)
    ms = ev(lambda: ops.attn_general(qd2, kp, vp, r2d, rpd, H, G, D, D, D ** -0.5, seq_lens=sl))
    add(f"attn_general grouped heads, decode B={B} ctx {L}", "like: decode attention", ms, bytes_=B * L * G * D * 2 * 2)
    # ---- row kernels -----------------------------------------------------------------------------------
    x32 = torch.randn(T, Wd, device=dev)
    a, b2 = torch.randn(T, Wd, device=dev, dtype=bf), torch.randn(T, Wd, device=dev, dtype=bf)
    w1, w2 = torch.ones(Wd, device=dev, dtype=bf), torch.ones(Wd, device=dev, dtype=bf)
    ms = ev(lambda: ops.residual_rmsnorm2(x32, w1, w2, 1e-6, a=a, b=b2))
    add(f"residual_rmsnorm2 (two norms) {T}x{Wd}", "", ms, bytes_=T * Wd * (4 + 4 + 2 + 2 + 2 + 2))
    ms = ev(lambda: ops.residual_rmsnorm(x32, w1, 1e-6, a=a, b=b2))
    add(f"residual_rmsnorm {T}x{Wd}", "like: norm", ms, bytes_=T * Wd * (4 + 4 + 2 + 2 + 2))
    mu = torch.rand(5, Wd, device=dev).to(bf)
    shift = torch.zeros(B + 1, Wd, device=dev)
    ms = ev(lambda: ops.token_shift_mix(a, mu, shift, rpi, prefix_lens=pre, extend_lens=ext, extend_start_loc=start,
                                        max_extend_len=L))
    add(f"token_shift_mix (5 mixes) {T}x{Wd}", "like: norm", ms, bytes_=T * Wd * 2 * 6)
    ids = torch.randint(0, VOCAB, (T,), device=dev)
    pos = torch.arange(T, device=dev) % L
    emb = torch.randn(VOCAB, Wd, device=dev, dtype=bf)
    hi, lo = _sinusoid_frequencies(Wd, dev)
    ms = ev(lambda: ops.embed_sincos(emb, ids, pos, hi, lo))
    add(f"embed_sincos {T}x{Wd}", "", ms, bytes_=T * Wd * 6)
    ms = ev(lambda: ops.embed_f32(emb, ids))
    add(f"embed_f32 {T}x{Wd}", "like: embedding", ms, bytes_=T * Wd * 6)
    up = torch.randn(T, z["ff"], device=dev, dtype=bf)
    ms = ev(lambda: ops.activation(up, "relu2"))
    add(f"activation relu2 {T}x{z['ff']}", "", ms, bytes_=T * z["ff"] * 2 * 2)
    gu = torch.randn(T, 2 * z["ff"], device=dev, dtype=bf)
    ms = ev(lambda: ops.silu_and_mul(gu))
    add(f"silu_and_mul {T}x{z['ff']}", "like: activation", ms, bytes_=T * z["ff"] * 2 * 3)
    o32 = torch.randn(T, H * D, device=dev)
    wn = torch.ones(D, device=dev, dtype=bf)
    ms = ev(lambda: ops.headnorm_gate(o32, qa, H, D, 1e-6, weight=wn))
    add(f"headnorm_gate with weight {T}x{H * D}", "", ms, bytes_=T * H * D * (4 + 2 + 2))
    ms = ev(lambda: ops.headnorm_gate(o32, qa, H, D, 1e-6))
    add(f"headnorm_gate {T}x{H * D}", "like: head norm", ms, bytes_=T * H * D * (4 + 2 + 2))
    gate = torch.randn(T, 8 * ((H + 7) // 8), device=dev, dtype=bf)
    ms = ev(lambda: ops.head_gate_sigmoid(qa, gate[:, :H], H, D))
    add(f"head_gate_sigmoid {T}x{H * D}", "like: activation", ms, bytes_=T * H * D * 2 * 2)
    pool = torch.zeros(slots, R, device=dev, dtype=bf)
    cw = torch.ones(R, device=dev, dtype=bf)
    wide = torch.randn(T, H * D + R + 8, device=dev, dtype=bf)
    locs = torch.arange(1, T + 1, device=dev)
    ms = ev(lambda: ops.rmsnorm_store(wide[:, H * D: H * D + R], cw, 1e-6, pool=pool, loc=locs))
    add(f"rmsnorm_store (norm into the cache) {T}x{R}", "like: norm", ms, bytes_=T * R * 2 * 2)
    # ---- routing ---------------------------------------------------------------------------------------
    E, k = z["experts"], z["top"]
    zl = torch.randn(T, E, device=dev)
    corr = torch.randn(E, device=dev) * 0.1
    ms = ev(lambda: ops.moe_route_scores(zl, E, k, "sigmoid", renormalize=True, correction=corr, num_groups=z["groups"],
                                         keep_groups=z["keep"]))
    add(f"moe_route_scores grouped {T}x{E}", "", ms, bytes_=T * E * 4 + T * k * 8)
    ms = ev(lambda: ops.moe_route_scores(zl, E, k, "sigmoid"))
    add(f"moe_route_scores {T}x{E}", "like: routing", ms, bytes_=T * E * 4 + T * k * 8)
    return rows


def run(sizes=("s", "m"), out=None, kernels=True):
    torch.cuda.set_device(0)
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")  # > L2, written between timed launches
    hbm, tf, src = BR.peaks()
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src, "fp32_core_tflops": BR.FP32_CORE_TFLOPS},
           "timing": "CUDA events, 3 warm-up launches, 160 MB written between timed launches", "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z, "models": {}}
        for label, cfg in (("llama", BR.llama_config(z)), ("rimidra-dense", BR.rimidra_config(z, False)),
                           ("rimidra-moe", BR.rimidra_config(z, True)), ("nupovik-dense", nupovik_config(z, False)),
                           ("nupovik-moe", nupovik_config(z, True))):
            entry["models"][label] = BR.model_throughput(cfg, n_prompts=4, prompt_len=2048, decode_bs=64, flush=flush)
            print(name, label, json.dumps(entry["models"][label]), file=sys.stderr, flush=True)
        if kernels:
            entry["kernels"] = kernel_table(z, flush)
            for r in entry["kernels"]:
                print(name, json.dumps(r), file=sys.stderr, flush=True)
        res["sizes"][name] = entry
    if out:
        with open(out, "w") as f:
            json.dump(res, f, indent=1)
    return res


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="s,m")
    ap.add_argument("--out", default="")
    ap.add_argument("--no-kernels", action="store_true")
    a = ap.parse_args()
    run(tuple(a.sizes.split(",")), a.out or None, not a.no_kernels)

"""Rimidra beside Llama at equal size: whole-model prefill / decode throughput through the worker
(ScheduleBatch → TpModelWorker, decode through the captured CUDA graphs) and the per-kernel times of
the mechanisms the family adds, each beside the like kernel of the Llama / DeepSeek paths, with the
fraction of the measured roofline.  Random weights, synthetic tokens.  `bench.py --family rimidra`
runs this; stand-alone: python scripts/bench_rimidra.py [--sizes s,m] [--out FILE]."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SIZES = {
    # name: width, layers, heads, kv_heads, head_dim, ff, window, experts, top, expert ff
    "s": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=128, ff=2816, window=512, experts=8, top=2, eff=704),
    "m": dict(width=2048, layers=8, heads=16, kv_heads=4, dim=128, ff=5632, window=1024, experts=16, top=2, eff=1408),
    "l": dict(width=4096, layers=8, heads=32, kv_heads=8, dim=128, ff=11008, window=2048, experts=16, top=2, eff=2816),
}
VOCAB = 32000
FP32_CORE_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12  # FMA units x 2 flop x max clock: the CUDA-core ceiling


def peaks():
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return pk["hbm_gbs"], pk["bf16_tflops"], "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, 1590.0, "fallback"


def rimidra_config(z, moe):
    from semi_pd_b200.configs import ModelConfig
    mlp = ({"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["eff"]},
            "shared": {"ff": z["eff"]}} if moe else {"kind": "dense", "ff": z["ff"]})
    ret = {"type": "retention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["dim"], "rot": {"dims": z["dim"] // 2, "base": 1e6},
                     "decay": [1.0 - 2.0 ** (-5 - 0.5 * h) for h in range(z["heads"])]}}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                     "mask": {"size": z["window"]}, "q_temp": {"coef": 0.3, "every": 128}, "scale": z["dim"] ** -0.5}}
    layers = [ret if i % 2 == 0 else att for i in range(z["layers"])]
    return ModelConfig(name="rimidra-bench", model_type="rimidra", hidden_size=z["width"], vocab_size=VOCAB,
                       num_hidden_layers=z["layers"], rms_norm_eps=1e-6, layer_specs=layers,
                       num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=z["dim"],
                       intermediate_size=0, max_position_embeddings=8192)


def llama_config(z):
    from semi_pd_b200.configs import ModelConfig
    return ModelConfig(name="llama-bench", hidden_size=z["width"], intermediate_size=z["ff"],
                       num_hidden_layers=z["layers"], num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
                       head_dim=z["dim"], vocab_size=VOCAB, max_position_embeddings=8192)


def event_ms(fn, iters=5, warm=3, flush=None):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def model_throughput(cfg, n_prompts, prompt_len, decode_bs, flush):
    """→ prefill tok/s (n_prompts x prompt_len in one extend batch) and decode tok/s (decode_bs requests
    at context prompt_len, CUDA-graph replay)."""
    from semi_pd_b200.configs import ServerArgs
    from semi_pd_b200.schedule_batch import Req, SamplingParams, ScheduleBatch
    from semi_pd_b200.tp_worker import TpModelWorker
    ctx = prompt_len + 64
    sa = ServerArgs(model_path=cfg.name, dtype="bfloat16", load_format="dummy",
                    max_total_tokens=(decode_bs + n_prompts) * (-(-ctx // 128) * 128) + 1024,
                    max_running_requests=decode_bs + n_prompts, context_length=ctx, cuda_graph_bs=[decode_bs])
    w = TpModelWorker(sa, 0, 0, model_config=cfg)
    pool, alloc = w.get_memory_pool()
    g = torch.Generator().manual_seed(1)

    def new_batch(n):
        reqs = [Req(f"r{i}", torch.randint(0, VOCAB, (prompt_len,), generator=g).tolist(), SamplingParams()) for i in range(n)]
        for r in reqs:
            r.init_next_round_input()
        b = ScheduleBatch.init_new(reqs, pool, alloc, w.device)
        b.prepare_for_extend()
        return b

    def release(b):
        for r in b.reqs:
            alloc.free_req(r.req_pool_idx)
            pool.free(r.req_pool_idx)

    # prefill: a fresh batch per timed launch (allocation outside the timed region)
    times = []
    for i in range(6):
        b = new_batch(n_prompts)
        mwb = b.get_model_worker_batch()
        flush.add_(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        w.forward_batch_generation(mwb)
        e1.record()
        e1.synchronize()
        if i >= 3:
            times.append(e0.elapsed_time(e1))
        release(b)
    prefill_ms = sum(times) / len(times)
    # decode: decode_bs requests prefilled in pieces, then timed graph replays
    dec = None
    for _ in range(decode_bs // n_prompts):
        b = new_batch(n_prompts)
        _, ids = w.forward_batch_generation(b.get_model_worker_batch())
        b.output_ids = ids.to(torch.int64)
        if dec is None:
            dec = b
        else:
            dec.merge_batch(b)

    def step():
        dec.prepare_for_decode()
        _, ids = w.forward_batch_generation(dec.get_model_worker_batch())
        dec.output_ids = ids.to(torch.int64)

    decode_ms = event_ms(step, iters=10, warm=3, flush=flush)
    release(dec)
    out = dict(prefill_tokens=n_prompts * prompt_len, prefill_ms=prefill_ms,
               prefill_tok_s=n_prompts * prompt_len / prefill_ms * 1e3, decode_bs=decode_bs, decode_ctx=prompt_len,
               decode_ms=decode_ms, decode_tok_s=decode_bs / decode_ms * 1e3)
    del w, dec
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def kernel_table(z, flush):
    """Per-kernel time of the family's mechanisms and of the like kernels of the existing paths."""
    from semi_pd_b200 import ops
    from semi_pd_b200.rimidra import _rotary_table
    hbm, tf, _ = peaks()
    dev = "cuda"
    H, G, D, Wd, win = z["heads"], z["kv_heads"], z["dim"], z["width"], z["window"]
    n_req, L = 4, 2048
    T = n_req * L
    bf = torch.bfloat16
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

    slots = T + 256
    kp = torch.randn(slots, G, D, device=dev, dtype=bf)
    vp = torch.randn(slots, G, D, device=dev, dtype=bf)
    r2t = torch.zeros(n_req + 64, L + 64, dtype=torch.int32, device=dev)
    for r in range(n_req):
        r2t[r, :L] = torch.arange(1 + r * L, 1 + (r + 1) * L, device=dev, dtype=torch.int32)
    rpi = torch.arange(n_req, device=dev, dtype=torch.int64)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    pre, ext, start = i32([0] * n_req), i32([L] * n_req), i32([r * L for r in range(n_req)])
    q = torch.randn(T, H * D, device=dev, dtype=bf)
    sinks = torch.zeros(H, device=dev)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
    # prefill attention
    vis = sum(min(i + 1, win) for i in range(L)) * n_req
    ms = event_ms(lambda: ops.attn_general(q, kp, vp, r2t, rpi, H, G, D, D, D ** -0.5, win, sinks, slopes, 0.3, 128,
                                           prefix_lens=pre, extend_lens=ext, extend_start_loc=start, max_extend_len=L),
                  flush=flush)
    add(f"attn_general prefill {n_req}x{L} window {win}", "", ms, flops=4.0 * H * D * vis)
    full = sum(i + 1 for i in range(L)) * n_req
    ms = event_ms(lambda: ops.attn_prefill(q, kp, vp, r2t, rpi, pre, ext, start, L, H, G, D, D ** -0.5), flush=flush)
    add(f"attn_prefill (tcgen05, causal) {n_req}x{L}", "like: prefill attention", ms, flops=4.0 * H * D * full)
    # decode attention, B requests at context L
    B = 64
    r2d = torch.randint(1, slots, (B + 1, L + 64), device=dev, dtype=torch.int32)
    rpd = torch.arange(B, device=dev, dtype=torch.int64)
    sl = torch.full((B,), L, dtype=torch.int64, device=dev)
    qd = torch.randn(B, H * D, device=dev, dtype=bf)
    ms = event_ms(lambda: ops.attn_general(qd, kp, vp, r2d, rpd, H, G, D, D, D ** -0.5, win, sinks, slopes, 0.3, 128,
                                           seq_lens=sl), flush=flush)
    add(f"attn_general decode B={B} window {win}", "", ms, bytes_=B * min(win, L) * G * D * 2 * 2)
    ms = event_ms(lambda: ops.attn_decode(qd, kp, vp, r2d, rpd, sl, H, G, D, D ** -0.5), flush=flush)
    add(f"attn_decode (tcgen05) B={B} ctx {L}", "like: decode attention", ms, bytes_=B * L * G * D * 2 * 2)
    # retention
    state = torch.zeros(B + 1, H, D, D, device=dev)
    qkv = torch.randn(T, 3 * H * D, device=dev, dtype=bf)
    dec = torch.full((H,), 0.97, device=dev)
    table = _rotary_table(D // 2, 1e6, L + 64, dev)
    rq, rk, rv = qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]
    ms = event_ms(lambda: ops.retention(rq, rk, rv, state, rpi, H, D, D, dec, table, D // 2, D ** -0.5, prefix_lens=pre,
                                        extend_lens=ext, extend_start_loc=start), flush=flush)
    add(f"retention prefill {n_req}x{L}", "like: prefill attention", ms, flops=4.0 * H * D * D * T, peak_tf=FP32_CORE_TFLOPS)
    qkvd = torch.randn(B, 3 * H * D, device=dev, dtype=bf)
    loc = torch.ones(B, dtype=torch.int64, device=dev)
    ms = event_ms(lambda: ops.retention(qkvd[:, :H * D], qkvd[:, H * D:2 * H * D], qkvd[:, 2 * H * D:], state, rpd, H, D, D,
                                        dec, table, D // 2, D ** -0.5, seq_lens=sl, out_cache_loc=loc), flush=flush)
    add(f"retention decode B={B}", "like: decode attention", ms, bytes_=B * H * D * D * 4 * 2)
    # norms and activations
    x32 = torch.randn(T, Wd, device=dev)
    a = torch.randn(T, Wd, device=dev, dtype=bf)
    b2 = torch.randn(T, Wd, device=dev, dtype=bf)
    wn = torch.zeros(Wd, device=dev, dtype=bf)
    ms = event_ms(lambda: ops.residual_rmsnorm(x32, wn, 1e-6, a=a, b=b2, weight_offset=1.0), flush=flush)
    add(f"residual_rmsnorm (fp32 stream) {T}x{Wd}", "", ms, bytes_=T * Wd * (4 + 4 + 2 + 2 + 2))
    xb, rb = torch.randn(T, Wd, device=dev, dtype=bf), torch.randn(T, Wd, device=dev, dtype=bf)
    ms = event_ms(lambda: ops.fused_add_rmsnorm(xb, rb, wn, 1e-6), flush=flush)
    add(f"fused_add_rmsnorm (bf16) {T}x{Wd}", "like: norm", ms, bytes_=T * Wd * 2 * 4)
    gu = torch.randn(T, 2 * z["ff"], device=dev, dtype=bf)
    ms = event_ms(lambda: ops.act_and_mul(gu, "gelu_tanh"), flush=flush)
    add(f"act_and_mul gelu {T}x{z['ff']}", "", ms, bytes_=T * z["ff"] * 2 * 3)
    ms = event_ms(lambda: ops.silu_and_mul(gu), flush=flush)
    add(f"silu_and_mul {T}x{z['ff']}", "like: activation", ms, bytes_=T * z["ff"] * 2 * 3)
    o32 = torch.randn(T, H * D, device=dev)
    ms = event_ms(lambda: ops.headnorm_gate(o32, q, H, D, 1e-6), flush=flush)
    add(f"headnorm_gate {T}x{H * D}", "like: norm", ms, bytes_=T * H * D * (4 + 2 + 2))
    # MoE plumbing
    E, k = z["experts"], z["top"]
    zl = torch.randn(T, E + 1, device=dev)
    ms = event_ms(lambda: ops.moe_route_scores(zl, E, k, "sigmoid"), flush=flush)
    add(f"moe_route_scores {T}x{E}", "", ms, bytes_=T * (E + 1) * 4 + T * k * 8)
    zb = torch.randn(T, E, device=dev, dtype=bf)
    ms = event_ms(lambda: ops.moe_route(zb, k), flush=flush)
    add(f"moe_route (softmax) {T}x{E}", "like: routing", ms, bytes_=T * E * 2 + T * k * 8)
    ids, wts = ops.moe_route_scores(zl, E, k, "sigmoid")
    row_token, inv_pos, tile_group = ops.moe_align(ids, E)
    R = row_token.numel()
    ms = event_ms(lambda: ops.moe_gather_scaled(a, row_token, inv_pos, wts), flush=flush)
    add(f"moe_gather_scaled {R}x{Wd}", "", ms, bytes_=(T * k + R) * Wd * 2)
    ms = event_ms(lambda: ops.moe_gather(a, row_token), flush=flush)
    add(f"moe_gather {R}x{Wd}", "like: gather", ms, bytes_=(T * k + R) * Wd * 2)
    y = torch.randn(R, Wd, device=dev, dtype=bf)
    ms = event_ms(lambda: ops.moe_combine_gated(y, inv_pos, T, k, shared=a, shared_gate=zl[:, E:]), flush=flush)
    add(f"moe_combine_gated {T}x{Wd}", "", ms, bytes_=T * Wd * 2 * (k + 2))
    ms = event_ms(lambda: ops.moe_combine(y, inv_pos, wts, a), flush=flush)
    add(f"moe_combine {T}x{Wd}", "like: combine", ms, bytes_=T * Wd * 2 * (k + 2))
    return rows


def run(sizes=("s", "m"), out=None, kernels=True):
    torch.cuda.set_device(0)
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")  # > L2, written between timed launches
    hbm, tf, src = peaks()
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src, "fp32_core_tflops": FP32_CORE_TFLOPS},
           "timing": "CUDA events, 3 warm-up launches, 160 MB written between timed launches", "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z, "models": {}}
        for label, cfg in (("llama", llama_config(z)), ("rimidra-dense", rimidra_config(z, False)),
                           ("rimidra-moe", rimidra_config(z, True))):
            entry["models"][label] = model_throughput(cfg, n_prompts=4, prompt_len=2048, decode_bs=64, flush=flush)
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

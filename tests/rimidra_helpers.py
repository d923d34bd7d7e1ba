"""Helpers of the Rimidra tests: write a model folder (config.json + model.safetensors) from an
oracle configuration and its random checkpoint, open a trace session of the product on it, and
compare logits the way a serving check would (mean over the vocabulary removed, RMS, relative)."""
import json
import os
import struct

import torch

from oracle import rimidra_oracle as R


def write_safetensors(path, tensors):
    """Minimal writer: 8-byte little-endian header length, JSON header, raw little-endian data."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        if t.is_floating_point():
            raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
            dt = "BF16"
        else:
            raw = t.to(torch.int32).contiguous().numpy().tobytes()
            dt = "I32"
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def write_model(folder, cfg, weights):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return str(folder)


def open_session(folder, dtype, max_tokens=1024, max_requests=4, cuda_graph=True):
    from semi_pd_b200.trace_runner import TraceSession, build_worker
    return TraceSession(build_worker(folder, dtype, max_tokens, max_requests, cuda_graph))


def rel_err(got, want):
    """Per row: RMS over the vocabulary of the mean-removed difference / RMS of the mean-removed reference."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-12)


TOL = {"float32": 3e-5, "bfloat16": 1e-1}


# ---- configurations (none has the sizes of a published or given model) -------------------------
def config_mixed():
    """retention + dense, attention + MoE(top 2, shared), both repeated with borrowed weights."""
    return R.make_config([
        R.retention_spec(heads=2, dim=16, vdim=32, rot_dims=8, base=10000.0, mlp=R.dense_mlp(48)),
        R.attention_spec(heads=4, kv_heads=2, dim=16, vdim=8, window=12, scale=0.3, coef=0.4, every=16,
                         mlp=R.moe_mlp(experts=4, top=2, ff=24, shared_ff=16)),
        R.retention_spec(heads=2, dim=16, vdim=32, rot_dims=8, base=10000.0, mlp=R.dense_mlp(48), weights_of=0),
        R.attention_spec(heads=4, kv_heads=2, dim=16, vdim=8, window=12, scale=0.3, coef=0.4, every=16,
                         mlp=R.moe_mlp(experts=4, top=2, ff=24, shared_ff=16), weights_of=1),
    ], width=64, vocab=96)


def config_ones():
    """Values that a usual model makes > 1 are 1 here: one head, one kv head, window 1, top 1, block
    length 1, no decay, full-width rotation; a layer without feed-forward; sizes off the GEMM tiles."""
    return R.make_config([
        R.attention_spec(heads=1, kv_heads=1, dim=8, vdim=8, window=1, scale=1.0, coef=0.1, every=1, mlp=None),
        R.retention_spec(heads=1, dim=8, vdim=8, decay=[1.0], rot_dims=8, base=100.0,
                         mlp=R.moe_mlp(experts=2, top=1, ff=8, shared_ff=0)),
        R.attention_spec(heads=2, kv_heads=1, dim=8, vdim=24, window=3, scale=0.5, coef=0.0, every=7,
                         mlp=R.dense_mlp(20)),
    ], width=40, vocab=50, eps=1e-5)


def config_wide():
    """attention first with a window longer than any prompt of the tests, 8:2 grouped heads, odd
    expert counts (router rows off the 8-multiple), three retention heads with different decays."""
    return R.make_config([
        R.attention_spec(heads=8, kv_heads=2, dim=32, vdim=32, window=512, scale=0.18, coef=0.3, every=50,
                         mlp=R.dense_mlp(96)),
        R.retention_spec(heads=3, dim=64, vdim=64, decay=[0.9, 0.99, 0.999], rot_dims=32, base=1e6,
                         mlp=R.moe_mlp(experts=5, top=3, ff=40, shared_ff=40)),
        R.attention_spec(heads=2, kv_heads=2, dim=64, vdim=64, window=130, scale=0.125, coef=0.3, every=128,
                         mlp=R.moe_mlp(experts=5, top=3, ff=40, shared_ff=40)),
    ], width=128, vocab=257)


def config_far():
    """A short window and a retention head that never forgets: what the first token says reaches
    position 300 and beyond only through the recurrent state."""
    return R.make_config([
        R.retention_spec(heads=2, dim=8, vdim=16, decay=[1.0, 0.9995], rot_dims=4, base=50.0, mlp=None),
        R.attention_spec(heads=2, kv_heads=1, dim=8, vdim=8, window=4, scale=0.35, coef=0.2, every=100,
                         mlp=R.dense_mlp(32)),
    ], width=32, vocab=64)


CONFIGS = {"mixed": config_mixed, "ones": config_ones, "wide": config_wide, "far": config_far}


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

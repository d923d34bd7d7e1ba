"""Plain, slow restatement of the Rimidra model family in float64 torch on the CPU — test
infrastructure only, one function per mechanism, sharing no code with semi_pd_b200.  Everything is
computed for a whole sequence at once (or, for the recurrence, token by token in a Python loop), so
any way of cutting, batching or caching the same tokens must reproduce these numbers.

Notation: x [T, W] residual stream; a layer computes u = N(x), x <- x + (Mix(u) + FF(u)), with
N(x) = x / sqrt(mean(x²) + eps) · (1 + w).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def offset_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef · ln(⌊(p + 1) / every⌋ + 1) per position."""
    return 1.0 + coef * torch.log(torch.floor((positions + 1.0) / every) + 1.0)


def distance_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


def windowed_sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int],
                            sinks: Optional[torch.Tensor], slopes: Optional[torch.Tensor],
                            q_temp: Optional[tuple] = None, first_position: int = 0) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of ONE sequence whose first row sits at position
    `first_position` (keys before it do not exist) → [T, H, dv].  Position i sees j with
    0 <= i − j < window; weight ∝ exp(q_i·k_j · scale · temp(i) − slope_h (i − j)); the denominator
    also holds exp(sink_h)."""
    T, H, _ = q.shape
    G = k.shape[1]
    pos = torch.arange(first_position, first_position + T, dtype=F64)
    if q_temp is not None:
        q = q * query_temperature(pos, q_temp[0], q_temp[1])[:, None, None]
    dist = pos[:, None] - pos[None, :]
    visible = dist >= 0
    if window is not None and window > 0:
        visible = visible & (dist < window)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if slopes is not None:
            s = s - slopes[h] * dist
        s = s.masked_fill(~visible, -math.inf)
        top = s.max(dim=-1, keepdim=True).values
        if sinks is not None:
            top = torch.maximum(top, sinks[h].to(F64))
        e = torch.exp(s - top)
        den = e.sum(dim=-1, keepdim=True)
        if sinks is not None:
            den = den + torch.exp(sinks[h].to(F64) - top)
        out[:, h] = (e / den) @ v[:, g]
    return out


def rotate_half_partial(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, H, d]: dimension i < dims/2 pairs with i + dims/2; (a, b) -> (a cos − b sin, b cos + a sin)
    with angle p · base^(−2i/dims); dimensions >= dims pass through."""
    if dims <= 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def retention_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float],
                         state: Optional[torch.Tensor] = None):
    """q, k [T, H, dk] (already rotated / scaled), v [T, H, dv]; S_t = γ_h S_{t−1} + k_t v_tᵀ, o_t = S_tᵀ q_t,
    token by token.  → (o [T, H, dv], final state [H, dk, dv])."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state.clone()
    gamma = torch.tensor(decay, dtype=F64)[:, None, None]
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = gamma * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def gated_ffn(u: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act) -> torch.Tensor:
    return (act(u @ gate.T) * (u @ up.T)) @ down.T


def sigmoid_topk_routing(u: torch.Tensor, router: torch.Tensor, top: int):
    """→ (expert ids [T, top], weights [T, top]) — the largest sigmoid scores, NOT renormalised."""
    scores = torch.sigmoid(u @ router.T)
    w, ids = torch.topk(scores, top, dim=-1)
    return ids, w


# ---------------------------------------------------------------------------------------------
# sublayers by checkpoint names
# ---------------------------------------------------------------------------------------------
def attention_mixer(u, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    T = u.shape[0]
    H, G = m["heads"], m.get("kv_heads", m["heads"])
    dk, dv = m["dim"], m.get("vdim", m["dim"])
    q = (u @ W[p + "q"].T).view(T, H, dk)
    k = (u @ W[p + "k"].T).view(T, G, dk)
    v = (u @ W[p + "v"].T).view(T, G, dv)
    qt = m.get("q_temp")
    o = windowed_sink_attention(q, k, v, m["scale"], (m.get("mask") or {}).get("size"), W.get(p + "sink"),
                                distance_slopes(H), (qt["coef"], qt["every"]) if qt else None)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def retention_mixer(u, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = u.shape[0]
    H, dk, dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rotate_half_partial((u @ W[p + "q"].T).view(T, H, dk), pos, rot.get("dims", 0), rot.get("base", 1e4))
    k = rotate_half_partial((u @ W[p + "k"].T).view(T, H, dk), pos, rot.get("dims", 0), rot.get("base", 1e4))
    k = k * dk ** -0.5
    v = (u @ W[p + "v"].T).view(T, H, dv)
    o, _ = retention_recurrence(q, k, v, m["decay"])
    o = unit_rms(o, eps).reshape(T, H * dv) * silu(u @ W[p + "g"].T)
    return o @ W[p + "o"].T


def feed_forward(u, W: Dict[str, torch.Tensor], p: str, m: Optional[dict]):
    if m is None:
        return torch.zeros_like(u)
    if m["kind"] == "dense":
        return gated_ffn(u, W[p + "gate"], W[p + "up"], W[p + "down"], gelu_tanh)
    E, top = m["router"]["experts"], m["router"]["top"]
    ids, w = sigmoid_topk_routing(u, W[p + "router"], top)
    out = torch.zeros_like(u)
    for e in range(E):
        for j in range(top):
            sel = ids[:, j] == e
            if sel.any():
                xin = w[sel, j][:, None] * u[sel]  # the weight scales the expert's INPUT
                out[sel] += gated_ffn(xin, W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"], W[f"{p}e{e}.down"], silu)
    if m.get("shared"):
        sh = gated_ffn(u, W[p + "shared.gate"], W[p + "shared.up"], W[p + "shared.down"], silu)
        out = out + sh * torch.sigmoid(u @ W[p + "shared.sg"].T)
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence; `residuals` collects x after every layer."""
    W = {n: (t.to(F64) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i) if layer.get('weights_of') is not None else i}."
        u = offset_rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "attention":
            mix = attention_mixer(u, W, p + "mix.", layer["mixer"])
        else:
            mix = retention_mixer(u, W, p + "mix.", layer["mixer"], eps)
        x = x + (mix + feed_forward(u, W, p + "mlp.", layer.get("mlp")))
        if residuals is not None:
            residuals.append(x.clone())
    return offset_rms_norm(x, W["final.norm"], eps) @ W["head"].T


# ---------------------------------------------------------------------------------------------
# small configurations and random checkpoints for the tests
# ---------------------------------------------------------------------------------------------
def attention_spec(heads=4, kv_heads=2, dim=16, vdim=16, window=12, scale=0.25, coef=0.25, every=16, mlp=None,
                   weights_of=None):
    s = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                        "mask": {"size": window}, "q_temp": {"coef": coef, "every": every},
                                        "scale": scale}, "mlp": mlp}
    if weights_of is not None:
        s["weights_of"] = weights_of
    return s


def retention_spec(heads=2, dim=16, vdim=16, decay=None, rot_dims=8, base=10000.0, mlp=None, weights_of=None):
    s = {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                        "decay": decay or [1.0 - 2.0 ** (-4 - h) for h in range(heads)],
                                        "rot": {"dims": rot_dims, "base": base}}, "mlp": mlp}
    if weights_of is not None:
        s["weights_of"] = weights_of
    return s


def dense_mlp(ff=48):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=4, top=2, ff=24, shared_ff=24):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def make_config(layers: List[dict], width=64, vocab=96, eps=1e-6) -> dict:
    return {"architecture": "Rimidra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    Wd, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (Wd,)
        dk, dv = m["dim"], m.get("vdim", m["dim"])
        if layer["type"] == "attention":
            H, G = m["heads"], m.get("kv_heads", m["heads"])
            out.update({p + "mix.q": (H * dk, Wd), p + "mix.k": (G * dk, Wd), p + "mix.v": (G * dv, Wd),
                        p + "mix.sink": (H,), p + "mix.o": (Wd, H * dv)})
        else:
            H = m["heads"]
            out.update({p + "mix.q": (H * dk, Wd), p + "mix.k": (H * dk, Wd), p + "mix.v": (H * dv, Wd),
                        p + "mix.g": (H * dv, Wd), p + "mix.o": (Wd, H * dv)})
        f = layer.get("mlp")
        if f is None:
            continue
        if f["kind"] == "dense":
            out.update({p + "mlp.gate": (f["ff"], Wd), p + "mlp.up": (f["ff"], Wd), p + "mlp.down": (Wd, f["ff"])})
        else:
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                out.update({f"{p}mlp.e{e}.gate": (ff, Wd), f"{p}mlp.e{e}.up": (ff, Wd), f"{p}mlp.e{e}.down": (Wd, ff)})
            out[p + "mlp.router"] = (f["router"]["experts"], Wd)
            if f.get("shared"):
                sf = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, Wd), p + "mlp.shared.up": (sf, Wd),
                            p + "mlp.shared.down": (Wd, sf), p + "mlp.shared.sg": (1, Wd)})
    out["final.norm"] = (Wd,)
    out["head"] = (cfg["vocab"], Wd)
    return out


def make_weights(cfg: dict, seed: int = 0, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random checkpoint, values exactly representable in bfloat16 (stored as float32): projections
    N(0, gain²/fan_in) (router rows larger, so that routing margins are wide), norm weights and sinks
    N(0, 0.3²)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            t = torch.randn(shape, generator=g) * 0.3
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = torch.randn(shape, generator=g) * 4.0 / math.sqrt(shape[-1])
        else:
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out

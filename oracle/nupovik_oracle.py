"""Plain float64 statement of the Nupovik design, one function per mechanism, token by token where
the design is recurrent.  Slow on purpose; shares no code with the package.  Weights are a dict by
checkpoint name (any float dtype, read as float64), `cfg` is the parsed config.json.

Notation: h is a mixer's (normed) input [T, width]; H heads; dk key size, dv value size per head.
"""
import math

import torch

F64 = torch.float64


def f64(t):
    return t.to(F64)


# ---- small pieces --------------------------------------------------------------------------------
def rms_norm(x, w, eps):
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * f64(w)


def silu(x):
    return x * torch.sigmoid(x)


def relu_sq(x):
    return torch.relu(x).pow(2)


def position_vector(positions, width):
    """[n, width]: even entries sin(p f_i), odd entries cos(p f_i), f_i = 10000^(-2 i / width)."""
    p = torch.as_tensor(positions, dtype=F64).reshape(-1, 1)
    i = torch.arange((width + 1) // 2, dtype=F64)
    ang = p * torch.pow(torch.tensor(10000.0, dtype=F64), -2.0 * i / width)
    out = torch.zeros(p.shape[0], width, dtype=F64)
    out[:, 0::2] = ang.sin()
    out[:, 1::2] = ang.cos()[:, : width // 2]
    return out


def embed(w, tokens, first_position=0):
    E = f64(w["embed"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    return E[tok] + position_vector(range(first_position, first_position + len(tok)), E.shape[1])


# ---- recurrences ---------------------------------------------------------------------------------
def sigmoid_pow_decay(z, tau):
    return torch.sigmoid(z).pow(1.0 / tau)


def double_exp_decay(z):
    return torch.exp(-torch.exp(z))


def decay_recurrence(q, k, v, w, S):
    """q, k, w [T, H, dk], v [T, H, dv], S [H, dk, dv]: S <- diag(w_t) S + k_t v_tᵀ, o_t = Sᵀ q_t (the new S)."""
    o = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=F64)
    for t in range(q.shape[0]):
        S = w[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def bonus_recurrence(r, k, v, w, u, S):
    """o_t = (S + diag(u) k_t v_tᵀ)ᵀ r_t with the old S, then S <- diag(w_t) S + k_t v_tᵀ.  u [H, dk]."""
    o = torch.zeros(r.shape[0], r.shape[1], v.shape[2], dtype=F64)
    for t in range(r.shape[0]):
        kv = k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S + u.unsqueeze(-1) * kv, r[t])
        S = w[t].unsqueeze(-1) * S + kv
    return o, S


def token_shift(h, prev, mu):
    """h [T, W], prev [W] (the row before h[0]), mu [n, W] → [n, T, W]."""
    shifted = torch.cat([prev.view(1, -1), h[:-1]], 0)
    return h.unsqueeze(0) + (shifted - h).unsqueeze(0) * mu.unsqueeze(1)


# ---- mixers --------------------------------------------------------------------------------------
def gla_mixer(h, w, p, m, eps, state=None):
    """Gated linear attention.  state: [H, dk, dv] or None (zeros); → (out [T, width], state)."""
    H, dk, dv, tau = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), float(m["tau"])
    T = h.shape[0]
    q = (h @ f64(w[p + "q"]).T).view(T, H, dk) * dk ** -0.5
    k = (h @ f64(w[p + "k"]).T).view(T, H, dk)
    v = (h @ f64(w[p + "v"]).T).view(T, H, dv)
    z = (h @ f64(w[p + "a1"]).T) @ f64(w[p + "a2"]).T + f64(w[p + "a2.b"])
    alpha = sigmoid_pow_decay(z, tau).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state.clone()
    o, S = decay_recurrence(q, k, v, alpha, S)
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ f64(w[p + "g"]).T)) @ f64(w[p + "o"]).T, S


def latent_attention_mixer(h, w, p, m, eps, cache=None):
    """Attention through a low-rank latent, no positions.  cache: the latents of earlier tokens
    [P, kv_rank] or None; → (out, cache with this call's latents appended)."""
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    scale = float(m["scale"])
    T = h.shape[0]
    q = (h @ f64(w[p + "q"]).T).view(T, H, dk)
    c = rms_norm(h @ f64(w[p + "dkv"]).T, w[p + "dkv.norm"], eps)
    c_all = c if cache is None else torch.cat([cache, c], 0)
    P = c_all.shape[0] - T
    k = (c_all @ f64(w[p + "uk"]).T).view(-1, H, dk)
    v = (c_all @ f64(w[p + "uv"]).T).view(-1, H, dv)
    s = torch.einsum("thd,jhd->htj", q, k) * scale
    i = torch.arange(T).view(T, 1) + P
    j = torch.arange(P + T).view(1, -1)
    s = s.masked_fill(~(j <= i).unsqueeze(0), -math.inf)
    o = torch.einsum("htj,jhd->thd", torch.softmax(s, -1), v)
    o = o * torch.sigmoid(h @ f64(w[p + "g"]).T).unsqueeze(-1)
    return o.reshape(T, H * dv) @ f64(w[p + "o"]).T, c_all


def wkv_mixer(h, w, p, m, eps, state=None):
    """Time mixing with a token shift.  state: (S [H, dk, dk], previous h [width]) or None."""
    H, dk = int(m["heads"]), int(m["dim"])
    T, width = h.shape
    S, prev = (torch.zeros(H, dk, dk, dtype=F64), torch.zeros(width, dtype=F64)) if state is None else \
        (state[0].clone(), state[1].clone())
    mixes = token_shift(h, prev, torch.stack([f64(w[p + "mu." + s]) for s in "rkvgw"]))

    def mixed(s):
        return mixes["rkvgw".index(s)]

    r = (mixed("r") @ f64(w[p + "r"]).T).view(T, H, dk)
    k = (mixed("k") @ f64(w[p + "k"]).T).view(T, H, dk)
    v = (mixed("v") @ f64(w[p + "v"]).T).view(T, H, dk)
    gate = silu(mixed("g") @ f64(w[p + "g"]).T)
    dec = double_exp_decay(torch.tanh(mixed("w") @ f64(w[p + "w1"]).T) @ f64(w[p + "w2"]).T + f64(w[p + "w0"]))
    o, S = bonus_recurrence(r, k, v, dec.view(T, H, dk), f64(w[p + "u"]).view(H, dk), S)
    o = rms_norm(o, None, eps).reshape(T, H * dk) * f64(w[p + "norm"])
    return (o * gate) @ f64(w[p + "o"]).T, (S, h[-1].clone())


# ---- feed-forwards -------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return relu_sq(h @ f64(w[p + "up"]).T) @ f64(w[p + "down"]).T


def route(h, w, p, r):
    """→ (ids [T, top], weights [T, top]) of the grouped sigmoid router."""
    return route_logits(h @ f64(w[p + "router"]).T, f64(w[p + "correction"]), r)


def route_logits(z, correction, r):
    E, top = int(r["experts"]), int(r["top"])
    G, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
    s = torch.sigmoid(z)
    choice = s + correction
    per = E // G
    grouped = choice.view(-1, G, per)
    gscore = grouped.topk(min(2, per), -1).values.sum(-1)
    kept = gscore.topk(keep, -1).indices
    mask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, kept, True)
    choice = grouped.masked_fill(~mask.unsqueeze(-1), -math.inf).reshape(-1, E)
    ids = choice.topk(top, -1).indices
    sw = s.gather(1, ids)
    return ids, sw / (sw.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, w, p, mlp):
    ids, wt = route(h, w, p, mlp["router"])
    out = torch.zeros(h.shape[0], f64(w[p + "e0.down"]).shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += wt[t, j] * (relu_sq(h[t] @ f64(w[f"{p}e{e}.up"]).T) @ f64(w[f"{p}e{e}.down"]).T)
    return out


# ---- the model -----------------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer index, starts a pass)] in execution order."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(L)]
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for _ in range(n):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, L)]


class Stepper:
    """A sequence fed in portions: keeps the cache / state of every layer run."""

    def __init__(self, cfg, w):
        self.cfg, self.w = cfg, w
        self.runs = layer_runs(cfg)
        self.mem = [None] * len(self.runs)
        self.n = 0

    def feed(self, tokens, residuals=None):
        """→ logits [len(tokens), vocab]; residuals (a list) receives x after every layer run."""
        cfg, w = self.cfg, self.w
        eps = float(cfg["norm"]["eps"])
        x0 = embed(w, tokens, self.n)
        self.n += len(tokens)
        x = x0
        for r, (i, opens) in enumerate(self.runs):
            spec, p = cfg["layers"][i], f"l{i}."
            if opens:
                x = torch.cat([x, x0], -1) @ f64(w["loop.in"]).T
            hm = rms_norm(x, w[p + "norm1"], eps)
            fn = {"gla": gla_mixer, "latent_attention": latent_attention_mixer, "wkv": wkv_mixer}[spec["type"]]
            mix, self.mem[r] = fn(hm, w, p + "mix.", spec["mixer"], eps, self.mem[r])
            mlp = spec.get("mlp")
            if mlp is not None:
                hf = rms_norm(x, w[p + "norm2"], eps)
                ff = dense_ff(hf, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(hf, w, p + "mlp.", mlp)
                mix = mix + ff
            x = x + mix
            if residuals is not None:
                residuals.append(x.clone())
        return (rms_norm(x, w["final.norm"], eps) @ f64(w["head"]).T) * float(cfg.get("logit_scale", 1.0))


def forward(cfg, w, tokens, residuals=None):
    return Stepper(cfg, w).feed(tokens, residuals)


# ---- configurations and random checkpoints for tests ---------------------------------------------
def dense_mlp(ff):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts, top, ff, groups=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def latent_spec(heads, dim, vdim, kv_rank, scale, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}}


def gla_spec(heads, dim, vdim, tau, mlp=None):
    return {"type": "gla", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def wkv_spec(heads, dim, mlp=None):
    return {"type": "wkv", "mlp": mlp, "mixer": {"heads": heads, "dim": dim}}


def make_config(layers, width, vocab, loop=None, eps=1e-6, logit_scale=None):
    cfg = {"architecture": "Nupovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


def make_weights(cfg, seed=0, low_rank=8, slow_decay=False):
    """A random checkpoint by tensor name, values rounded to bfloat16.  slow_decay: decays close to 1, so
    that what the first tokens wrote into a recurrent state still counts hundreds of tokens later."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    w = {}

    def mat(n, k, gain=1.0):
        return torch.randn(n, k, generator=g) * gain / math.sqrt(k)

    def vec(n, mean=0.0, std=0.1):
        return mean + torch.randn(n, generator=g) * std

    w["embed"], w["head"], w["final.norm"] = torch.randn(V, W, generator=g), mat(V, W), vec(W, 1.0)
    if cfg.get("loop"):
        w["loop.in"] = mat(W, 2 * W, math.sqrt(2.0))
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        H, dk = m["heads"], m["dim"]
        w[p + "norm1"] = vec(W, 1.0)
        if spec["type"] == "latent_attention":
            dv, r = m["vdim"], m["kv_rank"]
            w.update({p + "mix.q": mat(H * dk, W), p + "mix.dkv": mat(r, W), p + "mix.dkv.norm": vec(r, 1.0),
                      p + "mix.uk": mat(H * dk, r), p + "mix.uv": mat(H * dv, r), p + "mix.g": mat(H, W, 2.0),
                      p + "mix.o": mat(W, H * dv)})
        elif spec["type"] == "gla":
            dv = m.get("vdim", dk)
            w.update({p + "mix.q": mat(H * dk, W), p + "mix.k": mat(H * dk, W), p + "mix.v": mat(H * dv, W),
                      p + "mix.g": mat(H * dv, W), p + "mix.o": mat(W, H * dv), p + "mix.norm": vec(dv, 1.0),
                      p + "mix.a1": mat(low_rank, W), p + "mix.a2": mat(H * dk, low_rank),
                      p + "mix.a2.b": vec(H * dk, 6.0 if slow_decay else 1.0, 1.0)})
        else:
            for s in "rkvgw":
                w[p + "mix.mu." + s] = torch.rand(W, generator=g)
            w.update({p + "mix.r": mat(H * dk, W), p + "mix.k": mat(H * dk, W), p + "mix.v": mat(H * dk, W),
                      p + "mix.g": mat(H * dk, W), p + "mix.w1": mat(low_rank, W), p + "mix.w2": mat(H * dk, low_rank),
                      p + "mix.w0": vec(H * dk, -7.0 if slow_decay else -2.0, 1.0), p + "mix.u": vec(H * dk, 0.5, 0.5).view(H, dk),
                      p + "mix.norm": vec(H * dk, 1.0), p + "mix.o": mat(W, H * dk)})
        mlp = spec.get("mlp")
        if mlp is None:
            continue
        w[p + "norm2"] = vec(W, 1.0)
        if mlp["kind"] == "dense":
            w.update({p + "mlp.up": mat(mlp["ff"], W), p + "mlp.down": mat(W, mlp["ff"])})
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                w.update({f"{p}mlp.e{e}.up": mat(ff, W), f"{p}mlp.e{e}.down": mat(W, ff)})
            w.update({p + "mlp.router": mat(E, W, 2.0), p + "mlp.correction": vec(E, 0.0, 0.5)})
    return {k: v.to(torch.bfloat16) for k, v in w.items()}

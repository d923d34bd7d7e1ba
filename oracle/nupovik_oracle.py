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
    i = torch.arange(width // 2, dtype=F64)
    ang = p * torch.pow(torch.tensor(10000.0, dtype=F64), -2.0 * i / width)
    out = torch.zeros(p.shape[0], width, dtype=F64)
    out[:, 0::2] = ang.sin()
    out[:, 1::2] = ang.cos()
    return out


def embed(w, tokens, first_position=0):
    E = f64(w["embed"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    return E[tok] + position_vector(range(first_position, first_position + len(tok)), E.shape[1])


# ---- mixers --------------------------------------------------------------------------------------
def gla_mixer(h, w, p, m, eps, state=None):
    """Gated linear attention.  state: [H, dk, dv] or None (zeros); → (out [T, width], state)."""
    H, dk, dv, tau = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), float(m["tau"])
    T = h.shape[0]
    q = (h @ f64(w[p + "q"]).T).view(T, H, dk) * dk ** -0.5
    k = (h @ f64(w[p + "k"]).T).view(T, H, dk)
    v = (h @ f64(w[p + "v"]).T).view(T, H, dv)
    z = (h @ f64(w[p + "a1"]).T) @ f64(w[p + "a2"]).T + f64(w[p + "a2.b"])
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
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
    shifted = torch.cat([prev.view(1, -1), h[:-1]], 0)

    def mixed(s):
        return h + (shifted - h) * f64(w[p + "mu." + s])

    r = (mixed("r") @ f64(w[p + "r"]).T).view(T, H, dk)
    k = (mixed("k") @ f64(w[p + "k"]).T).view(T, H, dk)
    v = (mixed("v") @ f64(w[p + "v"]).T).view(T, H, dk)
    gate = silu(mixed("g") @ f64(w[p + "g"]).T)
    dec = torch.exp(-torch.exp(torch.tanh(mixed("w") @ f64(w[p + "w1"]).T) @ f64(w[p + "w2"]).T + f64(w[p + "w0"])))
    dec = dec.view(T, H, dk)
    u = f64(w[p + "u"]).view(H, dk)
    o = torch.zeros(T, H, dk, dtype=F64)
    for t in range(T):
        kv = k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S + u.unsqueeze(-1) * kv, r[t])
        S = dec[t].unsqueeze(-1) * S + kv
    o = rms_norm(o, None, eps).reshape(T, H * dk) * f64(w[p + "norm"])
    return (o * gate) @ f64(w[p + "o"]).T, (S, h[-1].clone())


# ---- feed-forwards -------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return relu_sq(h @ f64(w[p + "up"]).T) @ f64(w[p + "down"]).T


def route(h, w, p, r):
    """→ (ids [T, top], weights [T, top]) of the grouped sigmoid router."""
    E, top = int(r["experts"]), int(r["top"])
    G, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
    s = torch.sigmoid(h @ f64(w[p + "router"]).T)
    choice = s + f64(w[p + "correction"])
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

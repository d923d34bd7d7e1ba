"""Nupovik wiring — a hybrid decoder family behind the same ModelRunner / ForwardBatch / AttentionBackend
surface as llama.py and rimidra.py.  Every size and constant comes from the model's config
(`ModelConfig.layer_specs`, one entry per layer RUN).

    x  = embed[token] + sinusoid(position)                       fp32 residual stream, x0 = this x
    a block of layers may be repeated back to back, re-using its tensors (every repetition keeps a cache /
    state to itself); a repetition opens with  x = pass_in · concat(x, x0)
    layer:  x <- x + (mixer(norm1(x)) + ff(norm2(x)))            parallel, one RMS norm weight per sublayer
    logits = head · norm(x) · logit_scale

mixers
  latent_attention  causal softmax attention with no positional term, through a low-rank latent: the cache
                    holds the normed latent c = norm(W_dkv h) alone (one row of kv_rank per token); keys and values are
                    W_uk c, W_uv c per head.  The product runs the absorbed form: q_h is carried into the
                    latent space (W_uk_hᵀ q_h), the general attention kernel scores it against the latent pool
                    with every query head sharing the one latent "head", and W_uv_h lifts the result; a
                    per-head sigmoid gate read from the mixer's input multiplies the heads.
  gla               gated linear attention, S_t = diag(a_t) S_(t-1) + k_t v_tᵀ, o_t = S_tᵀ q_t dim^-1/2, with
                    a_t = sigmoid(low-rank projection + bias)^(1/tau) per key channel; per-head RMS norm with
                    a weight shared by the heads, SiLU output gate.
  wkv               time mixing with a token shift: five inputs h + (h_prev − h) · mu_s, decay
                    exp(−exp(W_w2 tanh(W_w1 ·) + w0)) per key channel, a bonus u on the token being read,
                    o_t = (S_(t-1) + diag(u) k_t v_tᵀ)ᵀ r_t; per-head RMS norm, a weight per channel, SiLU gate.
feed-forwards: dense W_down relu(W_up h)², or a mixture of such experts routed by sigmoid scores with a
correction that enters the selection only, a group limit (top-ranked groups stay eligible) and renormalised weights.

Kernels: tcgen05 GEMMs (ops.linear*, grouped and block-diagonal forms) for 16-bit aligned shapes, the CUDA-core
GEMM otherwise (float32 models, odd sizes); csrc/gated_recurrence.cu for both recurrences (decay computed in
the kernel from the raw projection) and the token shift; csrc/attn_general*.cu over the latent pool; the
residual add of layer i fused with the two norms of layer i + 1.  Softmax, norms, routing, the residual
stream, decays and recurrent state are fp32 in every dtype.  Single GPU.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import ops
from .attention_backend import RadixAttention
from .forward_batch_info import ForwardBatch, LogitsProcessorOutput
from .layers import LogitsProcessor


class _W:
    """A weight holder (same role as layers.LinearBase, without TP sharding)."""

    def __init__(self):
        self.weight: torch.Tensor = None


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


def _sinusoid_frequencies(width: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """f_i = 10000^(-2 i / width) in float64, split into an fp32 value and its fp32 rounding residue."""
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / width)
    hi = f.to(torch.float32)
    lo = (f - hi.double()).to(torch.float32)
    return hi.to(device).contiguous(), lo.to(device).contiguous()


class NupovikLatentAttention:
    """Latent attention mixer.  q ‖ latent ‖ gate are one GEMM (rows padded to a multiple of 8); the latent
    slice is normed straight into the cache pool."""

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float):
        self.layer_id, self.eps = layer_id, eps
        self.heads, self.dim, self.vdim, self.rank = int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"])
        self.q_size = self.heads * self.dim
        self.qcg_proj, self.c_norm, self.uk_t, self.uv, self.o_proj = _W(), _W(), _W(), _W(), _W()
        # every query head reads the one latent row: keys are the row, values are the row
        self.attn = RadixAttention(self.heads, self.rank, float(m["scale"]), num_kv_heads=1, layer_id=layer_id,
                                   v_head_dim=self.rank, general=True)

    def share(self, other: "NupovikLatentAttention"):
        self.qcg_proj, self.c_norm, self.uk_t, self.uv, self.o_proj = \
            other.qcg_proj, other.c_norm, other.uk_t, other.uv, other.o_proj

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        qcg = ops.linear_any(h, self.qcg_proj.weight)
        q = qcg[:, : self.q_size]
        c_raw = qcg[:, self.q_size: self.q_size + self.rank]
        g = qcg[:, self.q_size + self.rank: self.q_size + self.rank + self.heads]
        pool = forward_batch.token_to_kv_pool.get_key_buffer(self.layer_id)
        ops.rmsnorm_store(c_raw, self.c_norm.weight, self.eps, pool=pool.view(pool.shape[0], -1),
                          loc=forward_batch.out_cache_loc)
        q_lat = ops.linear_block_diag_any(q, self.uk_t.weight, self.heads, self.dim, self.rank)
        o_lat = self.attn(q_lat, None, None, forward_batch, save_kv_cache=False)
        o = ops.linear_block_diag_any(o_lat, self.uv.weight, self.heads, self.rank, self.vdim)
        return ops.linear_any(ops.head_gate_sigmoid(o, g, self.heads, self.vdim), self.o_proj.weight)

    __call__ = forward


class NupovikGLA:
    """Gated linear attention mixer.  q ‖ k ‖ v ‖ g ‖ (low-rank decay input) are one GEMM."""

    form = "sigmoid_pow"
    bonus = None

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float):
        self.layer_id, self.eps = layer_id, eps
        self.num_heads, self.head_dim = int(m["heads"]), int(m["dim"])
        self.v_head_dim = int(m.get("vdim", m["dim"]))
        self.tau = float(m["tau"])
        self.q_scale = self.head_dim ** -0.5
        self.qk_size, self.v_size = self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        self.in_proj, self.a2, self.a2_bias, self.norm, self.o_proj = _W(), _W(), _W(), _W(), _W()

    @property
    def z_bias(self) -> torch.Tensor:  # fp32 [heads · dim]
        return self.a2_bias.weight

    def share(self, other: "NupovikGLA"):
        self.in_proj, self.a2, self.a2_bias, self.norm, self.o_proj = \
            other.in_proj, other.a2, other.a2_bias, other.norm, other.o_proj

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        y = ops.linear_any(h, self.in_proj.weight)
        q, k, v, g, a = y.split([self.qk_size, self.qk_size, self.v_size, self.v_size,
                                 y.shape[1] - 2 * self.qk_size - 2 * self.v_size], dim=-1)
        # the decay's low-rank input: as many columns as the second projection reads
        z = ops.linear_any(a[:, : self.a2.weight.shape[1]], self.a2.weight)
        o = forward_batch.attn_backend.forward_gated_recurrence(q, k, v, z, self, forward_batch)
        y = ops.headnorm_gate(o, g, self.num_heads, self.v_head_dim, self.eps, weight=self.norm.weight)
        return ops.linear_any(y, self.o_proj.weight)

    __call__ = forward


class NupovikWKV:
    """Token-shift time mixing.  The five mixes come from one kernel (which also keeps the previous token's
    input in the layer's vector state); r, k, v, g and the decay's first projection each read their own."""

    form = "double_exp"
    tau = 1.0
    q_scale = 1.0

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float):
        self.layer_id, self.eps, self.hidden = layer_id, eps, hidden
        self.num_heads, self.head_dim = int(m["heads"]), int(m["dim"])
        self.v_head_dim = self.head_dim
        self.mu, self.r, self.k, self.v, self.g, self.w1, self.w2, self.norm, self.o_proj = (_W() for _ in range(9))
        self.w0, self.u = _W(), _W()  # fp32 [heads · dim] each

    _TENSORS = ("mu", "r", "k", "v", "g", "w1", "w2", "norm", "o_proj", "w0", "u")

    @property
    def z_bias(self) -> torch.Tensor:
        return self.w0.weight

    @property
    def bonus(self) -> torch.Tensor:
        return self.u.weight

    def share(self, other: "NupovikWKV"):
        for n in self._TENSORS:
            setattr(self, n, getattr(other, n))

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        mr, mk, mv, mg, mw = forward_batch.attn_backend.forward_token_shift(h, self.mu.weight, self, forward_batch)
        r = ops.linear_any(mr, self.r.weight)
        k = ops.linear_any(mk, self.k.weight)
        v = ops.linear_any(mv, self.v.weight)
        g = ops.linear_any(mg, self.g.weight)
        z = ops.linear_any(ops.activation(ops.linear_any(mw, self.w1.weight), "tanh"), self.w2.weight)
        o = forward_batch.attn_backend.forward_gated_recurrence(r, k, v, z, self, forward_batch)
        y = ops.headnorm_gate(o, g, self.num_heads, self.head_dim, self.eps, weight=self.norm.weight)
        return ops.linear_any(y, self.o_proj.weight)

    __call__ = forward


class NupovikDenseMLP:
    def __init__(self, hidden: int, m: dict):
        self.ff = int(m["ff"])
        self.up_proj, self.down_proj = _W(), _W()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear_any(ops.activation(ops.linear_any(h, self.up_proj.weight), "relu2"), self.down_proj.weight)

    __call__ = forward


class NupovikMoE:
    """Sigmoid-routed experts without gates; the experts' up and down weights are stacked for the grouped
    GEMMs over expert-aligned 128-row tiles; the weights multiply the experts' outputs in the combine."""

    def __init__(self, hidden: int, m: dict):
        r = m["router"]
        self.hidden = hidden
        self.num_experts, self.top_k = int(r["experts"]), int(r["top"])
        groups = r.get("groups") or {}
        self.num_groups, self.keep_groups = int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1)))
        self.ff = int(m["expert"]["ff"])
        self.router, self.w_up, self.w_down = _W(), _W(), _W()  # [E, hidden], [E · ff, hidden], [E · hidden, ff]
        self.correction: torch.Tensor = None                    # fp32 [E]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        T, E = h.shape[0], self.num_experts
        z = ops.linear_any(h, self.router.weight, out_f32=True)
        ids, w = ops.moe_route_scores(z, E, self.top_k, score_func="sigmoid", renormalize=True,
                                      correction=self.correction, num_groups=self.num_groups,
                                      keep_groups=self.keep_groups)
        row_token, inv_pos, tile_group = ops.moe_align(ids, E)
        xs = ops.moe_gather_scaled(h, row_token, inv_pos, None)
        act = ops.activation(ops.linear_grouped_any(xs, self.w_up.weight, tile_group, E, self.ff), "relu2")
        y = ops.linear_grouped_any(act, self.w_down.weight, tile_group, E, self.hidden)
        return ops.moe_combine_gated(y, inv_pos, T, self.top_k, topk_w=w)

    __call__ = forward


_MIXERS = {"latent_attention": NupovikLatentAttention, "gla": NupovikGLA, "wkv": NupovikWKV}


class NupovikDecoderLayer:
    """One layer RUN: its own cache / state (layer_id), tensors of its own or of the first run of the layer."""

    def __init__(self, config, layer_id: int):
        spec = config.layer_specs[layer_id]
        H = config.hidden_size
        self.layer_id = layer_id
        self.kind = spec["type"]
        self.name_index = int(spec.get("layer", layer_id))  # index in the checkpoint's tensor names
        self.weights_of = spec.get("weights_of")
        self.opens_pass = bool(spec.get("opens_pass"))
        self.norm1, self.norm2 = _W(), _W()
        self.mixer = _MIXERS[self.kind](H, spec["mixer"], layer_id, config.rms_norm_eps)
        mlp = spec.get("mlp")
        self.mlp = None if mlp is None else NupovikDenseMLP(H, mlp) if mlp["kind"] == "dense" else NupovikMoE(H, mlp)

    def share(self, other: "NupovikDecoderLayer"):
        self.norm1, self.norm2 = other.norm1, other.norm2
        self.mixer.share(other.mixer)
        self.mlp = other.mlp


class NupovikForCausalLM:
    def __init__(self, config, dtype=torch.bfloat16, device="cuda"):
        if config.layer_specs is None:
            raise ValueError("NupovikForCausalLM needs ModelConfig.layer_specs")
        self.config, self.dtype, self.device = config, dtype, device
        self.eps = config.rms_norm_eps
        self.logit_scale = float(getattr(config, "logit_scale", 1.0))
        self.embed_tokens, self.final_norm, self.lm_head, self.pass_in = _W(), _W(), _W(), _W()
        self.layers = [NupovikDecoderLayer(config, i) for i in range(config.num_hidden_layers)]
        for layer in self.layers:
            if layer.weights_of is not None:
                layer.share(self.layers[layer.weights_of])
        self.has_passes = any(layer.opens_pass for layer in self.layers)
        self.freq_hi, self.freq_lo = _sinusoid_frequencies(config.hidden_size, device)
        self.logits_processor = LogitsProcessor(config)

    def cache_shapes(self):
        """(kv shapes, matrix-state shapes, vector-state sizes) per layer run — what ModelRunner sizes the
        pools with.  A latent-attention run owns one row of kv_rank per token (values are read from the same
        row: v_dim 0); a recurrent run owns (heads, k_dim, v_dim) per request, wkv also a row of the width."""
        kv, st, sh = [], [], []
        for layer in self.layers:
            m = layer.mixer
            if layer.kind == "latent_attention":
                kv.append((1, m.rank, 0)); st.append(None); sh.append(None)
            else:
                kv.append(None); st.append((m.num_heads, m.head_dim, m.v_head_dim))
                sh.append(self.config.hidden_size if layer.kind == "wkv" else None)
        return kv, st, sh

    @torch.no_grad()
    def forward(self, input_ids, positions, forward_batch: ForwardBatch, input_embeds=None) -> LogitsProcessorOutput:
        x = ops.embed_sincos(self.embed_tokens.weight, input_ids, positions, self.freq_hi, self.freq_lo)
        x0 = x.clone() if self.has_passes else None  # x is updated in place from here on
        mix = ff = None
        hook = getattr(self, "_layer_hook", None)
        for layer in self.layers:
            if layer.opens_pass:
                if mix is not None:
                    ops.residual_rmsnorm(x, None, self.eps, a=mix, b=ff)  # close the previous layer
                    mix = ff = None
                x = ops.linear_any(ops.cast_concat(x, x0, self.dtype), self.pass_in.weight, out_f32=True)
            # x += (mix + ff) of the previous layer, then this layer's two norms — one kernel
            h1, h2 = ops.residual_rmsnorm2(x, layer.norm1.weight, layer.norm2.weight if layer.mlp is not None else None,
                                           self.eps, a=mix, b=ff)
            mix = layer.mixer(h1, forward_batch)
            ff = layer.mlp(h2) if layer.mlp is not None else None
            if hook is not None:  # debugging / tests: the residual stream after this layer run
                hook(layer.layer_id, x.clone() + (mix.float() + (ff.float() if ff is not None else 0)))
        rows = self.logits_processor.logit_rows(forward_batch)
        if rows is not None and rows.numel() == 0:  # a portion whose logits nobody asked for
            return LogitsProcessorOutput(next_token_logits=torch.empty(
                (0, self.config.vocab_size), device=x.device, dtype=torch.float32))
        if rows is None:
            hs = ops.residual_rmsnorm(x, self.final_norm.weight, self.eps, a=mix, b=ff)
        else:
            ops.residual_rmsnorm(x, None, self.eps, a=mix, b=ff)
            hs = ops.residual_rmsnorm(ops.embed_f32(x, rows), self.final_norm.weight, self.eps)  # fp32 row gather
        logits = ops.linear_any(hs, self.lm_head.weight, out_f32=True)
        if self.logit_scale != 1.0:
            ops.scale_f32_(logits, self.logit_scale)
        return LogitsProcessorOutput(next_token_logits=logits)

    __call__ = forward

    # ------------------------------------------------------------------------------------------
    # parameters.  Checkpoint names: embed, head, final.norm, loop.in, l<i>.norm1, l<i>.norm2,
    # l<i>.mix.* per mixer, l<i>.mlp.{up,down} (dense), l<i>.mlp.{router, correction, e<j>.{up,down}}
    # ------------------------------------------------------------------------------------------
    def full_shapes(self, low_rank: int = 16) -> Dict[str, Tuple[int, ...]]:
        """Name → shape of every tensor.  The low-rank sizes of the decay projections are not in the config
        (the checkpoint's shapes give them); `low_rank` is what dummy weights use."""
        cfg = self.config
        H = cfg.hidden_size
        shapes: Dict[str, Tuple[int, ...]] = {"embed": (cfg.vocab_size, H)}
        if self.has_passes:
            shapes["loop.in"] = (H, 2 * H)
        for spec in cfg.layer_specs:
            if spec.get("weights_of") is not None:
                continue
            p, m = f"l{spec['layer']}.", spec["mixer"]
            shapes[p + "norm1"] = (H,)
            nh, dk = int(m["heads"]), int(m["dim"])
            if spec["type"] == "latent_attention":
                dv, r = int(m["vdim"]), int(m["kv_rank"])
                shapes.update({p + "mix.q": (nh * dk, H), p + "mix.dkv": (r, H), p + "mix.dkv.norm": (r,),
                               p + "mix.uk": (nh * dk, r), p + "mix.uv": (nh * dv, r), p + "mix.g": (nh, H),
                               p + "mix.o": (H, nh * dv)})
            elif spec["type"] == "gla":
                dv = int(m.get("vdim", dk))
                shapes.update({p + "mix.q": (nh * dk, H), p + "mix.k": (nh * dk, H), p + "mix.v": (nh * dv, H),
                               p + "mix.g": (nh * dv, H), p + "mix.o": (H, nh * dv), p + "mix.norm": (dv,),
                               p + "mix.a1": (low_rank, H), p + "mix.a2": (nh * dk, low_rank), p + "mix.a2.b": (nh * dk,)})
            else:
                for s in "rkvgw":
                    shapes[p + "mix.mu." + s] = (H,)
                shapes.update({p + "mix.r": (nh * dk, H), p + "mix.k": (nh * dk, H), p + "mix.v": (nh * dk, H),
                               p + "mix.g": (nh * dk, H), p + "mix.w1": (low_rank, H), p + "mix.w2": (nh * dk, low_rank),
                               p + "mix.w0": (nh * dk,), p + "mix.u": (nh, dk), p + "mix.norm": (nh * dk,),
                               p + "mix.o": (H, nh * dk)})
            mlp = spec.get("mlp")
            if mlp is None:
                continue
            shapes[p + "norm2"] = (H,)
            if mlp["kind"] == "dense":
                ff = int(mlp["ff"])
                shapes.update({p + "mlp.up": (ff, H), p + "mlp.down": (H, ff)})
            else:
                ff, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
                for e in range(E):
                    shapes.update({f"{p}mlp.e{e}.up": (ff, H), f"{p}mlp.e{e}.down": (H, ff)})
                shapes.update({p + "mlp.router": (E, H), p + "mlp.correction": (E,)})
        shapes["final.norm"] = (H,)
        shapes["head"] = (cfg.vocab_size, H)
        return shapes

    _FREE_DIMS = {"mix.a1": 0, "mix.a2": 1, "mix.w1": 0, "mix.w2": 1}  # the low-rank dimension of these tensors

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        w = {k: v for k, v in weights}
        shapes = self.full_shapes()
        missing = set(shapes) - set(w)
        if missing:
            raise KeyError(f"missing parameters: {sorted(missing)[:4]} …")
        for name, shape in shapes.items():
            got, want = list(w[name].shape), list(shape)
            free = self._FREE_DIMS.get(name.split(".", 1)[-1])
            if free is not None and len(got) == len(want):
                want[free] = got[free]
            if got != want:
                raise ValueError(f"{name}: shape {tuple(got)} does not match the config's {tuple(shape)}")

        def put(t):
            return t.to(self.dtype).to(self.device).contiguous()

        def put32(t):
            return t.to(torch.float32).to(self.device).contiguous()

        def rows8(parts):
            t = torch.cat(parts, 0)
            pad = _pad8(t.shape[0]) - t.shape[0]
            return put(torch.cat([t, t.new_zeros((pad, t.shape[1]))], 0) if pad else t)

        self.embed_tokens.weight = put(w["embed"])
        self.final_norm.weight = put(w["final.norm"])
        self.lm_head.weight = put(w["head"])
        if self.has_passes:
            self.pass_in.weight = put(w["loop.in"])
        for layer in self.layers:
            if layer.weights_of is not None:
                continue
            p = f"l{layer.name_index}."
            layer.norm1.weight = put(w[p + "norm1"])
            if layer.mlp is not None:
                layer.norm2.weight = put(w[p + "norm2"])
            mx = layer.mixer
            if layer.kind == "latent_attention":
                mx.qcg_proj.weight = rows8([w[p + "mix.q"], w[p + "mix.dkv"], w[p + "mix.g"]])
                mx.c_norm.weight = put(w[p + "mix.dkv.norm"])
                # absorbed form: per head the transposed key lift [rank, dim], stacked; the value lift as stored
                uk = w[p + "mix.uk"].view(mx.heads, mx.dim, mx.rank)
                mx.uk_t.weight = put(uk.transpose(1, 2).reshape(mx.heads * mx.rank, mx.dim))
                mx.uv.weight = put(w[p + "mix.uv"])
            elif layer.kind == "gla":
                if w[p + "mix.a2"].shape[1] != w[p + "mix.a1"].shape[0]:
                    raise ValueError(f"{p}mix.a1 / a2: the low-rank sizes differ")
                mx.in_proj.weight = rows8([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"], w[p + "mix.a1"]])
                mx.a2.weight = put(w[p + "mix.a2"])
                mx.a2_bias.weight = put32(w[p + "mix.a2.b"])
                mx.norm.weight = put(w[p + "mix.norm"])
            else:
                if w[p + "mix.w2"].shape[1] != w[p + "mix.w1"].shape[0]:
                    raise ValueError(f"{p}mix.w1 / w2: the low-rank sizes differ")
                mx.mu.weight = put(torch.stack([w[p + "mix.mu." + s] for s in "rkvgw"], 0))
                for n in ("r", "k", "v", "g", "w1", "w2", "norm"):
                    getattr(mx, n).weight = put(w[p + "mix." + n])
                mx.w0.weight = put32(w[p + "mix.w0"])
                mx.u.weight = put32(w[p + "mix.u"].reshape(-1))
            mx.o_proj.weight = put(w[p + "mix.o"])
            mlp = layer.mlp
            if isinstance(mlp, NupovikDenseMLP):
                mlp.up_proj.weight = put(w[p + "mlp.up"])
                mlp.down_proj.weight = put(w[p + "mlp.down"])
            elif isinstance(mlp, NupovikMoE):
                E = mlp.num_experts
                mlp.w_up.weight = put(torch.cat([w[f"{p}mlp.e{e}.up"] for e in range(E)], 0))
                mlp.w_down.weight = put(torch.cat([w[f"{p}mlp.e{e}.down"] for e in range(E)], 0))
                mlp.router.weight = put(w[p + "mlp.router"])
                mlp.correction = put32(w[p + "mlp.correction"])

    def dummy_full_weights(self, seed: int = 1234) -> Dict[str, torch.Tensor]:
        """Random weights by checkpoint name: projections N(0, 1/fan_in), norm weights around 1, the other
        vectors N(0, 0.1²) (shift mixes in [0, 1]), rounded to bfloat16 like a stored checkpoint; one
        generator per parameter."""
        out = {}
        for idx, (name, shape) in enumerate(self.full_shapes().items()):
            g = torch.Generator().manual_seed(seed + idx)
            if ".mu." in name:
                t = torch.rand(shape, generator=g)
            elif len(shape) == 1 and "norm" in name:
                t = 1.0 + torch.randn(shape, generator=g) * 0.1
            elif len(shape) == 1 or name.endswith("mix.u"):
                t = torch.randn(shape, generator=g) * 0.1
            elif name == "embed":
                t = torch.randn(shape, generator=g)
            else:
                t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            out[name] = t.to(torch.bfloat16)
        return out

    def init_dummy_weights(self, seed: int = 1234):
        w = self.dummy_full_weights(seed)
        self.load_weights(w.items())
        return w

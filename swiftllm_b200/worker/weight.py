"""Weights of the data plane.  Attribute names, HF tensor keys and the `up_gate_proj = cat(up, gate)` fusion are
the reference's (swiftllm/worker/weight.py:56-177, :133); loaders cover the same sources (safetensors single /
sharded, pytorch_model.bin, dummy uniform(-1e-3, 1e-3)) plus seeded synthetic weights, and every projection is
sliced for tensor parallelism at load time:

    rank r of N holds   q_proj rows of q heads [r*nq/N, (r+1)*nq/N)        (column-parallel)
                        k_proj / v_proj rows of kv heads [r*nkv/N, ...)     (column-parallel)
                        up / gate rows [r*F/N, (r+1)*F/N), re-fused as [up_r ; gate_r]
                        o_proj / down_proj input columns of the same slices (row-parallel, all-reduced)
    norms and the embedding are replicated; lm_head is replicated, or (shard_lm_head) split by vocabulary rows.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Optional

import torch

from swiftllm_b200.model_config import LlamaModelConfig

# (attribute, HF key template, shape fn, TP split axis: 0 rows, 1 cols, None replicated)
_LAYER_ITEMS = [
    ("attn_norm", "model.layers.{i}.input_layernorm.weight", lambda c: (c.hidden_size,), None),
    ("q_proj", "model.layers.{i}.self_attn.q_proj.weight", lambda c: (c.hidden_size, c.hidden_size), 0),
    ("k_proj", "model.layers.{i}.self_attn.k_proj.weight", lambda c: (c.num_kv_heads * c.head_dim, c.hidden_size), 0),
    ("v_proj", "model.layers.{i}.self_attn.v_proj.weight", lambda c: (c.num_kv_heads * c.head_dim, c.hidden_size), 0),
    ("o_proj", "model.layers.{i}.self_attn.o_proj.weight", lambda c: (c.hidden_size, c.hidden_size), 1),
    ("ffn_norm", "model.layers.{i}.post_attention_layernorm.weight", lambda c: (c.hidden_size,), None),
    ("up_proj", "model.layers.{i}.mlp.up_proj.weight", lambda c: (c.ffn_inter_dim, c.hidden_size), 0),
    ("gate_proj", "model.layers.{i}.mlp.gate_proj.weight", lambda c: (c.ffn_inter_dim, c.hidden_size), 0),
    ("down_proj", "model.layers.{i}.mlp.down_proj.weight", lambda c: (c.hidden_size, c.ffn_inter_dim), 1),
]


def tp_slice(t: torch.Tensor, axis: Optional[int], tp_rank: int, tp_size: int) -> torch.Tensor:
    if axis is None or tp_size == 1:
        return t
    n = t.shape[axis]
    assert n % tp_size == 0, f"dimension {n} not divisible by tp_size {tp_size}"
    step = n // tp_size
    return t.narrow(axis, tp_rank * step, step)


class LlamaTransformerLayerWeight:
    def __init__(self, layer_id: int, model_config: LlamaModelConfig, dtype: torch.dtype):
        self.layer_id = layer_id
        self.model_config = model_config
        self.dtype = dtype

    def load_weights(self, getter: Callable, tp_rank: int, tp_size: int, device):
        for attr, key, shape_fn, axis in _LAYER_ITEMS:
            key = key.format(i=self.layer_id)
            shape = shape_fn(self.model_config)
            w = getter(key, shape, self.dtype)
            assert isinstance(w, torch.Tensor), f"Weight {key} is not a tensor"
            assert tuple(w.shape) == tuple(shape), f"Shape of weight {key} does not match"
            w = tp_slice(w, axis, tp_rank, tp_size).to(device=device, dtype=self.dtype).contiguous()
            setattr(self, attr, w)
        # up first, gate second (weight.py:133; silu_and_mul reads gate from the second half)
        self.up_gate_proj = torch.cat((self.up_proj, self.gate_proj), dim=0).contiguous()
        del self.up_proj, self.gate_proj
        # q | k | v fused into one GEMM operand (the fusion the reference left commented out, weight.py:131-132);
        # q_proj / k_proj / v_proj stay available as row views of it (no extra memory)
        nq_rows, nkv_rows = self.q_proj.shape[0], self.k_proj.shape[0]
        self.qkv_proj = torch.cat((self.q_proj, self.k_proj, self.v_proj), dim=0).contiguous()
        self.q_proj = self.qkv_proj[:nq_rows]
        self.k_proj = self.qkv_proj[nq_rows:nq_rows + nkv_rows]
        self.v_proj = self.qkv_proj[nq_rows + nkv_rows:]


class LlamaWeight:
    def __init__(self, model_config: LlamaModelConfig, dtype: torch.dtype, model_version: str = "llama"):
        self.model_config = model_config
        self.dtype = dtype
        self.model_version = model_version
        self.layers = [LlamaTransformerLayerWeight(i, model_config, dtype) for i in range(model_config.num_layers)]

    def load_weights(self, getter: Callable, tp_rank: int = 0, tp_size: int = 1, device="cuda", shard_lm_head: bool = False):
        c = self.model_config
        vs = (c.vocab_size, c.hidden_size)
        self.wte = getter("model.embed_tokens.weight", vs, self.dtype).to(device=device, dtype=self.dtype)
        self.lm_head_sharded = bool(shard_lm_head) and tp_size > 1
        if self.lm_head_sharded:
            assert c.vocab_size % tp_size == 0, f"shard_lm_head: vocab_size {c.vocab_size} not divisible by tp_size {tp_size}"
        if self.model_version == "llama3.2":      # tied embeddings (weight.py:157-163); a row slice of wte is a view
            self.lm_head = tp_slice(self.wte, 0, tp_rank, tp_size) if self.lm_head_sharded else self.wte
        else:
            lm_head = getter("lm_head.weight", vs, self.dtype)
            if self.lm_head_sharded:
                lm_head = tp_slice(lm_head, 0, tp_rank, tp_size)
            self.lm_head = lm_head.to(device=device, dtype=self.dtype).contiguous()
        self.final_norm = getter("model.norm.weight", (c.hidden_size,), self.dtype).to(device=device, dtype=self.dtype)
        for layer in self.layers:
            layer.load_weights(getter, tp_rank, tp_size, device)


class BupozenLayerWeight:
    """One parallel block.  Checkpoint names: `l<i>.norm1`, `l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}` (no dkv*
    in a layer that reads another layer's cache), `l<i>.mlp.{up, down}` or `l<i>.mlp.{router, e<k>.up, e<k>.down}`.
    Fusions made at load time: every projection that reads the block's normed input and feeds fp32 post-processing is one GEMM
    operand (`in_proj` = [dq ; g ; dkv]); the experts are concatenated (`up` rows / `down` columns expert by expert)."""

    def __init__(self, layer_id: int, model_config, dtype: torch.dtype):
        self.layer_id, self.model_config, self.dtype = layer_id, model_config, dtype

    def load_weights(self, getter: Callable, device):
        c, i = self.model_config, self.layer_id
        m, f, W = c.mixers[i], c.ffs[i], c.hidden_size

        def get(name, shape, dtype=None):
            w = getter(f"l{i}.{name}", shape, dtype or self.dtype)
            assert isinstance(w, torch.Tensor) and tuple(w.shape) == tuple(shape), f"l{i}.{name}: expected shape {tuple(shape)}"
            return w.to(device=device, dtype=dtype or self.dtype).contiguous()

        self.norm = get("norm1", (W,))
        parts = [get("mix.dq", (m.q_rank, W)), get("mix.g", (m.heads, W))]
        if m.kv_from is None:
            parts.append(get("mix.dkv", (m.cache_width, W)))
            self.dkv_norm = get("mix.dkv.norm", (m.kv_rank,))
        self.in_proj = torch.cat(parts, dim=0).contiguous()
        self.dq_norm = get("mix.dq.norm", (m.q_rank,))
        self.uq = get("mix.uq", (m.heads * (m.dim + m.rot_dim), m.q_rank))
        self.uk = get("mix.uk", (m.heads * m.dim, m.kv_rank)).view(m.heads, m.dim, m.kv_rank)       # q_lat[h] = q_nope[h] @ uk[h]
        self.uv = get("mix.uv", (m.heads * m.vdim, m.kv_rank)).view(m.heads, m.vdim, m.kv_rank)     # v[h] = out_lat[h] @ uv[h]^T
        self.o = get("mix.o", (W, m.heads * m.vdim))
        if f is None:
            return
        if f.kind == "dense":
            self.up, self.down = get("mlp.up", (f.ff, W)), get("mlp.down", (W, f.ff))
        else:
            self.router = get("mlp.router", (f.experts, W), torch.float32)                            # the router runs in fp32
            self.up = torch.cat([get(f"mlp.e{e}.up", (f.ff, W)) for e in range(f.experts)], dim=0).contiguous()
            self.down = torch.cat([get(f"mlp.e{e}.down", (W, f.ff)) for e in range(f.experts)], dim=1).contiguous()


class BupozenWeight:
    def __init__(self, model_config, dtype: torch.dtype):
        self.model_config, self.dtype = model_config, dtype
        self.layers = [BupozenLayerWeight(i, model_config, dtype) for i in range(model_config.num_layers)]

    def load_weights(self, getter: Callable, device="cuda"):
        c = self.model_config
        vs = (c.vocab_size, c.hidden_size)
        self.wte = getter("embed", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.final_norm = getter("final.norm", (c.hidden_size,), self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.lm_head = getter("head", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.lm_head_sharded = False
        for layer in self.layers:
            layer.load_weights(getter, device)


def load_bupozen_weights(model_config, dtype: torch.dtype, model_path: Optional[str], use_dummy: bool = False,
                         getter: Optional[Callable] = None, device="cuda") -> BupozenWeight:
    if getter is None:
        getter = dummy_getter(device) if use_dummy else checkpoint_getter(model_path, device)
    weight = BupozenWeight(model_config, dtype)
    weight.load_weights(getter, device)
    return weight


class RivudraLayerWeight:
    """One parallel block.  Checkpoint names: `l<i>.norm1`, `l<i>.mix.{q, k, v, g, o}`, `l<i>.mlp.{router, e<k>.{gate, up, down},
    shared.{gate, up, down}}`.  Fusions made at load time: `in_proj` = [q ; k ; v ; g] (one GEMM on the block's normed input);
    `up` = per expert [gate ; up], then the shared expert's [gate ; up]; `down` = the experts' and the shared expert's down
    projections side by side.  Norm weights are stored around zero and applied as 1 + w: kept as fp32 (1 + w)."""

    def __init__(self, layer_id: int, model_config, dtype: torch.dtype):
        self.layer_id, self.model_config, self.dtype = layer_id, model_config, dtype

    def load_weights(self, getter: Callable, device):
        c, i = self.model_config, self.layer_id
        m, f, W = c.mixers[i], c.ffs[i], c.hidden_size

        def get(name, shape, dtype=None):
            w = getter(f"l{i}.{name}", shape, dtype or self.dtype)
            assert isinstance(w, torch.Tensor) and tuple(w.shape) == tuple(shape), f"l{i}.{name}: expected shape {tuple(shape)}"
            return w.to(device=device, dtype=dtype or self.dtype).contiguous()

        self.norm = unit_offset_norm(get("norm1", (W,), torch.float32))
        self.in_proj = torch.cat([get("mix.q", (m.heads * m.dim, W)), get("mix.k", (m.kv_heads * m.dim, W)),
                                  get("mix.v", (m.kv_heads * m.vdim, W)), get("mix.g", (m.heads * m.vdim, W))], dim=0).contiguous()
        self.o = get("mix.o", (W, m.heads * m.vdim))
        if f is None:
            return
        self.router = get("mlp.router", (f.experts, W), torch.float32)                                # the router runs in fp32
        names = [(f"mlp.e{e}", f.ff) for e in range(f.experts)] + ([("mlp.shared", f.shared_ff)] if f.shared_ff else [])
        self.up = torch.cat([get(f"{n}.{part}", (ff, W)) for n, ff in names for part in ("gate", "up")], dim=0).contiguous()
        self.down = torch.cat([get(f"{n}.down", (W, ff)) for n, ff in names], dim=1).contiguous()


def unit_offset_norm(w: torch.Tensor) -> torch.Tensor:
    """A norm weight stored around zero -> the fp32 factor 1 + w it is applied as."""
    return (w.float() + 1.0).contiguous()


class RivudraWeight:
    def __init__(self, model_config, dtype: torch.dtype):
        self.model_config, self.dtype = model_config, dtype
        self.layers = [RivudraLayerWeight(i, model_config, dtype) for i in range(model_config.num_layers)]

    def load_weights(self, getter: Callable, device="cuda"):
        c = self.model_config
        vs = (c.vocab_size, c.hidden_size)
        self.wte = getter("embed", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.final_norm = unit_offset_norm(getter("final.norm", (c.hidden_size,), torch.float32).to(device=device))
        self.lm_head = getter("head", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.lm_head_sharded = False
        for layer in self.layers:
            layer.load_weights(getter, device)


def load_rivudra_weights(model_config, dtype: torch.dtype, model_path: Optional[str], use_dummy: bool = False,
                         getter: Optional[Callable] = None, device="cuda") -> RivudraWeight:
    if getter is None:
        getter = dummy_getter(device) if use_dummy else checkpoint_getter(model_path, device)
    weight = RivudraWeight(model_config, dtype)
    weight.load_weights(getter, device)
    return weight


class BuzaraxLayerWeight:
    """One sequential block.  Checkpoint names: `l<i>.norm1`, `l<i>.norm2` (scalars), `l<i>.dwa` ([i + 2]), and
    mixer "parallel": `l<i>.mix.left.{q, k, v, o}`, `l<i>.mix.right.{q, k, v, g, o, norm}`;
    mixer "rglru": `l<i>.mix.{y, y.b, x, x.b, conv, conv.b, ra, ra.b, ri, ri.b, lam, o}`;
    feed-forward: `l<i>.mlp.{gate, up, down}` or `l<i>.mlp.{router, correction, e<k>.{gate, up, down}}`.
    Fusions made at load time: every projection that reads the block's input is one GEMM operand (`in_proj`: [left q ; k ; v ;
    right q ; k ; v ; g], or [y ; x] with `in_bias`); the two output projections of a parallel mixer are one operand side by side
    (`o`; the mixers' weights in the sum are applied by the kernels that write its input); the two block-diagonal gate
    projections are one batched operand (`gate_w` [blocks, in, 2 * out], `gate_b`); `rate` = -8 softplus(lam) in fp32; the
    experts' [gate ; up] rows and down columns are concatenated expert by expert.  Scalars, `dwa`, the group norm, the router
    and its correction are fp32."""

    def __init__(self, layer_id: int, model_config, dtype: torch.dtype):
        self.layer_id, self.model_config, self.dtype = layer_id, model_config, dtype

    def load_weights(self, getter: Callable, device):
        from swiftllm_b200.model_config import GatedRecurrenceSpec
        c, i = self.model_config, self.layer_id
        m, f, W = c.mixers[i], c.ffs[i], c.hidden_size

        def get(name, shape, dtype=None):
            w = getter(f"l{i}.{name}", shape, dtype or self.dtype)
            assert isinstance(w, torch.Tensor) and tuple(w.shape) == tuple(shape), f"l{i}.{name}: expected shape {tuple(shape)}"
            return w.to(device=device, dtype=dtype or self.dtype).contiguous()

        self.norm1 = get("norm1", (), torch.float32).reshape(1)
        self.dwa = get("dwa", (i + 2,), torch.float32)
        if isinstance(m, GatedRecurrenceSpec):
            C, B, K = m.width, m.blocks, m.conv
            cb = C // B
            self.in_proj = torch.cat([get("mix.y", (C, W)), get("mix.x", (C, W))], dim=0).contiguous()
            self.in_bias = torch.cat([get("mix.y.b", (C,)), get("mix.x.b", (C,))], dim=0).contiguous()
            self.conv, self.conv_b = get("mix.conv", (C, K)), get("mix.conv.b", (C,))
            gw = torch.cat([get("mix.ra", (B, cb, cb)), get("mix.ri", (B, cb, cb))], dim=1)          # [B, 2 cb (out), cb (in)]
            self.gate_w = gw.transpose(1, 2).contiguous()                                               # [B, in, 2 out]
            self.gate_b = torch.cat([get("mix.ra.b", (B, cb)), get("mix.ri.b", (B, cb))], dim=1).reshape(B, 1, 2 * cb).contiguous()
            self.rate = (-8.0 * torch.nn.functional.softplus(get("mix.lam", (C,), torch.float32))).contiguous()
            self.o = get("mix.o", (W, C))
        else:
            a, b = m.left, m.right
            self.in_proj = torch.cat([
                get("mix.left.q", (a.heads * a.dim, W)), get("mix.left.k", (a.kv_heads * a.dim, W)),
                get("mix.left.v", (a.kv_heads * a.vdim, W)), get("mix.right.q", (b.heads * b.dim, W)),
                get("mix.right.k", (b.heads * b.dim, W)), get("mix.right.v", (b.heads * b.vdim, W)),
                get("mix.right.g", (b.heads * b.vdim, W))], dim=0).contiguous()
            self.o = torch.cat([get("mix.left.o", (W, a.heads * a.vdim)), get("mix.right.o", (W, b.heads * b.vdim))], dim=1).contiguous()
            self.lin_norm = get("mix.right.norm", (b.heads * b.vdim,), torch.float32)
            self.decay = torch.tensor(b.decay, dtype=torch.float32).to(device)
        if f is None:
            return
        self.norm2 = get("norm2", (), torch.float32).reshape(1)
        if f.kind == "dense":
            self.up = torch.cat([get("mlp.gate", (f.ff, W)), get("mlp.up", (f.ff, W))], dim=0).contiguous()
            self.down = get("mlp.down", (W, f.ff))
        else:
            self.router = get("mlp.router", (f.experts, W), torch.float32)                            # the router runs in fp32
            self.correction = get("mlp.correction", (f.experts,), torch.float32)
            self.up = torch.cat([get(f"mlp.e{e}.{part}", (f.ff, W)) for e in range(f.experts) for part in ("gate", "up")],
                                dim=0).contiguous()
            self.down = torch.cat([get(f"mlp.e{e}.down", (W, f.ff)) for e in range(f.experts)], dim=1).contiguous()


class BuzaraxWeight:
    def __init__(self, model_config, dtype: torch.dtype):
        self.model_config, self.dtype = model_config, dtype
        self.layers = [BuzaraxLayerWeight(i, model_config, dtype) for i in range(model_config.num_layers)]

    def load_weights(self, getter: Callable, device="cuda"):
        c = self.model_config
        vs = (c.vocab_size, c.hidden_size)
        self.wte = getter("embed", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.pairs = None
        if c.pair_hash is not None:
            self.pairs = getter("bigram", (c.pair_hash.buckets + 1, c.hidden_size), self.dtype).to(device=device, dtype=self.dtype).contiguous()
        # the final norm has ONE gain: kept as an fp32 vector of equal entries, the form the fused add + norm kernel reads
        g = getter("final.norm", (), torch.float32).to(device=device, dtype=torch.float32)
        self.final_norm = g.reshape(1).expand(c.hidden_size).contiguous()
        self.lm_head = getter("head", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.lm_head_sharded = False
        for layer in self.layers:
            layer.load_weights(getter, device)


def load_buzarax_weights(model_config, dtype: torch.dtype, model_path: Optional[str], use_dummy: bool = False,
                         getter: Optional[Callable] = None, device="cuda") -> BuzaraxWeight:
    if getter is None:
        getter = dummy_getter(device) if use_dummy else checkpoint_getter(model_path, device)
    weight = BuzaraxWeight(model_config, dtype)
    weight.load_weights(getter, device)
    return weight


class NaforaxLayerWeight:
    """One sandwich block.  Checkpoint names: `l<i>.{norm1, norm1b, norm2, norm2b}` ([width]), `l<i>.{canon1, canon2}` ([width,
    taps]), and
    mixer "attention": `l<i>.mix.{q, q.b, k, k.b, v, v.b, q.norm, k.norm, lq1, lk1, lq2, lk2, g, o, o.b}` (q rows head by head as
    [map 0 | map 1], k likewise);  mixer "mingru": `l<i>.mix.{z, z.b, x, x.b, g, o}`;
    mixer "mamba1": `l<i>.mix.{in, conv, conv.b, x, dt, dt.b, A_log, D, o}`;
    feed-forward: `l<i>.mlp.{gate, up, down}` or `l<i>.mlp.{router, e<k>.{gate, up, down}, shared.{gate, up, down, sg}}`.
    Fusions made at load time: every projection that reads the sublayer's input is one GEMM operand with one bias vector
    (`in_proj`, `in_bias`: [q ; k ; v ; g] or [z ; x ; g]); the q rows are reordered to [key/value head][map][head of the group]
    so that the attention kernel sees every map as a query head of its own whose key head is (key/value head, map);
    `lam` = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (fp32, one number); the experts' [gate ; up] rows and down columns are
    concatenated expert by expert with the shared expert last; the router and the shared expert's gate row are one fp32 operand.
    Norm weights, convolution taps, `A` = -exp(A_log), `D`, the step bias and the router are fp32."""

    def __init__(self, layer_id: int, model_config, dtype: torch.dtype):
        self.layer_id, self.model_config, self.dtype = layer_id, model_config, dtype

    def load_weights(self, getter: Callable, device):
        from swiftllm_b200.model_config import MinGruSpec, SelectiveScanSpec
        c, i = self.model_config, self.layer_id
        m, f, W, K = c.mixers[i], c.ffs[i], c.hidden_size, c.canon_taps

        def get(name, shape, dtype=None):
            w = getter(f"l{i}.{name}", shape, dtype or self.dtype)
            assert isinstance(w, torch.Tensor) and tuple(w.shape) == tuple(shape), f"l{i}.{name}: expected shape {tuple(shape)}"
            return w.to(device=device, dtype=dtype or self.dtype).contiguous()

        f32 = torch.float32
        self.norm1, self.norm1b, self.canon1 = get("norm1", (W,), f32), get("norm1b", (W,), f32), get("canon1", (W, K), f32)
        if isinstance(m, MinGruSpec):
            C = m.width
            self.in_proj = torch.cat([get("mix.z", (C, W)), get("mix.x", (C, W)), get("mix.g", (C, W))], dim=0).contiguous()
            self.in_bias = torch.cat([get("mix.z.b", (C,)), get("mix.x.b", (C,)), torch.zeros((C,), dtype=self.dtype, device=device)])
            self.o = get("mix.o", (W, C))
        elif isinstance(m, SelectiveScanSpec):
            C, N, R = m.inner, m.state, m.dt_rank
            self.in_proj = get("mix.in", (2 * C, W))
            self.conv, self.conv_b = get("mix.conv", (C, m.conv), f32), get("mix.conv.b", (C,), f32)
            self.x_proj = get("mix.x", (R + 2 * N, C))
            self.dt_proj, self.dt_bias = get("mix.dt", (C, R)), get("mix.dt.b", (C,), f32)
            self.A = (-torch.exp(get("mix.A_log", (C, N), f32))).contiguous()
            self.D = get("mix.D", (C,), f32)
            self.o = get("mix.o", (W, C))
        else:
            H, G, dk, dv = m.heads, m.kv_heads, m.dim, m.vdim
            hq = H // G
            # rows [h][map][dk] with h = g hq + hh  ->  [g][map][hh][dk]
            order = torch.arange(H * m.maps * dk, device=device).view(G, hq, m.maps, dk).permute(0, 2, 1, 3).reshape(-1)
            q, qb = get("mix.q", (H * m.maps * dk, W)), get("mix.q.b", (H * m.maps * dk,))
            self.in_proj = torch.cat([q[order], get("mix.k", (G * m.maps * dk, W)), get("mix.v", (G * dv, W)),
                                      get("mix.g", (H * dv, W))], dim=0).contiguous()
            self.in_bias = torch.cat([qb[order], get("mix.k.b", (G * m.maps * dk,)), get("mix.v.b", (G * dv,)),
                                      torch.zeros((H * dv,), dtype=self.dtype, device=device)]).contiguous()
            self.q_norm, self.k_norm = get("mix.q.norm", (dk,), f32), get("mix.k.norm", (dk,), f32)
            lq1, lk1, lq2, lk2 = (get(f"mix.{n}", (dk,), f32) for n in ("lq1", "lk1", "lq2", "lk2"))
            self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + m.diff)
            self.o, self.o_bias = get("mix.o", (W, H * dv)), get("mix.o.b", (W,))
        if f is None:
            return
        self.norm2, self.norm2b, self.canon2 = get("norm2", (W,), f32), get("norm2b", (W,), f32), get("canon2", (W, K), f32)
        if f.kind == "dense":
            self.up = torch.cat([get("mlp.gate", (f.ff, W)), get("mlp.up", (f.ff, W))], dim=0).contiguous()
            self.down = get("mlp.down", (W, f.ff))
        else:
            rows = [get("mlp.router", (f.experts, W), f32)] + ([get("mlp.shared.sg", (1, W), f32)] if f.shared_gated else [])
            self.router = torch.cat(rows, dim=0).contiguous()                                        # the router runs in fp32
            names = [(f"mlp.e{e}", f.ff) for e in range(f.experts)] + ([("mlp.shared", f.shared_ff)] if f.shared_ff else [])
            self.up = torch.cat([get(f"{n}.{part}", (ff, W)) for n, ff in names for part in ("gate", "up")], dim=0).contiguous()
            self.down = torch.cat([get(f"{n}.down", (W, ff)) for n, ff in names], dim=1).contiguous()


class NaforaxWeight:
    def __init__(self, model_config, dtype: torch.dtype):
        self.model_config, self.dtype = model_config, dtype
        self.layers = [NaforaxLayerWeight(i, model_config, dtype) for i in range(model_config.num_layers)]

    def load_weights(self, getter: Callable, device="cuda"):
        c = self.model_config
        vs = (c.vocab_size, c.hidden_size)
        self.wte = getter("embed", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.loop_step = None
        if c.loop is not None:
            self.loop_step = getter("loop.step", (c.loop[2], c.hidden_size), torch.float32).to(device=device, dtype=torch.float32).contiguous()
        self.final_norm = getter("final.norm", (c.hidden_size,), torch.float32).to(device=device, dtype=torch.float32).contiguous()
        self.lm_head = getter("head", vs, self.dtype).to(device=device, dtype=self.dtype).contiguous()
        self.lm_head_sharded = False
        for layer in self.layers:
            layer.load_weights(getter, device)


def load_naforax_weights(model_config, dtype: torch.dtype, model_path: Optional[str], use_dummy: bool = False,
                         getter: Optional[Callable] = None, device="cuda") -> NaforaxWeight:
    if getter is None:
        getter = dummy_getter(device) if use_dummy else checkpoint_getter(model_path, device)
    weight = NaforaxWeight(model_config, dtype)
    weight.load_weights(getter, device)
    return weight


# ---------------------------------------------------------------- getters
def dummy_getter(device="cuda"):
    """weight.py:215-218: uniform(-1e-3, 1e-3), unseeded ("mainly for profiling")."""
    def get(key, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=device).uniform_(-0.001, 0.001)
    return get


def synthetic_getter(seed: int = 0, std: float = 0.02, device="cuda", norm_offset: float = 1.0):
    """Seeded synthetic weights of realistic scale: N(0, std) projections, norm_offset + N(0, std) norms
    (0 for designs that store norm weights around zero).
    Deterministic per tensor key, so every TP rank generates the same full tensor before slicing."""
    import zlib

    def get(key, shape, dtype):
        g = torch.Generator(device=device)
        g.manual_seed((seed * 1000003 + zlib.crc32(key.encode())) & 0x7FFFFFFF)
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
        if key.endswith(("norm.weight", "layernorm.weight", ".norm", ".norm1")):
            t += norm_offset
        return t.to(dtype)
    return get


def dict_getter(tensors: dict):
    def get(key, shape, dtype):
        return tensors[key]
    return get


def checkpoint_getter(model_path: str, device="cuda"):
    """safetensors (single file or model.safetensors.index.json) or pytorch_model.bin(.index.json), as in
    weight.py:220-268."""
    st_files = [n for n in os.listdir(model_path) if n.endswith(".safetensors")]
    if st_files:
        import safetensors
        index_path = os.path.join(model_path, "model.safetensors.index.json")
        if os.path.exists(index_path):
            with open(index_path, "r", encoding="utf-8") as f:
                index = json.load(f)["weight_map"]
        else:
            assert len(st_files) == 1, "model.safetensors.index.json not found, but there are multiple .safetensors files"
            index = None

        def get(key, shape, dtype):
            fname = index[key] if index is not None else st_files[0]
            dev = str(device)
            with safetensors.safe_open(os.path.join(model_path, fname), framework="pt",
                                       device="cpu" if dev.startswith("cpu") else dev) as f:
                return f.get_tensor(key)
        return get

    index_path = os.path.join(model_path, "pytorch_model.bin.index.json")
    index = None
    if os.path.exists(index_path):
        with open(index_path, "r", encoding="utf-8") as f:
            index = json.load(f)["weight_map"]
    opened = {}

    def get(key, shape, dtype):
        fname = index[key] if index is not None else "pytorch_model.bin"
        path = os.path.join(model_path, fname)
        if path not in opened:
            opened[path] = torch.load(path, map_location="cpu", mmap=True)
        return opened[path][key]
    return get


def detect_model_version(model_path: Optional[str], model_config: LlamaModelConfig) -> str:
    # weight.py:205-211: "llama3.2" (tied lm_head) iff rope_scaling is a dict
    return "llama3.2" if isinstance(model_config.rope_scaling, dict) else "llama"


def load_weights(model_config: LlamaModelConfig, dtype: torch.dtype, model_path: Optional[str], use_dummy: bool = False,
                 model_version: str = "auto", getter: Optional[Callable] = None, tp_rank: int = 0, tp_size: int = 1,
                 device="cuda", shard_lm_head: bool = False) -> LlamaWeight:
    if model_version == "auto":
        model_version = detect_model_version(model_path, model_config)
    if getter is None:
        getter = dummy_getter(device) if use_dummy else checkpoint_getter(model_path, device)
    weight = LlamaWeight(model_config, dtype, model_version)
    weight.load_weights(getter, tp_rank, tp_size, device, shard_lm_head=shard_lm_head)
    return weight

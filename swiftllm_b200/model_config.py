"""HF `config.json` -> LlamaModelConfig.

The attribute names are the ones the reference's worker reads (`swiftllm/model_config.py:5-46`): num_layers, num_q_heads,
num_kv_heads, hidden_size, head_dim, vocab_size, max_position_embeddings, ffn_inter_dim, rotary_base / rope_theta,
rms_norm_eps, rope_scaling (1.0 when absent or null; a dict for Llama 3.2 style scaling) and get_kvslot_size()."""
import dataclasses
import json
import os
from typing import Optional

import torch

# attribute <- key of the HF config (required)
_REQUIRED = {
    "num_layers": "num_hidden_layers",
    "num_q_heads": "num_attention_heads",
    "hidden_size": "hidden_size",
    "vocab_size": "vocab_size",
    "max_position_embeddings": "max_position_embeddings",
    "ffn_inter_dim": "intermediate_size",
    "rms_norm_eps": "rms_norm_eps",
}


class LlamaModelConfig:
    family = "llama"

    def __init__(self, model_config: dict):
        arch, act = model_config.get("model_type"), model_config.get("hidden_act")
        assert arch == "llama", f"only the llama architecture is served, got model_type={arch!r}"
        assert act == "silu", f"the FFN kernel is SiLU-gated (silu_and_mul), got hidden_act={act!r}"
        missing = [k for k in _REQUIRED.values() if k not in model_config]
        assert not missing, f"config.json lacks {missing}"
        for attr, key in _REQUIRED.items():
            setattr(self, attr, model_config[key])
        self.num_kv_heads = model_config.get("num_key_value_heads") or self.num_q_heads      # MHA checkpoints omit it
        assert self.hidden_size % self.num_q_heads == 0 and self.num_q_heads % self.num_kv_heads == 0
        self.head_dim = self.hidden_size // self.num_q_heads
        theta = model_config.get("rope_theta")
        self.rope_theta = 10000 if theta is None else theta
        self.rotary_base = model_config.get("rotary_base", 10000) if theta is None else theta  # older configs' name for it
        scaling = model_config.get("rope_scaling")
        self.rope_scaling = 1.0 if scaling is None else scaling
        self.raw = dict(model_config)

    def get_kvslot_size(self, dtype: torch.dtype = torch.float16) -> int:
        """Bytes of KV cache one token occupies: K and V, every layer, every kv head."""
        per_layer = 2 * self.num_kv_heads * self.head_dim
        return per_layer * self.num_layers * dtype.itemsize

    @staticmethod
    def load_from_model_path(model_path: str) -> "LlamaModelConfig":
        with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
            return LlamaModelConfig(json.load(f))


# Llama-3-8B / 70B shapes for synthetic-weight benchmarks
LLAMA3_8B = dict(model_type="llama", num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                 hidden_size=4096, intermediate_size=14336, vocab_size=128256, max_position_embeddings=8192,
                 rope_theta=500000.0, rms_norm_eps=1e-5, hidden_act="silu", rope_scaling=None)
LLAMA3_70B = dict(model_type="llama", num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                  hidden_size=8192, intermediate_size=28672, vocab_size=128256, max_position_embeddings=8192,
                  rope_theta=500000.0, rms_norm_eps=1e-5, hidden_act="silu", rope_scaling=None)


# ---------------------------------------------------------------- Bupozen
@dataclasses.dataclass(frozen=True)
class LatentAttentionSpec:
    """Sizes and constants of one latent-attention mixer.  Per head: `dim` un-rotated and `rot_dim` rotated query / key entries,
    `vdim` value entries; all heads share one key/value latent of `kv_rank` entries plus one rotated key part of `rot_dim`."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    window: int                 # a query at position p sees p - window + 1 .. p; 0 = everything up to p
    rot_base: float
    rot_dims: int               # leading entries of the rotated part that turn (interleaved pairs); the rest pass through
    scale: float
    kv_from: Optional[int]      # layer whose cached latent / rotated key part this layer reads instead of making its own

    @property
    def cache_width(self) -> int:
        return self.kv_rank + self.rot_dim


@dataclasses.dataclass(frozen=True)
class WindowAttentionSpec:
    """Sizes and constants of one gated sliding-window attention mixer with grouped key/value heads: `heads` query heads share
    `kv_heads` key/value heads (query head h uses key/value head h // (heads // kv_heads)); per head `dim` query / key entries
    and `vdim` value entries; the softmax may have a value-less sink of score 0; the output has an element-wise sigmoid gate."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int                 # a query at position p sees p - window + 1 .. p; 0 = everything up to p
    rot_base: float
    rot_dims: int               # leading entries of every head that turn (interleaved pairs); the rest pass through
    scale: float
    sink: bool = True
    kv_from: Optional[int] = None   # every layer caches its own keys and values
    gate: bool = True               # element-wise sigmoid gate on the output (projection `g`)
    pair_halves: bool = False       # rotary pairs (i, i + rot_dims / 2) instead of (2i, 2i + 1)
    # (factor, original context, fast turns, slow turns): pairs that make fewer than `slow` turns over the original context are
    # slowed by `factor`, pairs that make more than `fast` are kept, a linear ramp between; cos and sin get 0.1 ln(factor) + 1
    rot_scaling: Optional[tuple] = None
    qk_unit_norm: bool = False      # rotated queries and keys are divided by their root mean square over the head
    softcap: float = 0.0            # > 0: score <- softcap * tanh(score / softcap)
    value_rotation: bool = False    # values are turned by their position over all vdim entries (plain frequencies of rot_base)
    out_scale: float = 1.0          # factor on the mixer's output (its weight in a sum of mixers)
    chunk: int = 0                  # > 0: a query at position p sees only positions >= floor(p / chunk) * chunk (and <= p)
    # score maps per head: every query head and key head has `maps` parts of `dim` entries, each part an attention of its own
    # over the head's values.  maps = 2 is differential attention: out = rms(map0 - lambda * map1) * (1 - diff), with
    # lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff from four learned vectors
    maps: int = 1
    diff: float = 0.0
    qk_weight_norm: bool = False    # RMS norm with a weight vector of `dim` entries on every query / key part BEFORE rotation
    bias: bool = False              # q, k, v and the output projection have biases

    @property
    def cache_width(self) -> int:
        return self.kv_heads * (self.maps * self.dim + self.vdim)

    @property
    def rot_key(self):
        """Key of the step's angle tables for queries and keys (TokenInferState.rotary)."""
        return (self.rot_base, self.rot_dims) if self.rot_scaling is None else (self.rot_base, self.rot_dims, self.rot_scaling)

    @property
    def vrot_key(self):
        return (self.rot_base, self.vdim) if self.value_rotation else None


@dataclasses.dataclass(frozen=True)
class LinearAttentionSpec:
    """Linear attention with a constant decay per head: S <- decay_h S + k v^T (dim x vdim per head, fp32, one per sequence),
    out = S^T q, with q, k, v = silu(projection); the heads' outputs are RMS-normed together (weight `norm`), gated by
    sigmoid(projection `g`) and projected."""
    heads: int
    dim: int
    vdim: int
    decay: tuple
    out_scale: float = 1.0


@dataclasses.dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers that read the same input; the result is left.out_scale * left + right.out_scale * right."""
    left: WindowAttentionSpec
    right: LinearAttentionSpec

    # the cache geometry is the attention's
    @property
    def kv_from(self):
        return self.left.kv_from

    @property
    def cache_width(self) -> int:
        return self.left.cache_width


@dataclasses.dataclass(frozen=True)
class GatedRecurrenceSpec:
    """A real-gated linear recurrent unit behind a causal convolution per channel, times a GELU branch: `width` channels whose
    two gates are block-diagonal projections (`blocks` blocks) of the convolution's output; `conv` taps.  No cache rows: the
    state (fp32 [width]) and the convolution's last conv - 1 inputs live per sequence."""
    width: int
    blocks: int
    conv: int
    kv_from: Optional[int] = None
    cache_width: int = 0            # no rows in the paged cache


@dataclasses.dataclass(frozen=True)
class MinGruSpec:
    """A gated recurrence whose gates read only the current token: z = sigmoid(W_z h + b), candidate c = g(W_x h + b) with
    g(u) = u + 1/2 for u >= 0 and sigmoid(u) below; S <- (1 - z) S + z c per channel (fp32, one per sequence); output
    W_o (S * silu(W_g h)).  No cache rows."""
    width: int
    kv_from: Optional[int] = None
    cache_width: int = 0


@dataclasses.dataclass(frozen=True)
class SelectiveScanSpec:
    """A selective state-space mixer: W_in h = [x | z] (`inner` channels each); x through a causal convolution of `conv` taps and a
    SiLU; W_x x = [dt (dt_rank) | B (state) | C (state)]; dt = softplus(W_dt dt + b); S[c, n] <- exp(dt_c A[c, n]) S + dt_c x_c B_n;
    y_c = sum_n S[c, n] C_n + D_c x_c; output W_o (y * silu(z)).  No cache rows: S (fp32 [inner, state]) and the convolution's last
    conv - 1 inputs live per sequence."""
    inner: int
    state: int
    dt_rank: int
    conv: int
    kv_from: Optional[int] = None
    cache_width: int = 0


@dataclasses.dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                   # "dense" | "moe"
    ff: int                     # hidden size of the dense layer / of ONE expert
    experts: int = 0
    top: int = 0
    # "relu2": relu(up)^2 | "clamped_glu": min(gate, limit) * sigmoid(1.702 .) * (clamp(up) + 1) | "silu_glu": silu(gate) * up
    # | "gelu_glu": gelu_tanh(gate) * up
    activation: str = "relu2"
    limit: float = 0.0          # clamped_glu: bound of the gate (above) and of the up projection (both sides)
    # routing.  "top_softmax": softmax over the `top` largest logits.  "softmax_grouped": scores are a softmax over all experts,
    # only experts of the `keep` best of `groups` groups can be chosen, the chosen scores are renormalised and scaled.
    # "sigmoid_bias": scores are sigmoids; the `top` largest score + bias (tensor `correction`) are chosen; weights are the scores.
    # "softmax_top": scores are a softmax over all experts; the `top` largest are chosen; weights are those scores as they are.
    routing: str = "top_softmax"
    groups: int = 1
    keep: int = 1
    route_scale: float = 1.0
    shared_ff: int = 0          # hidden size of a shared expert that every token uses (0: none)
    shared_limit: float = 0.0
    shared_gated: bool = False  # the shared expert's output is multiplied by sigmoid(w . h), one number per token


def _cache_geometry(mixers):
    """Layers that make their own cache rows own a slot; slots are grouped by row width (one cache tensor per width).
    -> (layer -> (row width, slot within that width's tensor), row width -> number of slots)."""
    cache_slot, slots_per_width = {}, {}
    for i, s in enumerate(mixers):
        if s.cache_width == 0:
            cache_slot[i] = None                # a mixer without cache rows (recurrent state only)
        elif s.kv_from is None:
            n = slots_per_width.get(s.cache_width, 0)
            cache_slot[i] = (s.cache_width, n)
            slots_per_width[s.cache_width] = n + 1
    for i, s in enumerate(mixers):
        if s.kv_from is not None:
            cache_slot[i] = cache_slot[s.kv_from]
    return cache_slot, slots_per_width


class BupozenModelConfig:
    """config.json of the Bupozen design: {"architecture": "Bupozen", "vocab", "width", "norm": {"eps"}, "layers": [{"type",
    "mixer": {...}, "mlp": {...} | null}, ...]}.  Every layer is a parallel block (one RMS norm feeds the mixer and the
    feed-forward); every size may differ from layer to layer."""
    family = "bupozen"
    embedding_scale = 1.0
    norm_unit_offset = False    # norm weights are stored as they are applied

    def __init__(self, model_config: dict):
        assert model_config.get("architecture") == "Bupozen", f"not a Bupozen config: {model_config.get('architecture')!r}"
        self.raw = dict(model_config)
        self.vocab_size = int(model_config["vocab"])
        self.hidden_size = int(model_config["width"])
        self.rms_norm_eps = float(model_config["norm"]["eps"])
        self.mixers, self.ffs = [], []
        for i, layer in enumerate(model_config["layers"]):
            assert layer["type"] == "latent_attention", f"layer {i}: unknown mixer type {layer['type']!r}"
            m = layer["mixer"]
            rot = m.get("rot") or {}
            mask = m.get("mask") or {}
            spec = LatentAttentionSpec(
                heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                q_rank=int(m["q_rank"]), window=int(mask.get("size", 0)), rot_base=float(rot.get("base", 10000.0)),
                rot_dims=int(rot.get("dims", m["rot_dim"])), scale=float(m["scale"]),
                kv_from=None if m.get("kv_from") is None else int(m["kv_from"]))
            assert spec.rot_dims % 2 == 0 and spec.rot_dims <= spec.rot_dim, f"layer {i}: rot.dims must be even and <= rot_dim"
            if spec.kv_from is not None:
                src = self.mixers[spec.kv_from] if spec.kv_from < i else None
                assert src is not None and src.kv_from is None and src.cache_width == spec.cache_width and \
                    src.kv_rank == spec.kv_rank, f"layer {i}: kv_from must name an earlier layer with its own latent of the same sizes"
            self.mixers.append(spec)
            f = layer.get("mlp")
            if f is None:
                self.ffs.append(None)
            elif f["kind"] == "dense":
                self.ffs.append(FeedForwardSpec("dense", int(f["ff"])))
            else:
                assert f["kind"] == "moe", f"layer {i}: unknown mlp kind {f['kind']!r}"
                self.ffs.append(FeedForwardSpec("moe", int(f["expert"]["ff"]), int(f["router"]["experts"]), int(f["router"]["top"])))
        self.num_layers = len(self.mixers)
        self.cache_slot, self.cache_slots_per_width = _cache_geometry(self.mixers)

    def get_kvslot_size(self, dtype: torch.dtype = torch.bfloat16) -> int:
        """Bytes of cache one token occupies: one [latent | rotated key part] row per layer that makes its own."""
        return sum(w * n for w, n in self.cache_slots_per_width.items()) * dtype.itemsize

    @staticmethod
    def load_from_model_path(model_path: str) -> "BupozenModelConfig":
        with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
            return BupozenModelConfig(json.load(f))


# ---------------------------------------------------------------- Rivudra
class RivudraModelConfig:
    """config.json of the Rivudra design: {"architecture": "Rivudra", "vocab", "width", "embedding": {"scale"}, "norm": {"eps"},
    "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base",
    "dims"}}, "mlp": {"kind": "moe", "router": {"experts", "top", "scale", "groups": {"count", "keep"}}, "expert": {"ff", "limit"},
    "shared": {"ff", "limit"}} | null}, ...]}.  Every layer is a parallel block (one RMS norm, weight stored around zero and
    applied as 1 + w, feeds the mixer and the feed-forward); every size may differ from layer to layer."""
    family = "rivudra"
    norm_unit_offset = True

    def __init__(self, model_config: dict):
        assert model_config.get("architecture") == "Rivudra", f"not a Rivudra config: {model_config.get('architecture')!r}"
        self.raw = dict(model_config)
        self.vocab_size = int(model_config["vocab"])
        self.hidden_size = int(model_config["width"])
        self.rms_norm_eps = float(model_config["norm"]["eps"])
        self.embedding_scale = float((model_config.get("embedding") or {}).get("scale", 1.0))
        self.mixers, self.ffs = [], []
        for i, layer in enumerate(model_config["layers"]):
            assert layer["type"] == "attention", f"layer {i}: unknown mixer type {layer['type']!r}"
            m = layer["mixer"]
            rot = m.get("rot") or {}
            mask = m.get("mask") or {}
            spec = WindowAttentionSpec(
                heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                window=int(mask.get("size", 0)), rot_base=float(rot.get("base", 10000.0)), rot_dims=int(rot.get("dims", 0)),
                scale=float(m["scale"]), sink=True)
            assert spec.heads % spec.kv_heads == 0, f"layer {i}: heads must be a multiple of kv_heads"
            assert spec.rot_dims % 2 == 0 and spec.rot_dims <= spec.dim, f"layer {i}: rot.dims must be even and <= dim"
            self.mixers.append(spec)
            f = layer.get("mlp")
            if f is None:
                self.ffs.append(None)
                continue
            assert f["kind"] == "moe", f"layer {i}: unknown mlp kind {f['kind']!r}"
            r, e, sh = f["router"], f["expert"], f.get("shared")
            groups = r.get("groups") or {}
            ff = FeedForwardSpec(
                "moe", int(e["ff"]), int(r["experts"]), int(r["top"]), activation="clamped_glu", limit=float(e["limit"]),
                routing="softmax_grouped", groups=int(groups.get("count", 1)), keep=int(groups.get("keep", groups.get("count", 1))),
                route_scale=float(r.get("scale", 1.0)), shared_ff=int(sh["ff"]) if sh else 0,
                shared_limit=float(sh["limit"]) if sh else 0.0)
            assert ff.experts % ff.groups == 0 and 0 < ff.keep <= ff.groups and ff.top <= ff.keep * (ff.experts // ff.groups), \
                f"layer {i}: {ff.top} experts cannot be chosen from {ff.keep} of {ff.groups} groups of {ff.experts} experts"
            self.ffs.append(ff)
        self.num_layers = len(self.mixers)
        self.cache_slot, self.cache_slots_per_width = _cache_geometry(self.mixers)

    def get_kvslot_size(self, dtype: torch.dtype = torch.bfloat16) -> int:
        """Bytes of cache one token occupies: one [keys | values] row per layer."""
        return sum(w * n for w, n in self.cache_slots_per_width.items()) * dtype.itemsize

    @staticmethod
    def load_from_model_path(model_path: str) -> "RivudraModelConfig":
        with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
            return RivudraModelConfig(json.load(f))


# ---------------------------------------------------------------- Buzarax
@dataclasses.dataclass(frozen=True)
class PairHashSpec:
    """A second embedding table indexed by a hash of (previous token, token): row (previous * mul_prev + token * mul_cur) mod
    buckets; the table's extra last row (number `buckets`) is the one of a sequence's first token."""
    buckets: int
    mul_prev: int
    mul_cur: int


class BuzaraxModelConfig:
    """config.json of the Buzarax design: {"architecture": "Buzarax", "vocab", "width", "norm": {"eps"}, "logit_softcap",
    "embedding": {"bigram": {"buckets", "mul_prev", "mul_cur"}}, "layers": [{"type": "parallel" | "rglru", "mixer": {...},
    "mlp": {"kind": "dense", "ff", "limit"} | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}} | null}, ...]}.
    "parallel": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot": {"base", "dims", "scaling": {"factor",
    "original", "fast", "slow"}}}, "right": {"heads", "dim", "vdim", "decay": [...]}, "left_scale", "right_scale"};
    "rglru": {"width", "blocks", "conv"}.  Layers are sequential blocks whose sublayers read the residual stream itself and
    whose outputs are normalised (one scalar gain) before they are added; after every layer the stream is a learned weighted
    sum of all earlier results (tensor `dwa`).  Every size may differ from layer to layer."""
    family = "buzarax"

    def __init__(self, model_config: dict):
        assert model_config.get("architecture") == "Buzarax", f"not a Buzarax config: {model_config.get('architecture')!r}"
        self.raw = dict(model_config)
        self.vocab_size = int(model_config["vocab"])
        self.hidden_size = int(model_config["width"])
        self.rms_norm_eps = float(model_config["norm"]["eps"])
        self.logit_softcap = float(model_config.get("logit_softcap") or 0.0)
        pair = (model_config.get("embedding") or {}).get("bigram")
        self.pair_hash = PairHashSpec(int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"])) if pair else None
        self.mixers, self.ffs = [], []
        for i, layer in enumerate(model_config["layers"]):
            m = layer["mixer"]
            if layer["type"] == "rglru":
                spec = GatedRecurrenceSpec(width=int(m["width"]), blocks=int(m["blocks"]), conv=int(m["conv"]))
                assert spec.width % spec.blocks == 0 and 1 <= spec.conv <= 8, f"layer {i}: width must split into blocks; 1 <= conv <= 8"
            else:
                assert layer["type"] == "parallel", f"layer {i}: unknown mixer type {layer['type']!r}"
                a, b = m["left"], m["right"]
                rot = a.get("rot") or {}
                sc = rot.get("scaling")
                left = WindowAttentionSpec(
                    heads=int(a["heads"]), kv_heads=int(a.get("kv_heads") or a["heads"]), dim=int(a["dim"]), vdim=int(a["vdim"]),
                    window=0, rot_base=float(rot.get("base", 10000.0)), rot_dims=int(rot.get("dims", 0)), scale=float(a["scale"]),
                    sink=True, gate=False, pair_halves=True,
                    rot_scaling=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None,
                    qk_unit_norm=True, softcap=float(a.get("softcap") or 0.0), value_rotation=True,
                    out_scale=float(m.get("left_scale", 1.0)))
                assert left.heads % left.kv_heads == 0, f"layer {i}: heads must be a multiple of kv_heads"
                assert left.rot_dims % 2 == 0 and left.rot_dims <= left.dim and left.vdim % 2 == 0, \
                    f"layer {i}: rot.dims must be even and <= dim, vdim even"
                right = LinearAttentionSpec(heads=int(b["heads"]), dim=int(b["dim"]), vdim=int(b["vdim"]),
                                            decay=tuple(float(d) for d in b["decay"]), out_scale=float(m.get("right_scale", 1.0)))
                assert len(right.decay) == right.heads, f"layer {i}: one decay per head"
                spec = ParallelMixerSpec(left, right)
            self.mixers.append(spec)
            f = layer.get("mlp")
            if f is None:
                self.ffs.append(None)
            elif f["kind"] == "dense":
                self.ffs.append(FeedForwardSpec("dense", int(f["ff"]), activation="clamped_glu", limit=float(f["limit"])))
            else:
                assert f["kind"] == "moe", f"layer {i}: unknown mlp kind {f['kind']!r}"
                self.ffs.append(FeedForwardSpec("moe", int(f["expert"]["ff"]), int(f["router"]["experts"]), int(f["router"]["top"]),
                                                activation="silu_glu", routing="sigmoid_bias"))
                assert self.ffs[-1].top <= self.ffs[-1].experts, f"layer {i}: top > experts"
        self.num_layers = len(self.mixers)
        self.cache_slot, self.cache_slots_per_width = _cache_geometry(self.mixers)

    def get_kvslot_size(self, dtype: torch.dtype = torch.bfloat16) -> int:
        """Bytes of cache one token occupies: one [keys | values] row per attention layer (recurrent layers hold none)."""
        return sum(w * n for w, n in self.cache_slots_per_width.items()) * dtype.itemsize

    def get_state_size(self, dtype: torch.dtype = torch.bfloat16) -> int:
        """Bytes of recurrent state one SEQUENCE occupies, whatever its length."""
        n = 4 if self.pair_hash else 0
        for s in self.mixers:
            if isinstance(s, GatedRecurrenceSpec):
                n += 4 * s.width + (s.conv - 1) * s.width * dtype.itemsize
            else:
                n += 4 * s.right.heads * s.right.dim * s.right.vdim
        return n

    @staticmethod
    def load_from_model_path(model_path: str) -> "BuzaraxModelConfig":
        with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
            return BuzaraxModelConfig(json.load(f))


# ---------------------------------------------------------------- Naforax
class NaforaxModelConfig:
    """config.json of the Naforax design: {"architecture": "Naforax", "vocab", "width", "norm": {"eps", "groups"}, "residual_mult",
    "logit_softcap", "canon": {"taps"}, "loop": {"start", "stop", "times"} | absent, "layers": [{"type": "attention" | "mingru" |
    "mamba1", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff",
    "limit"}, "shared": {"ff", "limit"} | absent} | null}, ...]}.
    "attention": {"heads", "kv_heads", "dim", "vdim", "scale", "diff", "mask": {"size"}, "rot": {"base", "dims"}};
    "mingru": {"width"}; "mamba1": {"inner", "state", "dt_rank", "conv"}.
    Layers are sandwich blocks, x <- x + m * norm_b(sublayer(c(norm_a(x)))): group RMS norms before and after every sublayer, and
    c(h) = h + causal per-channel convolution of h.  Layers start .. stop - 1 run `times` times in a row with the same weights;
    `runs` lists (layer, pass) in running order; every run owns its cache rows and recurrent state.  Every size may differ from
    layer to layer."""
    family = "naforax"

    def __init__(self, model_config: dict):
        assert model_config.get("architecture") == "Naforax", f"not a Naforax config: {model_config.get('architecture')!r}"
        self.raw = dict(model_config)
        self.vocab_size = int(model_config["vocab"])
        self.hidden_size = int(model_config["width"])
        self.rms_norm_eps = float(model_config["norm"]["eps"])
        self.norm_groups = int(model_config["norm"].get("groups", 1))
        assert self.hidden_size % self.norm_groups == 0, "norm.groups must divide the width"
        self.residual_mult = float(model_config.get("residual_mult", 1.0))
        self.logit_softcap = float(model_config.get("logit_softcap") or 0.0)
        self.canon_taps = int((model_config.get("canon") or {}).get("taps", 1))
        assert 1 <= self.canon_taps <= 8, "1 <= canon.taps <= 8"
        self.mixers, self.ffs = [], []
        for i, layer in enumerate(model_config["layers"]):
            m = layer["mixer"]
            if layer["type"] == "attention":
                rot = m.get("rot") or {}
                mask = m.get("mask") or {}
                spec = WindowAttentionSpec(
                    heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                    window=0, rot_base=float(rot.get("base", 10000.0)), rot_dims=int(rot.get("dims", 0)), scale=float(m["scale"]),
                    sink=False, gate=True, chunk=int(mask.get("size", 0)), maps=2, diff=float(m["diff"]), qk_weight_norm=True,
                    bias=True)
                assert spec.heads % spec.kv_heads == 0, f"layer {i}: heads must be a multiple of kv_heads"
                assert spec.rot_dims % 2 == 0 and spec.rot_dims <= spec.dim, f"layer {i}: rot.dims must be even and <= dim"
            elif layer["type"] == "mingru":
                spec = MinGruSpec(width=int(m["width"]))
            else:
                assert layer["type"] == "mamba1", f"layer {i}: unknown mixer type {layer['type']!r}"
                spec = SelectiveScanSpec(inner=int(m["inner"]), state=int(m["state"]), dt_rank=int(m["dt_rank"]), conv=int(m["conv"]))
                assert 1 <= spec.conv <= 8 and 1 <= spec.state <= 256, f"layer {i}: 1 <= conv <= 8, 1 <= state <= 256"
            self.mixers.append(spec)
            f = layer.get("mlp")
            if f is None:
                self.ffs.append(None)
            elif f["kind"] == "dense":
                self.ffs.append(FeedForwardSpec("dense", int(f["ff"]), activation="gelu_glu"))
            else:
                assert f["kind"] == "moe", f"layer {i}: unknown mlp kind {f['kind']!r}"
                r, e, sh = f["router"], f["expert"], f.get("shared")
                ff = FeedForwardSpec("moe", int(e["ff"]), int(r["experts"]), int(r["top"]), activation="clamped_glu",
                                     limit=float(e["limit"]), routing="softmax_top", shared_ff=int(sh["ff"]) if sh else 0,
                                     shared_limit=float(sh["limit"]) if sh else 0.0, shared_gated=bool(sh))
                assert 0 < ff.top <= ff.experts, f"layer {i}: top must be in 1 .. experts"
                self.ffs.append(ff)
        self.num_layers = len(self.mixers)
        loop = model_config.get("loop")
        if loop:
            a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            assert 0 <= a < b <= self.num_layers and times >= 1, "loop: 0 <= start < stop <= layers, times >= 1"
            self.loop = (a, b, times)
            self.runs = [(i, 0) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + \
                [(i, 0) for i in range(b, self.num_layers)]
        else:
            self.loop = None
            self.runs = [(i, 0) for i in range(self.num_layers)]
        # cache rows and state are per RUN (a repeated layer keeps one set per pass)
        self.cache_slot, self.cache_slots_per_width = _cache_geometry([self.mixers[i] for i, _ in self.runs])

    def get_kvslot_size(self, dtype: torch.dtype = torch.bfloat16) -> int:
        """Bytes of cache one token occupies: one [keys of both maps | values] row per attention run."""
        return sum(w * n for w, n in self.cache_slots_per_width.items()) * dtype.itemsize

    def get_state_size(self, dtype: torch.dtype = torch.bfloat16) -> int:
        """Bytes of recurrent state one SEQUENCE occupies, whatever its length: the input convolutions' last inputs of both
        sublayers (fp32) of every run, and the mixers' states."""
        n = 0
        for i, _ in self.runs:
            s = self.mixers[i]
            n += 4 * (self.canon_taps - 1) * self.hidden_size * (1 if self.ffs[i] is None else 2)
            if isinstance(s, MinGruSpec):
                n += 4 * s.width
            elif isinstance(s, SelectiveScanSpec):
                n += 4 * s.inner * s.state + (s.conv - 1) * s.inner * dtype.itemsize
        return n

    @staticmethod
    def load_from_model_path(model_path: str) -> "NaforaxModelConfig":
        with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
            return NaforaxModelConfig(json.load(f))

"""Softmax attention mixer with grouped key/value heads over the paged cache: ONE fused GEMM [q ; k ; v (; gate)] on the block's
input -> (rotary of k + cache store, one kernel) -> attention (rotary of q, window, softmax with an optional sink, optional
sigmoid output gate: one kernel) -> o GEMM.  The specification's options (model_config.WindowAttentionSpec: rotary pairs as
halves, stretched frequencies, unit-RMS queries and keys, capped scores, values turned by their position) go to the same two
kernels.  `attend` is the part between the two GEMMs, for mixers that fuse their projections with a neighbour's.

`DifferentialAttentionMixer`: two score maps per head over the same values.  Every map is a query head of its own for the same two
kernels (twice the heads, `vshare` = 2 key heads per value head, fp32 output); one more kernel subtracts the maps, normalises
the head and applies the gate."""
import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.window_attn import AttnOptions, diff_combine, window_attention, window_kv_store


class WindowAttentionMixer:
    def __init__(self, spec, weight, eps: float, cache_key):
        self.spec, self.weight = spec, weight
        self.cache_width, self.cache_slot = cache_key          # which cache tensor and which of its slots this layer uses
        self.options = AttnOptions(pair_halves=spec.pair_halves, qk_norm_eps=eps if spec.qk_unit_norm else -1.0,
                                   softcap=spec.softcap, out_scale=spec.out_scale)

    def register(self, model):
        m = self.spec
        model._register_rotary(m.rot_key, m.rot_base, m.rot_dims, m.rot_scaling)
        if m.value_rotation:
            model._register_rotary(m.vrot_key, m.rot_base, m.vdim)

    @property
    def proj_widths(self):
        """Columns of the fused input projection: q, k, v (, gate)."""
        m = self.spec
        return [m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim] + ([m.heads * m.vdim] if m.gate else [])

    def attend(self, q, k, v, gate, out, caches: dict, block_table, st):
        """q [T, H dk], k [T, G dk], v [T, G dv], gate [T, H dv] or None (column slices of a wider matrix are fine) -> out [T, H dv]."""
        m = self.spec
        if st.ignore_kvcache:
            out.zero_()
            return
        cos, sin = st.rotary[m.rot_key] if m.rot_dims > 0 else (None, None)
        vcos, vsin = st.rotary[m.vrot_key] if m.value_rotation else (None, None)
        cache = caches[self.cache_width]
        window_kv_store(k, v, cache, self.cache_slot, block_table, st, m.kv_heads, m.dim, m.vdim, m.rot_dims, cos, sin,
                        self.options, vcos, vsin)
        window_attention(q, gate, cache, self.cache_slot, block_table, st, out, m.heads, m.kv_heads, m.dim, m.vdim,
                         m.rot_dims, m.window, m.scale, m.sink, cos, sin, self.options, vcos, vsin)

    def forward(self, h: torch.Tensor, caches: dict, block_table: torch.Tensor, st) -> torch.Tensor:
        m, w = self.spec, self.weight
        proj = linear(h, w.in_proj)                             # [T, H dk | G dk | G dv (| H dv)]
        parts = list(torch.split(proj, self.proj_widths, dim=1)) + [None]
        out = torch.empty((h.shape[0], m.heads * m.vdim), dtype=h.dtype, device=h.device)
        self.attend(parts[0], parts[1], parts[2], parts[3], out, caches, block_table, st)
        return linear(out, w.o)


class DifferentialAttentionMixer:
    """ONE GEMM with bias [q ; k ; v ; gate] (q rows ordered [key/value head][map][head of the group] at load time) -> per-part
    RMS norm with weight + rotary of k + cache store (one kernel; the row holds both maps' keys and ONE set of values) ->
    attention per map (norm + rotary of q, chunked causal mask, softmax, fp32 output: one kernel) -> map 0 - lambda * map 1,
    unit-RMS over the head, (1 - diff), sigmoid gate (one kernel) -> o GEMM with bias."""

    def __init__(self, spec, weight, eps: float, cache_key):
        assert spec.maps == 2 and spec.qk_weight_norm and spec.gate and not spec.value_rotation and not spec.sink
        self.spec, self.weight, self.eps = spec, weight, eps
        self.cache_width, self.cache_slot = cache_key
        self.options = AttnOptions(pair_halves=spec.pair_halves, softcap=spec.softcap, q_norm=weight.q_norm, k_norm=weight.k_norm,
                                   prenorm_eps=eps, chunk=spec.chunk, vshare=spec.maps, out_f32=True)

    def register(self, model):
        m = self.spec
        model._register_rotary(m.rot_key, m.rot_base, m.rot_dims, m.rot_scaling)

    def state_layout(self) -> dict:
        return {}

    @property
    def proj_widths(self):
        m = self.spec
        return [m.heads * m.maps * m.dim, m.kv_heads * m.maps * m.dim, m.kv_heads * m.vdim, m.heads * m.vdim]

    def forward(self, h: torch.Tensor, caches: dict, block_table: torch.Tensor, states, st) -> torch.Tensor:
        m, w = self.spec, self.weight
        T = h.shape[0]
        proj = torch.nn.functional.linear(h, w.in_proj, w.in_bias)
        q, k, v, gate = torch.split(proj, self.proj_widths, dim=1)
        out = torch.empty((T, m.heads * m.vdim), dtype=h.dtype, device=h.device)
        if st.ignore_kvcache:
            out.zero_()
            return torch.nn.functional.linear(out, w.o, w.o_bias)
        cos, sin = st.rotary[m.rot_key] if m.rot_dims > 0 else (None, None)
        cache = caches[self.cache_width]
        H2, G2 = m.heads * m.maps, m.kv_heads * m.maps
        window_kv_store(k, v, cache, self.cache_slot, block_table, st, G2, m.dim, m.vdim, m.rot_dims, cos, sin, self.options)
        a = torch.empty((T, H2 * m.vdim), dtype=torch.float32, device=h.device)
        window_attention(q, None, cache, self.cache_slot, block_table, st, a, H2, G2, m.dim, m.vdim, m.rot_dims, m.window,
                         m.scale, False, cos, sin, self.options)
        diff_combine(a, gate, out, m.heads, m.kv_heads, m.vdim, w.lam, self.eps, 1.0 - m.diff)
        return torch.nn.functional.linear(out, w.o, w.o_bias)

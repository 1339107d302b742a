"""TEST INFRASTRUCTURE: run the PRODUCT's host path (swiftllm_b200.LlamaModel: metadata staging, infer state, block manager
with its host mirror, layer sequencing, last-token gather, swap / free) on the CPU of the build container, with every CUDA
kernel wrapper replaced by the oracle's restatement of that kernel.  Nothing here ships; the product itself has no CPU path
(its wrappers fail loudly without the CUDA library).  What this buys: the Python side of the data plane is exercised by
`-m "not gpu"` tests against `oracle.model.OracleLlama`, so host-logic regressions are caught before a GPU is involved."""
from __future__ import annotations

import contextlib
import importlib

import torch
from torch.overrides import TorchFunctionMode

from oracle import kernels as K


def _is_cuda_dev(x):
    return (isinstance(x, torch.device) and x.type == "cuda") or (isinstance(x, str) and x.startswith("cuda"))


class _CudaToCpu(TorchFunctionMode):
    """device=cuda -> cpu (positional or keyword), pinned host memory -> ordinary memory."""

    def __torch_function__(self, func, types_, args=(), kwargs=None):
        kwargs = dict(kwargs or {})
        if getattr(func, "__name__", "") == "pin_memory":
            return args[0]
        if kwargs.get("pin_memory", False):
            kwargs["pin_memory"] = False
        to_cuda = False
        if "device" in kwargs and _is_cuda_dev(kwargs["device"]):
            kwargs["device"] = "cpu"; to_cuda = True
        if any(_is_cuda_dev(a) for a in args):
            args = tuple("cpu" if _is_cuda_dev(a) else a for a in args); to_cuda = True
        out = func(*args, **kwargs)
        # a host -> device transfer always yields a NEW tensor; `.to("cpu")` of a CPU tensor would alias its source
        if to_cuda and getattr(func, "__name__", "") in ("to", "cuda") and args and out is args[0]:
            out = out.clone()
        return out


# ---------------------------------------------------------------- oracle-backed stand-ins of the kernel wrappers
def _fused_add_rmsnorm_inplace(x, residual, weight, eps):
    xo, ro = K.fused_add_rmsnorm(x, residual, weight, eps)
    x.copy_(xo); residual.copy_(ro)


def _rmsnorm_inplace(x, weight, eps):
    x.copy_(K.rmsnorm(x, weight, eps))


def _rotary_embedding_inplace(q, k, infer_state):
    qo, ko = K.rotary_embedding(q, k, infer_state.position_cos, infer_state.position_sin)
    q.copy_(qo); k.copy_(ko)


def _silu_and_mul_inplace(x):
    F = x.shape[1] // 2
    x[:, :F] = K.silu_and_mul(x)[:, :F]


def _store_kvcache(k, v, k_cache, v_cache, block_table, model_config, engine_config, st, cur_layer):
    kw = {}
    if getattr(st, "prefill_prefix_lens", None) is not None:
        kw["prefill_prefix_lens"] = st.prefill_prefix_lens.tolist()
    K.store_kvcache_inplace(k, v, k_cache, v_cache, block_table.numpy(), st.seq_ids.tolist(), st.prefill_seq_start_locs.tolist(),
                            st.prefill_seq_lens.tolist(), st.decoding_seq_lens.tolist(), st.num_prefill_seqs, st.num_prefill_tokens,
                            k_cache.shape[3], cur_layer, **kw)


def _rotary_store_kvcache_decode(q, k, v, k_cache, v_cache, block_table, st, cur_layer):
    assert st.num_prefill_seqs == 0
    _rotary_embedding_inplace(q, k, st)
    K.store_kvcache_inplace(k, v, k_cache, v_cache, block_table.numpy(), st.seq_ids.tolist(), [], [], st.decoding_seq_lens.tolist(),
                            0, 0, k_cache.shape[3], cur_layer)


def _paged_attention(q, k_cache, v_cache, block_table, model_config, engine_config, st, cur_layer, o):
    out = K.paged_attention_exact(q, k_cache, v_cache, block_table.numpy(), st.seq_ids[st.num_prefill_seqs:].tolist(),
                                  st.decoding_seq_lens.tolist(), st.softmax_scale, k_cache.shape[3], cur_layer, q.dtype)
    o.copy_(out.reshape(o.shape))


def _prefill_attention(q, k, v, o, model_config, engine_config, st):
    out = K.prefill_attention_exact(q, k, v, st.prefill_seq_start_locs.tolist(), st.prefill_seq_lens.tolist(), st.softmax_scale, q.dtype)
    o.copy_(out.reshape(o.shape))


def _prefill_attention_paged(q, k_cache, v_cache, block_table, o, model_config, engine_config, st, cur_layer):
    out = K.prefix_prefill_attention_exact(q, k_cache, v_cache, block_table.numpy(), st.seq_ids[:st.num_prefill_seqs].tolist(),
                                           st.prefill_seq_start_locs.tolist(), st.prefill_seq_lens.tolist(),
                                           st.prefill_prefix_lens.tolist(), st.softmax_scale, k_cache.shape[3], cur_layer, q.dtype)
    o.copy_(out.reshape(o.shape))


def _allocate_blocks(nsab, block_table, is_free, seq_ids, target_lens, block_size, new_blocks, status):
    """block_manager.py:43-79 of the reference: the lowest free ids, ascending, handed out in batch order."""
    free_ids = torch.nonzero(is_free).flatten().tolist()
    p, out = 0, []
    for sid, tl in zip(seq_ids.tolist(), target_lens.tolist()):
        have = int(nsab[sid])
        need = (tl + block_size - 1) // block_size - have
        for i in range(need):
            b = free_ids[p]; p += 1
            block_table[sid, have + i] = b
            is_free[b] = False
            out.append(b)
        nsab[sid] = have + need
    if new_blocks is not None and out:
        new_blocks.copy_(torch.tensor(out, dtype=torch.int64))


def _unset(nsab, block_table, seq_ids, is_free):
    for sid in seq_ids.tolist():
        n = int(nsab[sid])
        is_free[block_table[sid, :n].long()] = True
        nsab[sid] = 0


def _gather_and_unset(nsab, block_table, seq_ids, is_free, total_blocks=None):
    ids = []
    for sid in seq_ids.tolist():
        ids += block_table[sid, : int(nsab[sid])].tolist()
    _unset(nsab, block_table, seq_ids, is_free)
    return torch.tensor(ids, dtype=torch.int32)


def _swap_blocks(src_ids, dst_ids, is_swap_in, k_cache, v_cache, k_swap, v_swap):
    K.swap_blocks_inplace(src_ids, dst_ids, is_swap_in, k_cache, v_cache, k_swap, v_swap)



# ---------------------------------------------------------------- stand-ins of the parallel-block / latent-attention kernels
# (restated from the kernels' contracts in include/swiftllm_b200.h; fp32 arithmetic, results rounded to the storage dtype)
def _add_rmsnorm_f32(residual, a, b, weight, eps, out=None, out_dtype=None):
    if a is not None or b is not None:
        y = a.float() if a is not None else torch.zeros_like(residual)
        if b is not None:
            y = y + b.float()
        residual += y
    o = (residual / torch.sqrt((residual * residual).mean(-1, keepdim=True) + eps) * weight.float()).to(
        out.dtype if out is not None else (out_dtype or weight.dtype))
    if out is None:
        return o
    out.copy_(o)
    return out


def _rmsnorm_strided(x, weight, eps):
    xf = x.float()
    return (xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def _relu2_inplace(x):
    x.copy_((torch.relu(x.float()) ** 2).to(x.dtype))


def _moe_route(logits, top):
    vals, idx = torch.topk(logits, top, dim=-1)
    return torch.zeros_like(logits).scatter_(1, idx, torch.softmax(vals, dim=-1))


def _moe_relu2_scale_inplace(u, weights, ff):
    T, E = weights.shape
    u.copy_(((torch.relu(u.float()) ** 2).view(T, E, ff) * weights[:, :, None]).view(T, E * ff).to(u.dtype))


def _rot_pairs(v, cos, sin, rot_dims):
    """v [T, ..., d] fp32; pairs (2i, 2i+1) of the first rot_dims entries turn by the angles cos/sin [T, rot_dims/2]."""
    if rot_dims == 0:
        return v
    shape = (v.shape[0],) + (1,) * (v.dim() - 2) + (rot_dims // 2,)
    c, s = cos.view(shape), sin.view(shape)
    u, w = v[..., 0:rot_dims:2], v[..., 1:rot_dims:2]
    out = v.clone()
    out[..., 0:rot_dims:2] = u * c - w * s
    out[..., 1:rot_dims:2] = w * c + u * s
    return out


def _cache_rows(cache, slot, block_table, seq, positions):
    bs = cache.shape[2]
    blocks = block_table[seq, torch.as_tensor(positions) // bs].long()
    return cache[blocks, slot, torch.as_tensor(positions) % bs]


def _latent_kv_store(dkv, norm_weight, cache, slot, block_table, st, r, dr, rot_dims, eps, cos, sin):
    c = _rmsnorm_strided(dkv[:, :r], norm_weight, eps)
    kr = _rot_pairs(dkv[:, r:].float(), cos, sin, rot_dims).to(dkv.dtype)
    bs = cache.shape[2]
    for t, (sq, p) in enumerate(zip(st.token_seq_ids.tolist(), st.token_positions.tolist())):
        cache[int(block_table[sq, p // bs]), slot, p % bs] = torch.cat([c[t], kr[t]])


def _latent_attention(q_lat, q_rot, gate, cache, slot, block_table, st, out, rot_dims, window, scale, cos, sin):
    r = q_lat.shape[2]
    qr = _rot_pairs(q_rot.float(), cos, sin, rot_dims)
    qa = torch.cat([q_lat.float(), qr], dim=-1) * scale                     # [T, H, r + dr]
    for t, (sq, p) in enumerate(zip(st.token_seq_ids.tolist(), st.token_positions.tolist())):
        lo = max(0, p - window + 1) if window > 0 else 0
        rows = _cache_rows(cache, slot, block_table, sq, list(range(lo, p + 1))).float()      # [n, r + dr]
        pr = torch.softmax(qa[t] @ rows.T, dim=-1)                          # [H, n]
        o = pr @ rows[:, :r]
        if gate is not None:
            o = o * torch.sigmoid(gate[t].float())[:, None]
        out[t] = o.to(out.dtype)


def _moe_route_grouped(logits, top, groups, keep, scale, norm_eps):
    s = torch.softmax(logits, dim=-1)
    T, E = s.shape
    gbest = s.view(T, groups, E // groups).max(-1).values
    kept = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, torch.topk(gbest, keep, dim=-1).indices, True)
    choice = s.masked_fill(~kept.repeat_interleave(E // groups, dim=1), float("-inf"))
    idx = torch.topk(choice, top, dim=-1).indices
    w = s.gather(1, idx)
    return torch.zeros_like(s).scatter_(1, idx, w / (w.sum(-1, keepdim=True) + norm_eps) * scale)


def _moe_clamped_glu_scale(u, weights, experts, ff, limit, shared_ff, shared_limit, alpha, shared_gated=False):
    T = u.shape[0]
    uf = u.float()

    def act(block, n, lim):
        g, v = block[..., :n].clamp(max=lim), block[..., n:].clamp(-lim, lim)
        return g * torch.sigmoid(alpha * g) * (v + 1.0)
    parts = []
    if experts:
        parts.append((act(uf[:, :2 * experts * ff].view(T, experts, 2 * ff), ff, limit) * weights[:, :experts, None]).reshape(T, experts * ff))
    if shared_ff:
        parts.append(act(uf[:, 2 * experts * ff:], shared_ff, shared_limit) * (weights[:, experts:experts + 1] if shared_gated else 1.0))
    return torch.cat(parts, dim=1).to(u.dtype)


def _rot_any(v, cos, sin, rot_dims, halves):
    """v [T, ..., d] fp32; halves: pairs (i, i + rot_dims/2), else (2i, 2i+1)."""
    if not halves:
        return _rot_pairs(v, cos, sin, rot_dims)
    if rot_dims == 0:
        return v
    hf = rot_dims // 2
    shape = (v.shape[0],) + (1,) * (v.dim() - 2) + (hf,)
    c, s = cos.view(shape), sin.view(shape)
    u, w = v[..., :hf], v[..., hf:rot_dims]
    out = v.clone()
    out[..., :hf] = u * c - w * s
    out[..., hf:rot_dims] = w * c + u * s
    return out


def _unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def _window_kv_store(k, v, cache, slot, block_table, st, kv_heads, dk, dv, rot_dims, cos, sin, opt=None, vcos=None, vsin=None):
    T = k.shape[0]
    halves = bool(opt and opt.pair_halves)
    kr = k.float().view(T, kv_heads, dk)
    if opt and opt.k_norm is not None:
        kr = _unit_rms(kr, opt.prenorm_eps) * opt.k_norm
    kr = _rot_any(kr, cos, sin, rot_dims, halves)
    if opt and opt.qk_norm_eps >= 0:
        kr = _unit_rms(kr, opt.qk_norm_eps)
    kr = kr.reshape(T, kv_heads * dk).to(k.dtype)
    if vcos is not None:
        v = _rot_any(v.float().view(T, kv_heads, dv), vcos, vsin, dv, halves).reshape(T, kv_heads * dv).to(k.dtype)
    bs = cache.shape[2]
    for t, (sq, p) in enumerate(zip(st.token_seq_ids.tolist(), st.token_positions.tolist())):
        cache[int(block_table[sq, p // bs]), slot, p % bs] = torch.cat([kr[t], v[t]])


def _window_attention(q, gate, cache, slot, block_table, st, out, heads, kv_heads, dk, dv, rot_dims, window, scale, sink, cos, sin,
                      opt=None, vcos=None, vsin=None):
    T = q.shape[0]
    halves = bool(opt and opt.pair_halves)
    qa = q.float().view(T, heads, dk)
    if opt and opt.q_norm is not None:
        qa = _unit_rms(qa, opt.prenorm_eps) * opt.q_norm
    qa = _rot_any(qa, cos, sin, rot_dims, halves)
    if opt and opt.qk_norm_eps >= 0:
        qa = _unit_rms(qa, opt.qk_norm_eps)
    qa = qa * scale
    rep = heads // kv_heads
    vshare = opt.vshare if opt else 1
    for t, (sq, p) in enumerate(zip(st.token_seq_ids.tolist(), st.token_positions.tolist())):
        lo = max(0, p - window + 1) if window > 0 else 0
        if opt and opt.chunk > 0:
            lo = max(lo, p // opt.chunk * opt.chunk)
        rows = _cache_rows(cache, slot, block_table, sq, list(range(lo, p + 1))).float()      # [n, G dk + G / vshare dv]
        ks = rows[:, :kv_heads * dk].view(-1, kv_heads, dk).repeat_interleave(rep, dim=1)     # [n, H, dk]
        vs = rows[:, kv_heads * dk:].view(-1, kv_heads // vshare, dv).repeat_interleave(rep * vshare, dim=1)
        sc = torch.einsum("hd,nhd->hn", qa[t], ks)
        if opt and opt.softcap > 0:
            sc = opt.softcap * torch.tanh(sc / opt.softcap)
        if sink:
            sc = torch.cat([sc, torch.zeros(heads, 1)], dim=1)
        pr = torch.softmax(sc, dim=-1)[:, :rows.shape[0]]
        o = torch.einsum("hn,nhd->hd", pr, vs)
        if vcos is not None:
            o = _rot_any(o[None], vcos[t:t + 1], -vsin[t:t + 1], dv, halves)[0]
        o = o.reshape(heads * dv) * (opt.out_scale if opt else 1.0)
        if gate is not None:
            o = o * torch.sigmoid(gate[t].float())
        out[t] = o.to(out.dtype)


def _diff_combine(a, gate, out, heads, kv_heads, dv, lam, eps, factor):
    T, hq = a.shape[0], heads // kv_heads
    maps = a.view(T, kv_heads, 2, hq, dv)
    o = _unit_rms(maps[:, :, 0] - lam * maps[:, :, 1], eps).reshape(T, heads * dv) * factor
    if gate is not None:
        o = o * torch.sigmoid(gate.float())
    out.copy_(o.to(out.dtype))


# ---------------------------------------------------------------- stand-ins of the sandwich-block kernels
def _group_rms(x, groups, eps):
    T, W = x.shape
    return _unit_rms(x.view(T, groups, W // groups), eps).reshape(T, W)


def _group_norm_add_norm(x, y, wb, mult, wn, eps, groups, n_out=None):
    if y is not None:
        x += mult * _group_rms(y.float(), groups, eps) * wb
    if wn is None:
        return None
    n = _group_rms(x, groups, eps) * wn
    if n_out is not None:
        n_out.copy_(n)
        return n_out
    return n


def _group_norm_cast(x, w, eps, groups, out_dtype):
    return (_group_rms(x, groups, eps) * w).to(out_dtype)


def _stream_add(x, a=None, v=None):
    if a is not None:
        x += a
    if v is not None:
        x += v


def _gelu_glu(u):
    F = u.shape[1] // 2
    uf = u.float()
    return (torch.nn.functional.gelu(uf[:, :F], approximate="tanh") * uf[:, F:]).to(u.dtype)


def _moe_route_softmax(logits, experts, top, gated):
    s = torch.softmax(logits[:, :experts], dim=-1)
    idx = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    w = torch.zeros_like(logits)
    w[:, :experts] = torch.zeros_like(s).scatter_(1, idx, s.gather(1, idx))
    if gated:
        w[:, experts] = torch.sigmoid(logits[:, experts])
    return w


def _linear_f32_out(a, w):
    return a.float() @ w.float().t()


def _short_conv(xin, w, bias, tail, st, out_dtype, add_input=False, silu=False, move_tail=False):
    T, C = xin.shape
    K = w.shape[1]
    xf = xin.float()
    out = torch.zeros((T, C))
    pos = st.token_positions.tolist()
    for sq, lo, hi in _segments(st):
        for t in range(lo, hi):
            acc = torch.zeros(C) if bias is None else bias.clone()
            for k in range(K):
                if pos[t] - k < 0:
                    continue
                src = xf[t - k] if t - k >= lo else tail[sq, K - 1 - (k - (t - lo))].float()
                acc = acc + w[:, K - 1 - k] * src
            if silu:
                acc = torch.nn.functional.silu(acc)
            out[t] = acc + (xf[t] if add_input else 0.0)
    if move_tail and K > 1:
        _conv_tail_update(xin, tail, st)
    return out.to(out_dtype)


def _conv_tail_update(xin, tail, st):
    K = tail.shape[1] + 1
    pos = st.token_positions.tolist()
    for sq, lo, hi in _segments(st):
        old = tail[sq].clone() if pos[lo] > 0 else torch.zeros_like(tail[sq])
        hist = torch.cat([old, xin[lo:hi].to(tail.dtype)], dim=0)
        tail[sq] = hist[-(K - 1):]


def _mingru_scan(proj, state, st, channels):
    C = channels
    pf = proj.float()
    out = torch.zeros((proj.shape[0], C))
    pos = st.token_positions.tolist()
    for sq, lo, hi in _segments(st):
        S = state[sq].clone() if pos[lo] > 0 else torch.zeros(C)
        for t in range(lo, hi):
            z, u, g = torch.sigmoid(pf[t, :C]), pf[t, C:2 * C], pf[t, 2 * C:]
            S = (1.0 - z) * S + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            out[t] = S * torch.nn.functional.silu(g)
        state[sq] = S
    return out.to(proj.dtype)


def _selective_scan(x, dt, dt_bias, A, bc, b_off, c_off, D, z, state, st):
    T, C = x.shape
    N = A.shape[1]
    xf, zf, bcf = x.float(), z.float(), bc.float()
    step = torch.nn.functional.softplus(dt.float() + dt_bias)
    out = torch.zeros((T, C))
    pos = st.token_positions.tolist()
    for sq, lo, hi in _segments(st):
        S = state[sq].clone() if pos[lo] > 0 else torch.zeros((C, N))
        for t in range(lo, hi):
            S = torch.exp(step[t][:, None] * A) * S + (step[t] * xf[t])[:, None] * bcf[t, b_off:b_off + N][None, :]
            out[t] = ((S * bcf[t, c_off:c_off + N][None, :]).sum(1) + D * xf[t]) * torch.nn.functional.silu(zf[t])
        state[sq] = S
    return out.to(x.dtype)


# ---------------------------------------------------------------- stand-ins of the sequential-block / recurrent kernels
def _segments(st):
    s = st.seg_starts.tolist()
    return [(sq, s[b], s[b + 1]) for b, sq in enumerate(st.seq_ids.tolist()) if s[b + 1] > s[b]]


def _embed_pair_hash(tokens, st, last_token, embed, pairs, buckets, mul_prev, mul_cur, x_copy=None):
    x = embed[tokens.long()].float()
    if pairs is not None:
        pos = st.token_positions.tolist()
        toks = tokens.tolist()
        for sq, lo, hi in _segments(st):
            for t in range(lo, hi):
                if pos[t] == 0:
                    row = buckets
                else:
                    prev = toks[t - 1] if t > lo else int(last_token[sq])
                    row = (prev * mul_prev + toks[t] * mul_cur) % buckets
                x[t] += pairs[row].float()
            last_token[sq] = toks[hi - 1]
    if x_copy is not None:
        x_copy.copy_(x)
    return x, x.to(embed.dtype)


def _postnorm_add_mix(x, y, gain, eps, h, history=None, slot=0, mix=None):
    if y is not None:
        x += _unit_rms(y.float(), eps) * gain
    if history is not None:
        history[slot] = x
    if mix is not None:
        x.copy_(sum(mix[j] * history[j] for j in range(slot + 1)))
    h.copy_(x.to(h.dtype))


def _tanh_cap_inplace(x, cap):
    x.copy_(cap * torch.tanh(x / cap))


def _moe_route_sigmoid(logits, bias, top):
    s = torch.sigmoid(logits)
    idx = torch.topk(s + (bias if bias is not None else 0.0), top, dim=-1).indices
    return torch.zeros_like(s).scatter_(1, idx, s.gather(1, idx))


def _moe_silu_glu_scale(u, weights, experts, ff):
    T = u.shape[0]
    b = u.float().view(T, experts, 2 * ff)
    g, v = b[..., :ff], b[..., ff:]
    return (g * torch.sigmoid(g) * v * weights[:, :, None]).reshape(T, experts * ff).to(u.dtype)


def _causal_conv(xin, w, bias, tail, st):
    T, C = xin.shape
    K = w.shape[1]
    u = torch.zeros(T, C)
    pos = st.token_positions.tolist()
    for sq, lo, hi in _segments(st):
        before = tail[sq].float() if (K > 1 and pos[lo] > 0) else torch.zeros(K - 1, C)
        seq = torch.cat([before, xin[lo:hi].float()])                         # row K-1 + i: the segment's token i
        for i in range(hi - lo):
            u[lo + i] = (bias.float() if bias is not None else 0.0) + (seq[i:i + K] * w.float().T).sum(0)
    return u.to(xin.dtype)


def _rglru_scan(u, gates, ybr, rate, xin, state, tail, st):
    T, C = u.shape
    blocks, K = gates.shape[0], tail.shape[1] + 1
    cb = C // blocks
    g = gates.float()
    r = torch.sigmoid(g[:, :, :cb]).transpose(0, 1).reshape(T, C)
    ig = torch.sigmoid(g[:, :, cb:]).transpose(0, 1).reshape(T, C)
    a = torch.exp(rate * r)
    y = ybr.float()
    gelu = 0.5 * y * (1.0 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
    out = torch.zeros(T, C)
    pos = st.token_positions.tolist()
    for sq, lo, hi in _segments(st):
        S = state[sq].clone() if pos[lo] > 0 else torch.zeros(C)
        for t in range(lo, hi):
            S = a[t] * S + torch.sqrt(torch.clamp(1.0 - a[t] * a[t], min=0.0)) * (ig[t] * u[t].float())
            out[t] = S * gelu[t]
        state[sq] = S
        if K > 1:
            before = tail[sq].float() if pos[lo] > 0 else torch.zeros(K - 1, C)
            tail[sq] = torch.cat([before, xin[lo:hi].float()])[-(K - 1):].to(tail.dtype)
    return out.to(u.dtype)


def _linear_attention(q, k, v, decay, state, st, heads, dk, dv):
    T = q.shape[0]
    silu = torch.nn.functional.silu
    qf, kf, vf = silu(q.float()).view(T, heads, dk), silu(k.float()).view(T, heads, dk), silu(v.float()).view(T, heads, dv)
    out = torch.zeros(T, heads, dv)
    pos = st.token_positions.tolist()
    for sq, lo, hi in _segments(st):
        S = state[sq].clone() if pos[lo] > 0 else torch.zeros(heads, dk, dv)
        for t in range(lo, hi):
            S = decay[:, None, None] * S + kf[t][:, :, None] * vf[t][:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
        state[sq] = S
    return out.reshape(T, heads * dv)


def _gated_rmsnorm(x, weight, gate, eps, out, out_scale=1.0):
    y = _unit_rms(x, eps) * weight * out_scale
    if gate is not None:
        y = y * torch.sigmoid(gate.float())
    out.copy_(y.to(out.dtype))


class GlooFusedAllReduce:
    """CPU stand-in of swiftllm_b200.worker.tp_comm.FusedAllReduce with the SAME observable semantics as the CUDA kernels
    (csrc/allreduce_norm.cu), exchanged over gloo: partials are summed in rank order in fp32, residual <- h(h(sum) + residual),
    output = rmsnorm(residual) * weight.  two_shot: only the rows a rank owns (t % world == rank) are reduced / added /
    normalised by it; its other residual rows are POISONED with NaN (the kernel simply does not maintain them), and the
    normalised rows are gathered from their owners."""

    def __init__(self, max_tokens, hidden, dtype, device, group=None, two_shot=False, nvls=False, ll=False):
        import torch.distributed as dist
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.two_shot, self.nvls, self.hidden, self.max_tokens = bool(two_shot) or bool(nvls) or bool(ll), bool(nvls), hidden, max_tokens
        self.max_fused_tokens = max_tokens
        self.ll = bool(ll)        # the LL kernel has the two-shot kernel's observable semantics (row owners, sharded residual)
        self.data = torch.zeros((2, max_tokens, hidden), dtype=dtype)

    def partial_out(self, slot, num_tokens):
        return self.data[slot, :num_tokens]

    def reduce_add_norm(self, slot, num_tokens, residual, weight, eps):
        import torch.distributed as dist
        mine = self.data[slot, :num_tokens].contiguous()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        acc = torch.zeros(mine.shape, dtype=torch.float32)
        for prt in parts:                                  # fixed rank order, fp32 accumulation
            acc += prt.float()
        s = acc.to(mine.dtype) + residual                  # h(h(sum) + r)
        if not self.two_shot:
            residual.copy_(s)
            return K.rmsnorm(s, weight, eps)
        own = (torch.arange(num_tokens) % self.world) == self.rank
        residual[own] = s[own]
        residual[~own] = float("nan")
        out = torch.zeros_like(s)
        if bool(own.any()):
            out[own] = K.rmsnorm(residual[own], weight, eps)
        dist.all_reduce(out, group=self.group)             # every row has exactly one non-zero contributor: exact
        return out


def _swap_blocks_device(src_ids, dst_ids, is_swap_in, k_cache, v_cache, k_swap, v_swap):
    assert src_ids.dtype == torch.int64 and dst_ids.dtype == torch.int64
    K.swap_blocks_inplace(src_ids.tolist(), dst_ids.tolist(), is_swap_in, k_cache, v_cache, k_swap, v_swap)


_PATCHES = [
    ("swiftllm_b200.worker.layers.transformer_layer", "fused_add_rmsnorm_inplace", _fused_add_rmsnorm_inplace),
    ("swiftllm_b200.worker.layers.transformer_layer", "rotary_embedding_inplace", _rotary_embedding_inplace),
    ("swiftllm_b200.worker.layers.transformer_layer", "silu_and_mul_inplace", _silu_and_mul_inplace),
    ("swiftllm_b200.worker.layers.transformer_layer", "store_kvcache", _store_kvcache),
    ("swiftllm_b200.worker.layers.transformer_layer", "paged_attention", _paged_attention),
    ("swiftllm_b200.worker.layers.transformer_layer", "rotary_store_kvcache_decode", _rotary_store_kvcache_decode),
    ("swiftllm_b200.worker.layers.transformer_layer", "prefill_attention", _prefill_attention),
    ("swiftllm_b200.worker.layers.transformer_layer", "prefill_attention_paged", _prefill_attention_paged),
    ("swiftllm_b200.worker.layers.post_layer", "rmsnorm_inplace", _rmsnorm_inplace),
    ("swiftllm_b200.worker.block_manager", "_allocate_kernel", _allocate_blocks),
    ("swiftllm_b200.worker.block_manager", "unset_block_table_and_num_seq_alloc_blocks", _unset),
    ("swiftllm_b200.worker.block_manager", "gather_allocated_blocks_and_unset", _gather_and_unset),
    ("swiftllm_b200.swiftllm_c", "swap_blocks", _swap_blocks),
    ("swiftllm_b200.swiftllm_c", "swap_blocks_device", _swap_blocks_device),
    ("swiftllm_b200.worker.parallel_block_model", "add_rmsnorm_f32", _add_rmsnorm_f32),
    ("swiftllm_b200.worker.layers.window_attention", "window_kv_store", _window_kv_store),
    ("swiftllm_b200.worker.layers.window_attention", "window_attention", _window_attention),
    ("swiftllm_b200.worker.layers.feed_forward", "moe_route_grouped", _moe_route_grouped),
    ("swiftllm_b200.worker.layers.feed_forward", "moe_clamped_glu_scale", _moe_clamped_glu_scale),
    ("swiftllm_b200.worker.layers.latent_attention", "rmsnorm_strided", _rmsnorm_strided),
    ("swiftllm_b200.worker.layers.latent_attention", "latent_kv_store", _latent_kv_store),
    ("swiftllm_b200.worker.layers.latent_attention", "latent_attention", _latent_attention),
    ("swiftllm_b200.worker.layers.feed_forward", "relu2_inplace", _relu2_inplace),
    ("swiftllm_b200.worker.buzarax_model", "embed_pair_hash", _embed_pair_hash),
    ("swiftllm_b200.worker.buzarax_model", "tanh_cap_inplace", _tanh_cap_inplace),
    ("swiftllm_b200.worker.buzarax_model", "add_rmsnorm_f32", _add_rmsnorm_f32),
    ("swiftllm_b200.worker.layers.sequential_block", "postnorm_add_mix", _postnorm_add_mix),
    ("swiftllm_b200.worker.layers.feed_forward", "moe_route_sigmoid", _moe_route_sigmoid),
    ("swiftllm_b200.worker.layers.feed_forward", "moe_silu_glu_scale", _moe_silu_glu_scale),
    ("swiftllm_b200.worker.layers.gated_recurrence", "causal_conv", _causal_conv),
    ("swiftllm_b200.worker.layers.gated_recurrence", "rglru_scan", _rglru_scan),
    ("swiftllm_b200.worker.layers.linear_attention", "linear_attention", _linear_attention),
    ("swiftllm_b200.worker.layers.linear_attention", "gated_rmsnorm", _gated_rmsnorm),
    ("swiftllm_b200.worker.layers.window_attention", "diff_combine", _diff_combine),
    ("swiftllm_b200.worker.naforax_model", "embed_pair_hash", _embed_pair_hash),
    ("swiftllm_b200.worker.naforax_model", "tanh_cap_inplace", _tanh_cap_inplace),
    ("swiftllm_b200.worker.naforax_model", "group_norm_add_norm", _group_norm_add_norm),
    ("swiftllm_b200.worker.naforax_model", "group_norm_cast", _group_norm_cast),
    ("swiftllm_b200.worker.naforax_model", "stream_add", _stream_add),
    ("swiftllm_b200.worker.layers.sandwich_block", "group_norm_add_norm", _group_norm_add_norm),
    ("swiftllm_b200.worker.layers.sandwich_block", "short_conv", _short_conv),
    ("swiftllm_b200.worker.layers.selective_scan", "short_conv", _short_conv),
    ("swiftllm_b200.worker.layers.selective_scan", "selective_scan", _selective_scan),
    ("swiftllm_b200.worker.layers.selective_scan", "linear_f32_out", _linear_f32_out),
    ("swiftllm_b200.worker.layers.min_gru", "mingru_scan", _mingru_scan),
    ("swiftllm_b200.worker.layers.feed_forward", "gelu_glu", _gelu_glu),
    ("swiftllm_b200.worker.layers.feed_forward", "moe_route_softmax", _moe_route_softmax),
    ("swiftllm_b200.worker.layers.feed_forward", "moe_route", _moe_route),
    ("swiftllm_b200.worker.layers.feed_forward", "moe_relu2_scale_inplace", _moe_relu2_scale_inplace),
]


@contextlib.contextmanager
def product_on_cpu(extra_patches=()):
    """Inside this context `swiftllm_b200.LlamaModel` runs on CPU tensors with oracle-backed kernels."""
    from oracle.ref_shim import cuda_as_cpu        # fake CUDA streams / events (shared with the reference's CPU shim)
    saved = []
    cur_dev = torch.cuda.current_device
    torch.cuda.current_device = lambda: 0
    try:
        for mod_name, attr, fn in list(_PATCHES) + list(extra_patches):
            mod = importlib.import_module(mod_name)
            saved.append((mod, attr, getattr(mod, attr)))
            setattr(mod, attr, fn)
        with cuda_as_cpu(), _CudaToCpu():
            yield
    finally:
        for mod, attr, old in saved:
            setattr(mod, attr, old)
        torch.cuda.current_device = cur_dev

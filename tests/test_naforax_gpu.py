"""GPU: the Naforax worker and its CUDA kernels (csrc/sandwich_ops.cu, csrc/scan_ops.cu, the chunk / pre-norm / shared-value /
fp32-output options of csrc/window_attn.cu and its two-map combine) - every kernel alone against a plain loop written here or in
oracle/naforax.py, then the scenarios of tests/bupozen_cases.py and tests/naforax_cases.py through the worker (fp32 tight, bf16
loose)."""
import math
import types

import pytest
import torch

import bupozen_cases as B
import naforax_cases as C
from oracle import naforax as O
from test_bupozen_gpu import _make
from test_buzarax_gpu import _schedule, _step

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return 1e-5 if dtype == torch.float32 else 1.2e-2


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,groups", [(48, 3), (64, 1), (1000, 2), (4096, 2), (96, 96)])
def test_group_norms_add_and_next_norm(dtype, width, groups):
    from swiftllm_b200.worker.kernels.sandwich_ops import group_norm_add_norm, group_norm_cast, stream_add
    g = torch.Generator().manual_seed(width)
    T = 37
    x, y = torch.randn(T, width, generator=g) * 3, torch.randn(T, width, generator=g).to(dtype)
    wb, wn = torch.randn(width, generator=g), torch.randn(width, generator=g)
    ref_x = x + 0.7 * O.group_norm(y.float(), wb, groups, 1e-5)
    ref_n = O.group_norm(ref_x, wn, groups, 1e-5)
    xd = x.to(DEV)
    n = group_norm_add_norm(xd, y.to(DEV), wb.to(DEV), 0.7, wn.to(DEV), 1e-5, groups)
    assert B.rel_err(xd, ref_x) < 1e-6 and B.rel_err(n, ref_n) < 1e-5
    # each half alone
    xd = x.to(DEV)
    assert group_norm_add_norm(xd, y.to(DEV), wb.to(DEV), 0.7, None, 1e-5, groups) is None and B.rel_err(xd, ref_x) < 1e-6
    xd = x.to(DEV)
    assert B.rel_err(group_norm_add_norm(xd, None, None, 1.0, wn.to(DEV), 1e-5, groups), O.group_norm(x, wn, groups, 1e-5)) < 1e-5
    assert torch.equal(xd.cpu(), x)
    out = group_norm_cast(x.to(DEV), wn.to(DEV), 1e-5, groups, dtype)
    assert out.dtype == dtype and B.rel_err(out.float(), O.group_norm(x, wn, groups, 1e-5)) < _tol(dtype)
    a, v = torch.randn(T, width, generator=g), torch.randn(width, generator=g)
    xd = x.to(DEV)
    stream_add(xd, a.to(DEV), v.to(DEV))
    assert B.rel_err(xd, x + a + v) < 1e-6
    stream_add(xd, None, v.to(DEV))
    assert B.rel_err(xd, x + a + 2 * v) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_gated_unit(dtype):
    from swiftllm_b200.worker.kernels.sandwich_ops import gelu_glu
    u = (torch.randn(19, 2 * 70, generator=torch.Generator().manual_seed(1)) * 2).to(dtype)
    ref = O.gelu_tanh(u[:, :70].float()) * u[:, 70:].float()
    assert B.rel_err(gelu_glu(u.to(DEV)).float(), ref) < _tol(dtype)


@pytest.mark.parametrize("experts,top,gated", [(6, 2, True), (3, 1, False), (33, 4, True), (16, 3, False), (200, 32, True), (5, 5, True)])
def test_softmax_routing_keeps_plain_scores(experts, top, gated):
    from swiftllm_b200.worker.kernels.sandwich_ops import moe_route_softmax
    g = torch.Generator().manual_seed(experts)
    logits = torch.randn(41, experts + (1 if gated else 0), generator=g) * 2
    logits[:, 1 % experts] = logits[:, 0]                         # ties: the lower index wins
    w = moe_route_softmax(logits.to(DEV), experts, top, gated).cpu()
    s = torch.softmax(logits[:, :experts], dim=-1)
    idx = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    ref = torch.zeros_like(s).scatter_(1, idx, s.gather(1, idx))
    assert torch.equal(w[:, :experts] != 0, ref != 0) and B.rel_err(w[:, :experts], ref) < 1e-6
    if gated:
        assert B.rel_err(w[:, experts], torch.sigmoid(logits[:, experts])) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_clamped_experts_with_a_gated_shared_expert(dtype):
    from swiftllm_b200.worker.kernels.parallel_block import moe_clamped_glu_scale
    g = torch.Generator().manual_seed(2)
    T, E, ff, sff = 13, 5, 6, 9
    u = (torch.randn(T, 2 * (E * ff + sff), generator=g) * 2).to(dtype)
    w = torch.rand(T, E + 1, generator=g)
    w[:, 2] = 0.0

    def act(gate, up, lim):
        gate, up = gate.clamp(max=lim), up.clamp(-lim, lim)
        return gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    uf = u.float()
    parts = [act(uf[:, 2 * e * ff:2 * e * ff + ff], uf[:, 2 * e * ff + ff:2 * (e + 1) * ff], 0.75) * w[:, e:e + 1] for e in range(E)]
    parts.append(act(uf[:, 2 * E * ff:2 * E * ff + sff], uf[:, 2 * E * ff + sff:], 1.5) * w[:, E:])
    y = moe_clamped_glu_scale(u.to(DEV), w.to(DEV), E, ff, 0.75, sff, 1.5, 1.702, shared_gated=True)
    assert B.rel_err(y.float(), torch.cat(parts, dim=1)) < _tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C_,K,silu,add,f32_in", [(24, 4, False, True, True), (33, 1, False, True, True), (20, 2, True, False, False),
                                                   (192, 3, True, False, False), (130, 8, False, True, True)])
@pytest.mark.parametrize("fused", [False, True])
def test_short_convolution_with_carried_tail(dtype, C_, K, silu, add, f32_in, fused):
    """Two sequences in rows 2 and 0 of the tail tensor (which starts full of junk), fed in portions down to one token.
    `fused`: the convolution moves the tails on itself (decoded rows inside its kernel), else a separate call does."""
    from swiftllm_b200.worker.kernels.scan_ops import conv_tail_update, short_conv
    g = torch.Generator().manual_seed(C_ + K)
    lens, rows = [150, 37], [2, 0]
    plan = [[(0, 1), (1, 2)], [(0, 2), (1, 1)], [(0, 97), (1, 1)], [(1, 33)], [(0, 49)], [(0, 1)]]
    tin = torch.float32 if f32_in else dtype
    xin = [torch.randn(n, C_, generator=g).to(tin) for n in lens]
    w, bias = torch.randn(C_, K, generator=g), (torch.randn(C_, generator=g) if silu else None)
    ref = []
    for s in range(2):
        u = O.causal_conv(xin[s].float(), w, bias)
        if silu:
            u = O.silu(u)
        ref.append(u + xin[s].float() if add else u)
    tail = torch.full((3, K - 1, C_), 1e4, dtype=tin, device=DEV)
    got = [[] for _ in lens]
    for segs in _schedule(lens, plan):
        order = sorted(segs, key=lambda e: e[2] == 1)                  # prompt portions first
        st = _step([(rows[s], p0, n) for s, p0, n in order])
        st.num_prefill_tokens = sum(n for _, _, n in order if n > 1)
        st.num_prefill_seqs = sum(1 for _, _, n in order if n > 1)
        x = torch.cat([xin[s][p0:p0 + n] for s, p0, n in order]).to(DEV)
        out = short_conv(x, w.to(DEV), None if bias is None else bias.to(DEV), tail if K > 1 else None, st, dtype, add_input=add,
                         silu=silu, move_tail=fused).float().cpu()
        if K > 1 and not fused:
            conv_tail_update(x, tail, st)
        o = 0
        for s, p0, n in order:
            got[s].append((p0, out[o:o + n])); o += n
    for s in range(2):
        full = torch.cat([c for _, c in sorted(got[s], key=lambda e: e[0])])
        assert B.rel_err(full, ref[s]) < _tol(dtype), s


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tiled", [True, False])
@pytest.mark.parametrize("C_", [20, 33, 288, 130])
def test_mingru_state_through_portions(dtype, C_, tiled):
    """`tiled`: every segment through the kernel that is parallel over time (tiles of 64 tokens), or through the plain one."""
    from swiftllm_b200.worker.kernels.scan_ops import mingru_scan
    g = torch.Generator().manual_seed(C_)
    lens, rows = [150, 37], [2, 0]
    plan = [[(0, 1), (1, 2)], [(0, 2), (1, 1)], [(0, 97), (1, 1)], [(1, 33)], [(0, 49)], [(0, 1)]]
    proj = [(torch.randn(n, 3 * C_, generator=g) * 1.5).to(dtype) for n in lens]
    ref = []
    for s in range(2):
        p = proj[s].float()
        z, u, gl = torch.sigmoid(p[:, :C_]), p[:, C_:2 * C_], p[:, 2 * C_:]
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        S, out = torch.zeros(C_), []
        for t in range(lens[s]):
            S = (1 - z[t]) * S + z[t] * cand[t]
            out.append(S * O.silu(gl[t]))
        ref.append(torch.stack(out))
    state = torch.full((3, C_), 1e4, device=DEV)
    got = [[] for _ in lens]
    for segs in _schedule(lens, plan):
        st = _step([(rows[s], p0, n) for s, p0, n in segs])
        st.num_prefill_seqs = len(segs) if tiled else 0
        x = torch.cat([proj[s][p0:p0 + n] for s, p0, n in segs]).to(DEV)
        out = mingru_scan(x, state, st, C_).float().cpu()
        o = 0
        for s, p0, n in segs:
            got[s].append(out[o:o + n]); o += n
    for s in range(2):
        assert B.rel_err(torch.cat(got[s]), ref[s]) < _tol(dtype), s


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tiled", [True, False])
@pytest.mark.parametrize("C_,N,dt_f32", [(18, 5, True), (7, 40, True), (256, 16, False), (11, 1, True), (40, 200, False), (130, 32, True)])
def test_selective_scan_state_through_portions(dtype, C_, N, dt_f32, tiled):
    """`tiled`: every segment through the kernel that stages tiles of tokens in shared memory, or through the plain one."""
    from swiftllm_b200.worker.kernels.scan_ops import selective_scan
    g = torch.Generator().manual_seed(C_ + N)
    lens, rows = [90, 37], [2, 0]
    plan = [[(0, 1), (1, 2)], [(0, 2), (1, 1)], [(0, 57), (1, 1)], [(1, 33)], [(0, 29)], [(0, 1)]]
    R = 3
    x = [torch.randn(n, C_, generator=g).to(dtype) for n in lens]
    z = [torch.randn(n, C_, generator=g).to(dtype) for n in lens]
    dt = [(torch.randn(n, C_, generator=g) - 1.0).to(torch.float32 if dt_f32 else dtype) for n in lens]
    bc = [torch.randn(n, R + 2 * N, generator=g).to(dtype) for n in lens]
    A = -torch.exp(torch.randn(C_, N, generator=g) * 0.5)
    D, bias = torch.randn(C_, generator=g), torch.randn(C_, generator=g) * 0.3
    ref = []
    for s in range(2):
        step = O.softplus(dt[s].float() + bias)
        S, out = torch.zeros(C_, N, dtype=torch.float64), []
        for t in range(lens[s]):
            xt = x[s][t].double()
            S = torch.exp(step[t].double()[:, None] * A.double()) * S + (step[t].double() * xt)[:, None] * bc[s][t, R:R + N].double()[None]
            y = (S * bc[s][t, R + N:].double()[None]).sum(1) + D.double() * xt
            out.append((y * O.silu(z[s][t].double())).float())
        ref.append(torch.stack(out))
    state = torch.full((3, C_, N), 1e4, device=DEV)
    got = [[] for _ in lens]
    for segs in _schedule(lens, plan):
        st = _step([(rows[s], p0, n) for s, p0, n in segs])
        st.num_prefill_seqs = len(segs) if tiled else 0
        cat = lambda parts: torch.cat([parts[s][p0:p0 + n] for s, p0, n in segs]).to(DEV)
        out = selective_scan(cat(x), cat(dt), bias.to(DEV), A.to(DEV), cat(bc), R, R + N, D.to(DEV), cat(z), state, st).float().cpu()
        o = 0
        for s, p0, n in segs:
            got[s].append(out[o:o + n]); o += n
    for s in range(2):
        assert B.rel_err(torch.cat(got[s]), ref[s]) < (2e-5 if dtype == torch.float32 else 1.2e-2), s


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dv", [(6, 2, 6), (4, 4, 112), (5, 1, 200), (3, 3, 33)])
def test_two_maps_into_one_gated_head(dtype, H, G, dv):
    from swiftllm_b200.worker.kernels.window_attn import diff_combine
    g = torch.Generator().manual_seed(H + dv)
    T, hq = 21, H // G
    a = torch.randn(T, G, 2, hq, dv, generator=g)
    gate = torch.randn(T, H * dv + 8, generator=g).to(dtype)
    o = a[:, :, 0] - 1.7 * a[:, :, 1]
    ref = (O.unit_rms(o, 1e-5) * 0.65).reshape(T, H * dv) * torch.sigmoid(gate[:, 8:].float())
    out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
    diff_combine(a.reshape(T, -1).to(DEV), gate.to(DEV)[:, 8:], out, H, G, dv, 1.7, 1e-5, 0.65)
    assert B.rel_err(out.float(), ref) < _tol(dtype)


@pytest.mark.parametrize("H,G,dk,dv,dims,chunk", [(4, 2, 32, 16, 32, 64), (3, 1, 64, 64, 16, 50), (6, 3, 48, 80, 24, 72),
                                                  (4, 4, 16, 128, 0, 37), (2, 2, 128, 32, 64, 300)])
def test_chunked_two_map_attention_tensor_core_and_cuda_core_agree(H, G, dk, dv, dims, chunk):
    """Norm with weight before interleaved rotary, chunked mask, two key heads per value head, fp32 output: the same mixed step
    (prompt portions that start inside a sequence and cross chunk edges, decoded tokens) through the cache store and both
    attention kernels, and against a plain loop for a few rows."""
    from swiftllm_b200.worker.kernels import window_attn as WA
    g = torch.Generator().manual_seed(H + dk)
    bs, lens = 16, [300, 77, 1, 200, 130]
    new = [150, 40, 1, 1, 1]
    nb = sum((n + bs - 1) // bs for n in lens)
    perm = torch.randperm(nb, generator=g).tolist()
    table = torch.full((5, 32), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for b in range((n + bs - 1) // bs):
            table[s, b] = perm.pop()
    table = table.to(DEV)
    qn, kn = (1 + 0.3 * torch.randn(dk, generator=g)).to(DEV), (1 + 0.3 * torch.randn(dk, generator=g)).to(DEV)
    opt = WA.AttnOptions(q_norm=qn, k_norm=kn, prenorm_eps=1e-5, chunk=chunk, vshare=2, out_f32=True)
    H2, G2 = 2 * H, 2 * G

    def angles(pos, n, base=100.0):
        a = torch.tensor(pos, dtype=torch.float64)[:, None] * torch.tensor([base ** (-2.0 * i / n) for i in range(n // 2)],
                                                                           dtype=torch.float64)[None]
        return torch.cos(a).float().to(DEV), torch.sin(a).float().to(DEV)
    cache = torch.zeros(nb, 1, bs, G2 * dk + G * dv, dtype=torch.bfloat16, device=DEV)
    all_seq = [s for s, n in enumerate(lens) for _ in range(n)]
    all_pos = [p for n in lens for p in range(n)]
    st_all = types.SimpleNamespace(token_seq_ids=torch.tensor(all_seq, dtype=torch.int32, device=DEV),
                                   token_positions=torch.tensor(all_pos, dtype=torch.int32, device=DEV))
    k = torch.randn(len(all_seq), G2 * dk, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(len(all_seq), G * dv, generator=g).to(torch.bfloat16).to(DEV)
    cs, sn = angles(all_pos, dims) if dims else (None, None)
    WA.window_kv_store(k, v, cache, 0, table, st_all, G2, dk, dv, dims, cs, sn, opt)
    tok_seq = [s for s, n in enumerate(new) for _ in range(n)]
    tok_pos = [lens[s] - n + p for s, n in enumerate(new) for p in range(n)]
    T = len(tok_seq)
    q = torch.randn(T, H2 * dk, generator=g).to(torch.bfloat16).to(DEV)
    cs, sn = angles(tok_pos, dims) if dims else (None, None)
    st = types.SimpleNamespace(token_seq_ids=torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
                               token_positions=torch.tensor(tok_pos, dtype=torch.int32, device=DEV), num_prefill_tokens=191)
    scale = 3.0 / math.sqrt(dk)
    outs = []
    for simt in (True, False):
        old = WA.set_simt(simt)
        try:
            out = torch.zeros(T, H2 * dv, dtype=torch.float32, device=DEV)
            WA.window_attention(q, None, cache, 0, table, st, out, H2, G2, dk, dv, dims, 0, scale, False, cs, sn, opt)
            outs.append(out.cpu())
        finally:
            WA.set_simt(old)
    assert B.rel_err(outs[1], outs[0]) < 1.5e-2
    row_err = (outs[1] - outs[0]).pow(2).mean(-1).sqrt() / outs[0].pow(2).mean(-1).sqrt()
    assert float(row_err.max()) < 5e-2
    # a plain loop on the rounded inputs, for rows at a chunk's first and last position and in its middle
    kf, vf, qf = k.float().cpu().view(-1, G2, dk), v.float().cpu().view(-1, G, dv), q.float().cpu().view(T, H2, dk)
    kf = O.unit_rms(kf, 1e-5) * kn.cpu()
    qf = O.unit_rms(qf, 1e-5) * qn.cpu()
    first = [0]
    for n in lens:
        first.append(first[-1] + n)
    picked = [r for r in range(T) if tok_pos[r] % chunk in (0, 1, chunk - 1) or r in (0, T - 1)][:12]
    for r in picked:
        s, p = tok_seq[r], tok_pos[r]
        lo = p // chunk * chunk
        keys = O.rotate_pairs(kf[first[s] + lo:first[s] + p + 1], list(range(lo, p + 1)), 100.0, dims).to(torch.bfloat16).float()
        qr = O.rotate_pairs(qf[r:r + 1], [p], 100.0, dims)[0]
        vals = vf[first[s] + lo:first[s] + p + 1]
        for h2 in range(H2):
            g2 = h2 // (H2 // G2)
            w = torch.softmax((keys[:, g2] @ qr[h2]) * scale, dim=0)
            ref = w @ vals[:, g2 // 2]
            assert B.rel_err(outs[0][r].view(H2, dv)[h2], ref) < 2e-2, (r, h2)


# ---------------------------------------------------------------- the worker
@pytest.mark.parametrize("name", sorted(C.SINGLE))
def test_single_mechanisms(name):
    B.case_whole_prompt(_make, C.SINGLE[name], n=17)


def test_whole_prompt():
    B.case_whole_prompt(_make, C.full_config())


def test_prefill_vs_decode():
    B.case_prefill_vs_decode(_make, C.full_config())


def test_portions():
    B.case_portions(_make, C.full_config())


def test_mixed_batch():
    B.case_mixed_batch(_make, C.full_config())


def test_blocks_and_rows_reused():
    B.case_blocks_and_rows_reused(_make, C.full_config())


def test_state_rows_used_again():
    C.case_state_rows_used_again(_make)


def test_long_decode():
    B.case_long_decode(_make, C.full_config())


def test_greedy_generation():
    B.case_greedy_generation(_make, C.config([(C.mingru(), C.moe()), (C.attn(), C.dense()), (C.mamba(), None)], loop=(0, 2, 2)))


def test_far_key():
    C.case_far_key(_make)


def test_chunk_edges():
    C.case_chunk_edges(_make)


def test_first_tokens_and_block_borders():
    C.case_first_tokens_and_block_borders(_make)


def test_lambda_and_head_norm():
    C.case_lambda_and_head_norm(_make)


def test_slow_recurrences_remember():
    C.case_slow_recurrences_remember(_make)


def test_convolutions_across_short_portions():
    C.case_convolutions_across_short_portions(_make)


def test_router_scores_are_not_renormalised():
    C.case_router_scores_are_not_renormalised(_make)


def test_passes_keep_their_own_state():
    C.case_passes_keep_their_own_state(_make)


def _tc_config():
    """Head sizes that are multiples of 16 (the shapes the 16-bit tensor-core attention takes), sequences over several key tiles
    and chunks."""
    return C.config([(C.attn(heads=8, kv_heads=2, dim=32, vdim=16, dims=32, chunk=40), C.moe()),
                     (C.mingru(width=64), C.dense()),
                     (C.attn(heads=6, kv_heads=1, dim=64, vdim=64, dims=16, chunk=64), None),
                     (C.mamba(inner=96, state=16, dt_rank=4), C.moe(experts=5, top=1)),
                     (C.attn(heads=4, kv_heads=4, dim=16, vdim=48, dims=0, chunk=33), C.dense())], width=64, groups=2, loop=(1, 3, 2))


def test_bfloat16_worker_close_to_fp32_oracle():
    """bf16 projections / cache, fp32 residual, norms, attention weights and states: the logits stay within bf16 rounding of the
    fp32 oracle on the same weights, and do not depend on how the prompt was cut beyond that."""
    for cfg, n, cuts, bs, nb in ((C.full_config(), 33, [5, 2, 1, 1, 24], 4, 40), (_tc_config(), 150, [61, 4, 64, 2, 1, 1, 17], 8, 60)):
        t = O.random_tensors(cfg, seed=11)
        toks = B.tokens_for(cfg, n, 11)
        ref = O.forward(cfg, t, toks)[-40:]
        m = B.make_worker(_make, cfg, t, dtype="bfloat16", block_size=bs, num_blocks=nb)
        whole = B.run_portions(m, toks, 0, [n])[-40:]
        cut = B.run_portions(m, toks, 1, cuts)[-40:]
        assert B.rel_err(whole, ref) < 4e-2 and B.rel_err(cut, ref) < 4e-2 and B.rel_err(cut, whole) < 3e-2


def test_cuda_graph_decode_matches_eager():
    """Pure-decode steps replayed from a CUDA graph: the per-sequence state rows (recurrences, scans, every convolution's tail)
    move on inside the graph exactly as in eager steps."""
    cfg = C.config([(C.mingru(), C.moe()), (C.attn(), C.dense()), (C.mamba(), None)], width=64, groups=2, loop=(0, 2, 2))
    t = O.random_tensors(cfg, seed=13)
    t["head"] = (t["head"].float() * 4).to(t["head"].dtype)
    prompts = [B.tokens_for(cfg, n, 70 + k) for k, n in enumerate((7, 3, 12))]
    runs = []
    for graph in (False, True):
        m = B.make_worker(_make, cfg, t, dtype="float32", block_size=4, num_blocks=40)
        m.engine_config.use_cuda_graph = graph
        last = m.forward(prompts, [0, 1, 2], [])
        lens, toks = [len(p) for p in prompts], [list(last)]
        for step in range(9):
            live = [0, 1, 2] if step < 6 else [0, 2]
            for i in live:
                lens[i] += 1
            out = m.forward([[toks[-1][i]] for i in live], live, [lens[i] for i in live])
            nxt = list(toks[-1])
            for i, o in zip(live, out):
                nxt[i] = o
            toks.append(nxt)
        assert m.gpu_block_manager.check_device_status() >= 0
        runs.append(toks)
    assert runs[0] == runs[1]
    want = B.oracle_greedy(cfg, t, prompts[0], 10)
    assert [s[0] for s in runs[0]] == want


def test_memory_profile_then_generation():
    """The entry point's order of calls: the forged profiling batch (no cache, no state tensors yet) sizes the pool, then the
    worker generates through the scheduler loop as the oracle does."""
    from swiftllm_b200.worker.chunking import run_greedy
    cfg = C.config([(C.attn(), C.moe()), (C.mingru(), None), (C.mamba(), C.dense())], loop=(1, 3, 2))
    t = O.random_tensors(cfg, seed=19)
    t["head"] = (t["head"].float() * 4).to(t["head"].dtype)
    import swiftllm_b200
    from swiftllm_b200.worker.weight import dict_getter
    ec = swiftllm_b200.EngineConfig(model_path="", use_dummy=False, block_size=4, gpu_mem_utilization=0.5, num_cpu_blocks=0,
                                    max_seqs_in_block_table=4, max_blocks_per_seq=16, max_batch_size=4, max_tokens_in_batch=64,
                                    dtype="float32")
    m = swiftllm_b200.create_model(ec, swiftllm_b200.registry.model_config_from_dict(cfg))
    m.load_weights(dict_getter(t))
    n = m.profile_num_blocks()
    assert n == 4 * 16                                    # capped by the block table
    m.init_kvcache_and_swap(n)
    prompts = [B.tokens_for(cfg, k, 80 + k) for k in (9, 2, 14)]
    got = run_greedy(m, prompts, new_tokens=4, max_tokens_in_step=10, max_chunk=5, seq_ids=[1, 3, 0])
    assert got == [B.oracle_greedy(cfg, t, p, 4) for p in prompts]


def test_trace_replay_command_line(tmp_path):
    """bin/trace_run on a checkpoint folder of this design: a mixed schedule (portions beside decoded tokens, requests that end
    and whose rows, blocks and state rows are used again) in both dtypes, against the oracle run on each whole sequence."""
    import json
    import os
    import subprocess
    import numpy as np
    from safetensors.torch import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = C.config([
        (C.attn(heads=10, kv_heads=2, dim=16, vdim=24, base=5000.0, dims=16, chunk=24), C.moe(experts=9, top=3, ff=24)),
        (C.mingru(width=40), C.dense(ff=50)),
        (C.attn(heads=3, kv_heads=3, dim=8, vdim=8, base=300.0, dims=6, chunk=9), None),
        (C.mamba(inner=72, state=8, dt_rank=5, conv=4), C.moe()),
    ], width=72, vocab=131, eps=1e-6, groups=4, loop=(1, 4, 2))
    t = O.random_tensors(cfg, seed=21)
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in t.items()}, str(model_dir / "model.safetensors"))
    reqs = {k: B.tokens_for(cfg, n, s) for s, (k, n) in enumerate((("a", 70), ("b", 41), ("c", 17), ("d", 5), ("e", 30)))}
    ref = {k: O.forward(cfg, t, v).numpy() for k, v in reqs.items()}
    plan = [[("a", 33), ("b", 2)], [("a", 31), ("b", 30), ("c", 17)], [("a", 1), ("b", 1), ("d", 5)], [("a", 1), ("b", 1), ("e", 3)],
            [("a", 2), ("b", 7), ("e", 27)], [("a", 2)]]
    for dtype, limit in (("float32", 1e-4), ("bfloat16", 4e-2)):
        out = tmp_path / dtype
        out.mkdir()
        at, lines, rows = {k: 0 for k in reqs}, [], []
        for n, step in enumerate(plan):
            entries, end, rr = [], [], []
            for k, c in step:
                lo, hi = at[k], at[k] + c
                entries.append({"id": k, "tokens": reqs[k][lo:hi], "want": list(range(0, c, 2))})
                rr += [(k, p) for p in range(lo, hi, 2)]
                at[k] = hi
                if hi == len(reqs[k]):
                    end.append(k)
            lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
            rows.append(rr)
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True, cwd=root)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
        errs = []
        for n, rr in enumerate(rows):
            got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rr), -1)
            for j, (k, pos) in enumerate(rr):
                errs.append(np.sqrt(((got[j] - ref[k][pos]) ** 2).mean() / (ref[k][pos] ** 2).mean()))
                assert errs[-1] < 2.5 * limit, (dtype, n, k, pos, errs[-1])         # no single position far off ...
        assert np.sqrt(np.mean(np.square(errs))) < limit, dtype                     # ... and all of them within rounding

"""GPU: the Buzarax worker and its CUDA kernels (csrc/recurrent.cu, csrc/stream_ops.cu, the options of csrc/window_attn.cu)
- every kernel alone against a plain loop written here or in oracle/buzarax.py, then the scenarios of tests/bupozen_cases.py and
tests/buzarax_cases.py through the worker (fp32 tight, bf16 loose)."""
import math
import types

import pytest
import torch

import bupozen_cases as B
import buzarax_cases as C
from oracle import buzarax as O
from test_bupozen_gpu import _make, tol

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _step(segments):
    """segments: (sequence row, first position, tokens) in batch order -> the step's metadata as the kernels read it."""
    tok_seq = [s for s, _, n in segments for _ in range(n)]
    tok_pos = [p0 + i for _, p0, n in segments for i in range(n)]
    starts = [0]
    for _, _, n in segments:
        starts.append(starts[-1] + n)
    i32 = dict(dtype=torch.int32, device=DEV)
    return types.SimpleNamespace(token_seq_ids=torch.tensor(tok_seq, **i32), token_positions=torch.tensor(tok_pos, **i32),
                                 seg_starts=torch.tensor(starts, **i32), seq_ids=torch.tensor([s for s, _, _ in segments], **i32),
                                 batch_size=len(segments), num_tokens=len(tok_seq))


def _schedule(lens, plan):
    """plan: steps of (sequence, tokens) -> per step the segments (row, first position, tokens) and the slices of each sequence."""
    at = [0] * len(lens)
    for step in plan:
        segs = []
        for s, n in step:
            segs.append((s, at[s], n))
            at[s] += n
        yield segs
    assert at == list(lens)


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C_,blocks,K", [(24, 3, 4), (33, 11, 1), (20, 1, 2), (192, 6, 3), (130, 2, 8)])
def test_convolution_and_gated_recurrence(dtype, C_, blocks, K):
    """Two sequences in rows 2 and 0 of the state tensors (which start full of junk), fed in portions down to one token, some of
    them long enough for the tiled scan; against the plain loops on each whole sequence."""
    from swiftllm_b200.worker.kernels.recurrent import causal_conv, rglru_scan
    g = torch.Generator().manual_seed(C_ + K)
    lens, rows = [150, 37], [2, 0]
    plan = [[(0, 1), (1, 2)], [(0, 2), (1, 1)], [(0, 97), (1, 1)], [(1, 33)], [(0, 49)], [(0, 1)]]
    cb = C_ // blocks
    xin = [torch.randn(n, C_, generator=g).to(dtype) for n in lens]
    ybr = [torch.randn(n, C_, generator=g).to(dtype) for n in lens]
    w = torch.randn(C_, K, generator=g).to(dtype)
    bias = torch.randn(C_, generator=g).to(dtype)
    gw = (torch.randn(blocks, cb, 2 * cb, generator=g) / math.sqrt(cb)).to(dtype)
    gb = torch.randn(blocks, 1, 2 * cb, generator=g).to(dtype)
    rate = -8.0 * torch.nn.functional.softplus(torch.randn(C_, generator=g) - 2.0)
    # reference, fp32 on the rounded inputs
    ref = []
    for s in range(2):
        u = O.causal_conv(xin[s].float(), w.float(), bias.float())
        if dtype != torch.float32:
            u = u.to(dtype).float()                          # the kernel hands u on in the storage type
        gl = torch.baddbmm(gb.float(), u.view(-1, blocks, cb).transpose(0, 1), gw.float())
        if dtype != torch.float32:
            gl = gl.to(dtype).float()
        r = torch.sigmoid(gl[:, :, :cb]).transpose(0, 1).reshape(-1, C_)
        i = torch.sigmoid(gl[:, :, cb:]).transpose(0, 1).reshape(-1, C_)
        a = torch.exp(rate * r)
        S, out = torch.zeros(C_), []
        for t in range(lens[s]):
            S = a[t] * S + torch.sqrt(1 - a[t] * a[t]) * (i[t] * u[t])
            out.append(S * O.gelu_tanh(ybr[s][t].float()))
        ref.append(torch.stack(out))
    state = torch.full((3, C_), 1e4, device=DEV)
    tail = torch.full((3, K - 1, C_), 77.0, dtype=dtype, device=DEV)
    got = [[], []]
    for segs in _schedule(lens, plan):
        st = _step([(rows[s], p0, n) for s, p0, n in segs])
        x = torch.cat([xin[s][p0:p0 + n] for s, p0, n in segs]).to(DEV)
        y = torch.cat([ybr[s][p0:p0 + n] for s, p0, n in segs]).to(DEV)
        wide = torch.cat([y, x], dim=1)                       # the kernels take column slices of the fused projection
        yv, xv = wide[:, :C_], wide[:, C_:]
        u = causal_conv(xv, w.to(DEV), bias.to(DEV), tail, st)
        gates = torch.baddbmm(gb.to(DEV), u.view(-1, blocks, cb).transpose(0, 1), gw.to(DEV))
        out = rglru_scan(u, gates, yv, rate.to(DEV), xv, state, tail, st).float().cpu()
        at = 0
        for s, p0, n in segs:
            got[s].append(out[at:at + n]); at += n
    for s in range(2):
        assert B.rel_err(torch.cat(got[s]), ref[s]) < (1e-5 if dtype == torch.float32 else 2e-2), s
    assert float(state[1].min()) == 1e4                       # the row nobody owns is untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv", [(3, 5, 7), (1, 9, 4), (2, 40, 36), (4, 12, 3), (5, 48, 80), (2, 128, 128), (1, 16, 200), (2, 24, 64)])
def test_linear_attention_state_through_portions(dtype, H, dk, dv):
    from swiftllm_b200.worker.kernels.recurrent import linear_attention
    g = torch.Generator().manual_seed(H * dk + dv)
    lens, rows = [90, 21], [1, 2]
    plan = [[(0, 2), (1, 1)], [(0, 1), (1, 1)], [(0, 70), (1, 19)], [(0, 16)], [(0, 1)]]
    q = [(torch.randn(n, H * dk, generator=g)).to(dtype) for n in lens]
    k = [(torch.randn(n, H * dk, generator=g)).to(dtype) for n in lens]
    v = [(torch.randn(n, H * dv, generator=g)).to(dtype) for n in lens]
    decay = torch.tensor([0.5 + 0.4999 * (h + 1) / H for h in range(H)])
    ref = []
    for s in range(2):
        qq, kk, vv = O.silu(q[s].float()).view(-1, H, dk), O.silu(k[s].float()).view(-1, H, dk), O.silu(v[s].float()).view(-1, H, dv)
        out = torch.zeros(lens[s], H, dv)
        for h in range(H):
            S = torch.zeros(dk, dv)
            for t in range(lens[s]):
                S = decay[h] * S + torch.outer(kk[t, h], vv[t, h])
                out[t, h] = S.T @ qq[t, h]
        ref.append(out.view(-1, H * dv))
    state = torch.full((3, H, dk, dv), -300.0, device=DEV)
    got = [[], []]
    for segs in _schedule(lens, plan):
        st = _step([(rows[s], p0, n) for s, p0, n in segs])
        wide = torch.cat([torch.cat([a[s][p0:p0 + n] for s, p0, n in segs]) for a in (q, k, v)], dim=1).to(DEV)
        out = linear_attention(wide[:, :H * dk], wide[:, H * dk:2 * H * dk], wide[:, 2 * H * dk:], decay.to(DEV), state, st, H, dk, dv)
        assert out.dtype == torch.float32
        at = 0
        for s, p0, n in segs:
            got[s].append(out[at:at + n].cpu()); at += n
    for s in range(2):
        assert B.rel_err(torch.cat(got[s]), ref[s]) < 2e-5, s
    assert float(state[0].max()) == -300.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_rmsnorm_into_a_slice(dtype):
    from swiftllm_b200.worker.kernels.recurrent import gated_rmsnorm
    g = torch.Generator().manual_seed(4)
    x = torch.randn(9, 84, generator=g) * 5
    w = 1 + 0.1 * torch.randn(84, generator=g)
    gate = torch.randn(9, 84, generator=g).to(dtype)
    wide = torch.zeros(9, 100, dtype=dtype, device=DEV)
    gated_rmsnorm(x.to(DEV), w.to(DEV), gate.to(DEV), 1e-5, wide[:, 10:94], 1.3)
    ref = O.unit_rms(x, 1e-5) * w * torch.sigmoid(gate.float()) * 1.3
    assert B.rel_err(wide[:, 10:94], ref) < tol(dtype) and float(wide[:, :10].abs().max()) == 0 and float(wide[:, 94:].abs().max()) == 0
    gated_rmsnorm(x.to(DEV), w.to(DEV), None, 1e-5, wide[:, 10:94])
    assert B.rel_err(wide[:, 10:94], O.unit_rms(x, 1e-5) * w) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_with_pair_table(dtype):
    """The previous token comes from the row above or, at the start of a portion, from the sequence's state; position 0 takes
    the table's extra row whatever the state row holds."""
    from swiftllm_b200.worker.kernels.stream_ops import embed_pair_hash
    g = torch.Generator().manual_seed(5)
    vocab, W, buckets, mp, mc = 61, 40, 23, 31, 5
    embed = torch.randn(vocab, W, generator=g).to(dtype)
    pairs = torch.randn(buckets + 1, W, generator=g).to(dtype)
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    seqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (12, 5)]
    refs = [O.embed(s, {"embed": embed.float(), "bigram": pairs.float()}, cfg) for s in seqs]
    last = torch.full((4,), 7, dtype=torch.int32, device=DEV)
    got = [[], []]
    for segs in _schedule([12, 5], [[(0, 1), (1, 3)], [(0, 1), (1, 1)], [(0, 9)], [(1, 1)], [(0, 1)]]):
        st = _step([((3, 1)[s], p0, n) for s, p0, n in segs])
        ids = torch.tensor([t for s, p0, n in segs for t in seqs[s][p0:p0 + n]], dtype=torch.int32, device=DEV)
        copy = torch.empty(ids.shape[0], W, device=DEV)
        x, h = embed_pair_hash(ids, st, last, embed.to(DEV), pairs.to(DEV), buckets, mp, mc, x_copy=copy)
        assert x.dtype == torch.float32 and h.dtype == dtype and torch.equal(x, copy) and torch.equal(h, x.to(dtype))
        at = 0
        for s, p0, n in segs:
            got[s].append(x[at:at + n].cpu()); at += n
    for s in range(2):
        assert torch.allclose(torch.cat(got[s]), refs[s], rtol=0, atol=1e-6)
    assert last.tolist() == [7, seqs[1][-1], 7, seqs[0][-1]]
    x, _ = embed_pair_hash(ids, st, None, embed.to(DEV), None, 0, 0, 0)
    assert torch.equal(x.cpu(), embed.float()[ids.cpu().long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 1000])
def test_postnorm_add_and_depth_mix(dtype, width):
    from swiftllm_b200.worker.kernels.stream_ops import postnorm_add_mix
    g = torch.Generator().manual_seed(width)
    T, slots = 6, 4
    x = torch.randn(T, width, generator=g)
    y = (torch.randn(T, width, generator=g) * 3).to(dtype)
    gain = torch.tensor(0.8)
    hist = torch.randn(slots, T, width, generator=g)
    mix = torch.tensor([0.2, -0.5, 1.1])
    X = x + 0.8 * O.unit_rms(y.float(), 1e-5)
    # plain: add only
    xd, hd = x.clone().to(DEV), torch.empty(T, width, dtype=dtype, device=DEV)
    postnorm_add_mix(xd, y.to(DEV), gain.to(DEV), 1e-5, hd)
    assert B.rel_err(xd, X) < 1e-6 and torch.equal(hd, xd.to(dtype))
    # with the weighted sum over depth: slot 2 receives X, the stream becomes the mix of slots 0..2
    xd, hh = x.clone().to(DEV), hist.clone().to(DEV)
    postnorm_add_mix(xd, y.to(DEV), gain.to(DEV), 1e-5, hd, hh, 2, mix.to(DEV))
    assert B.rel_err(hh[2], X) < 1e-6 and torch.equal(hh[3].cpu(), hist[3]) and torch.equal(hh[:2].cpu(), hist[:2])
    assert B.rel_err(xd, 0.2 * hist[0] - 0.5 * hist[1] + 1.1 * X) < 1e-6 and torch.equal(hd, xd.to(dtype))


def test_tanh_cap():
    from swiftllm_b200.worker.kernels.stream_ops import tanh_cap_inplace
    z = torch.linspace(-80, 80, 1001)
    x = z.clone().to(DEV)
    tanh_cap_inplace(x, 6.0)
    assert torch.allclose(x.cpu(), O.tanh_cap(z, 6.0), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("experts,top", [(6, 2), (3, 1), (33, 4), (16, 3), (200, 32), (5, 5)])
def test_sigmoid_routing_with_a_choice_only_correction(experts, top):
    from swiftllm_b200.worker.kernels.stream_ops import moe_route_sigmoid
    g = torch.Generator().manual_seed(experts)
    h = torch.randn(29, 16, generator=g)
    router = torch.randn(experts, 16, generator=g)
    corr = torch.randn(experts, generator=g) * 0.5
    idx, wts = O.sigmoid_route(h, router, corr, top)
    ref = torch.zeros(29, experts)
    for t in range(29):
        for e, w in zip(idx[t], wts[t]):
            ref[t, e] = w
    got = moe_route_sigmoid((h @ router.T).to(DEV).contiguous(), corr.to(DEV), top).cpu()
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-7) and bool(((got > 0).sum(1) == top).all())


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_gated_experts_scaled(dtype):
    from swiftllm_b200.worker.kernels.stream_ops import moe_silu_glu_scale
    g = torch.Generator().manual_seed(6)
    T, E, ff = 7, 5, 12
    u = torch.randn(T, E * 2 * ff, generator=g).to(dtype)
    w = torch.rand(T, E, generator=g)
    w[w < 0.5] = 0.0
    uu = u.float().view(T, E, 2, ff)
    ref = (O.silu(uu[:, :, 0]) * uu[:, :, 1] * w[:, :, None]).view(T, E * ff)
    got = moe_silu_glu_scale(u.to(DEV), w.to(DEV), E, ff)
    assert got.dtype == dtype and B.rel_err(got, ref) < tol(dtype)
    assert bool((got.cpu().view(T, E, ff)[w == 0] == 0).all())


@pytest.mark.parametrize("H,G,dk,dv,dims,cap", [(8, 2, 32, 16, 32, 5.0), (6, 1, 64, 64, 16, 0.0), (6, 3, 112, 80, 56, 12.0),
                                                (12, 4, 48, 80, 0, 3.0), (4, 2, 128, 128, 128, 30.0)])
def test_attention_options_tensor_core_and_cuda_core_agree(H, G, dk, dv, dims, cap):
    """Halves rotary, unit-RMS queries and keys, capped scores, turned values, a factor on the output, no window: the same mixed
    step (prompt portions that start inside a sequence, decoded tokens) through the cache store and both attention kernels."""
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
    opt = WA.AttnOptions(pair_halves=True, qk_norm_eps=1e-6, softcap=cap, out_scale=0.75)

    def angles(pos, n, base=100.0):
        a = torch.tensor(pos, dtype=torch.float64)[:, None] * torch.tensor([base ** (-2.0 * i / n) for i in range(n // 2)],
                                                                           dtype=torch.float64)[None]
        return torch.cos(a).float().to(DEV), torch.sin(a).float().to(DEV)
    cache = torch.zeros(nb, 1, bs, G * (dk + dv), dtype=torch.bfloat16, device=DEV)
    # fill the cache through the store kernel: every sequence's full length as one prompt
    all_seq = [s for s, n in enumerate(lens) for _ in range(n)]
    all_pos = [p for n in lens for p in range(n)]
    st_all = types.SimpleNamespace(token_seq_ids=torch.tensor(all_seq, dtype=torch.int32, device=DEV),
                                   token_positions=torch.tensor(all_pos, dtype=torch.int32, device=DEV))
    k = torch.randn(len(all_seq), G * dk, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(len(all_seq), G * dv, generator=g).to(torch.bfloat16).to(DEV)
    cs, sn = angles(all_pos, dims) if dims else (None, None)
    vc, vs = angles(all_pos, dv)
    WA.window_kv_store(k, v, cache, 0, table, st_all, G, dk, dv, dims, cs, sn, opt, vc, vs)
    tok_seq = [s for s, n in enumerate(new) for _ in range(n)]
    tok_pos = [lens[s] - n + p for s, n in enumerate(new) for p in range(n)]
    T = len(tok_seq)
    q = torch.randn(T, H * dk, generator=g).to(torch.bfloat16).to(DEV)
    cs, sn = angles(tok_pos, dims) if dims else (None, None)
    vc, vs = angles(tok_pos, dv)
    st = types.SimpleNamespace(token_seq_ids=torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
                               token_positions=torch.tensor(tok_pos, dtype=torch.int32, device=DEV), num_prefill_tokens=191)
    outs = []
    for simt in (True, False):
        old = WA.set_simt(simt)
        try:
            out = torch.zeros(T, H * dv, dtype=torch.bfloat16, device=DEV)
            WA.window_attention(q, None, cache, 0, table, st, out, H, G, dk, dv, dims, 0, 3.0 / math.sqrt(dk), True, cs, sn, opt, vc, vs)
            outs.append(out.float().cpu())
        finally:
            WA.set_simt(old)
    assert B.rel_err(outs[1], outs[0]) < 1.5e-2
    row_err = (outs[1] - outs[0]).pow(2).mean(-1).sqrt() / outs[0].pow(2).mean(-1).sqrt()
    assert float(row_err.max()) < 5e-2


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
    B.case_long_decode(_make, C.config([(C.rglru(), C.moe()), (C.parallel(), None)]))


def test_greedy_generation():
    B.case_greedy_generation(_make, C.config([(C.rglru(), C.moe()), (C.parallel(), C.dense())]))


def test_far_key():
    C.case_far_key(_make)


def test_first_tokens_and_block_borders():
    C.case_first_tokens_and_block_borders(_make)


def test_sink():
    C.case_sink(_make)


def test_score_cap_binds():
    C.case_score_cap_binds(_make)


def test_slow_recurrence_remembers():
    C.case_slow_recurrence_remembers(_make)


def test_convolution_across_short_portions():
    C.case_convolution_across_short_portions(_make)


def test_correction_changes_the_choice_only():
    C.case_correction_changes_the_choice_only(_make)


def _tc_config():
    """Head sizes that are multiples of 16 (the shapes the 16-bit tensor-core attention takes), sequences over several key tiles."""
    return C.config([(C.parallel(C.attn(heads=8, kv_heads=2, dim=32, vdim=16, dims=32), C.lin(heads=2, dim=16, vdim=24)), C.moe()),
                     (C.rglru(width=64, blocks=4), C.dense()),
                     (C.parallel(C.attn(heads=6, kv_heads=1, dim=64, vdim=64, dims=16, scaling=None, softcap=None)), None),
                     (C.parallel(C.attn(heads=4, kv_heads=4, dim=16, vdim=48, dims=0, scaling=None), C.lin(heads=1, dim=32, vdim=32)),
                      C.moe(experts=5, top=1))], width=64)


def test_bfloat16_worker_close_to_fp32_oracle():
    """bf16 projections / cache, fp32 residual and states: the logits stay within bf16 rounding of the fp32 oracle on the same
    weights, and do not depend on how the prompt was cut beyond that."""
    for cfg, n, cuts, bs, nb in ((C.full_config(), 33, [5, 2, 1, 1, 24], 4, 40), (_tc_config(), 150, [61, 4, 64, 2, 1, 1, 17], 8, 60)):
        t = O.random_tensors(cfg, seed=11)
        toks = B.tokens_for(cfg, n, 11)
        ref = O.forward(cfg, t, toks)[-40:]
        m = B.make_worker(_make, cfg, t, dtype="bfloat16", block_size=bs, num_blocks=nb)
        whole = B.run_portions(m, toks, 0, [n])[-40:]
        cut = B.run_portions(m, toks, 1, cuts)[-40:]
        assert B.rel_err(whole, ref) < 4e-2 and B.rel_err(cut, ref) < 4e-2 and B.rel_err(cut, whole) < 3e-2


def test_cuda_graph_decode_matches_eager():
    """Pure-decode steps replayed from a CUDA graph: the per-sequence state rows (recurrence, convolution tail, linear-attention
    state, previous token) move on inside the graph exactly as in eager steps."""
    cfg = C.config([(C.rglru(), C.moe()), (C.parallel(), C.dense()), (C.rglru(width=16, blocks=2, conv=2), None)], width=64)
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
    # and the eager run is the oracle's greedy continuation
    want = B.oracle_greedy(cfg, t, prompts[0], 10)
    assert [s[0] for s in runs[0]] == want


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
        (C.parallel(C.attn(heads=10, kv_heads=2, dim=16, vdim=24, base=5000.0, dims=16, scaling=(4.0, 64, 16.0, 1.0)),
                    C.lin(heads=5, dim=8, vdim=16)), C.moe(experts=9, top=3, ff=24)),
        (C.rglru(width=40, blocks=5, conv=3), C.dense(ff=50, limit=1.5)),
        (C.parallel(C.attn(heads=3, kv_heads=3, dim=8, vdim=8, base=300.0, dims=6, scaling=None)), None),
        (C.rglru(width=72, blocks=2, conv=4), C.moe()),
    ], width=72, vocab=131, eps=1e-6)
    t = O.random_tensors(cfg, seed=21)
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in t.items()}, str(model_dir / "model.safetensors"))
    reqs = {k: B.tokens_for(cfg, n, s) for s, (k, n) in enumerate((("a", 70), ("b", 41), ("c", 17), ("d", 5), ("e", 30)))}
    ref = {k: O.forward(cfg, t, v).numpy() for k, v in reqs.items()}
    plan = [[("a", 33), ("b", 2)], [("a", 31), ("b", 30), ("c", 17)], [("a", 1), ("b", 1), ("d", 5)], [("a", 1), ("b", 1), ("e", 3)],
            [("a", 2), ("b", 7), ("e", 27)], [("a", 2)]]
    for dtype, limit in (("float32", 2e-4), ("bfloat16", 5e-2)):
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
        for n, rr in enumerate(rows):
            got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rr), -1)
            for j, (k, pos) in enumerate(rr):
                err = np.sqrt(((got[j] - ref[k][pos]) ** 2).mean() / (ref[k][pos] ** 2).mean())
                assert err < limit, (dtype, n, k, pos, err)

"""Configurations and scenarios for the Naforax worker (swiftllm_b200.worker.naforax_model) against the plain restatement of the
design in oracle/naforax.py.  The schedule scenarios (whole prompts, decoding, portions, mixed batches, reused blocks and rows,
greedy generation) are the ones of tests/bupozen_cases.py; here are the design's own configurations and the scenarios whose
weights are made so that one particular fault would show.  They run on the CPU (kernels replaced by tests/cpu_shim.py) and on a
GPU (the CUDA kernels): tests/test_naforax_cpu.py and tests/test_naforax_gpu.py call them with the `make` factory of their world.

All configurations are small and deliberately irregular: head sizes that are not multiples of 16 or of each other, value sizes
unrelated to key sizes, rotary on a part of a map / all of it / none, one / several / as many key-value heads as query heads,
chunks of 1, 5, 7 and more positions than the sequence has, one to four taps in both kinds of convolution, one and three norm
groups, states of 1 to 40 entries, layers without feed-forward, experts without a shared one, top-1 routing, a repeated range at
the start / in the middle / over everything, one, two and three passes, models without a repeated range or a logit cap."""
import math

import torch

from bupozen_cases import TOL, make_worker, rel_err, run_portions, tokens_for
from oracle import naforax as O


def attn(heads=6, kv_heads=2, dim=10, vdim=6, base=100.0, dims=6, chunk=7, scale=None, diff=0.35):
    return "attention", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "mask": {"size": chunk},
                         "rot": {"base": base, "dims": dims}, "scale": scale if scale is not None else 2.0 / math.sqrt(dim)}


def mingru(width=20):
    return "mingru", {"width": width}


def mamba(inner=18, state=5, dt_rank=3, conv=4):
    return "mamba1", {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=12, limit=0.75, shared=(10, 1.25)):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def config(layers, width=48, vocab=97, eps=1e-5, groups=3, mult=0.6, taps=3, loop=None, logit_cap=6.0):
    cfg = {"architecture": "Naforax", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
           "residual_mult": mult, "canon": {"taps": taps},
           "layers": [{"type": kind, "mixer": m, "mlp": f} for (kind, m), f in layers]}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_cap:
        cfg["logit_softcap"] = logit_cap
    return cfg


def full_config():
    """Every branch at once; layers 1 .. 3 (a recurrence, an attention, a scan) run three times."""
    return config([
        (attn(), dense()),
        (mingru(), moe()),
        (attn(heads=4, kv_heads=4, dim=8, vdim=12, dims=8, chunk=5), None),
        (mamba(), moe(experts=5, top=1, shared=None)),
        (attn(heads=5, kv_heads=1, dim=6, vdim=20, dims=0, chunk=64), moe(experts=33, top=4, ff=8)),
        (mamba(inner=7, state=40, dt_rank=1, conv=1), dense(ff=17)),
        (mingru(width=33), None),
    ], loop=(1, 4, 3))


SINGLE = {
    "attention_dense": config([(attn(), dense())]),
    "attention_no_ff_one_group": config([(attn(), None)], groups=1),
    "attention_mha_full_rotary": config([(attn(heads=3, kv_heads=3, dims=10), dense())]),
    "attention_mqa_wide_value_no_rotary": config([(attn(heads=5, kv_heads=1, dim=4, vdim=70, dims=0, chunk=3), dense())]),
    "attention_chunk_of_one": config([(attn(chunk=1), dense())]),
    "attention_16bit_shapes": config([(attn(heads=4, kv_heads=2, dim=16, vdim=32, dims=4, chunk=6), None)]),
    "mingru_moe": config([(mingru(), moe())]),
    "mingru_no_ff_one_tap": config([(mingru(width=7), None)], taps=1),
    "mamba_dense": config([(mamba(), dense())], taps=2),
    "mamba_one_state_two_taps": config([(mamba(inner=11, state=1, dt_rank=2, conv=2), None)], taps=4),
    "mamba_many_states": config([(mamba(inner=6, state=37, dt_rank=5, conv=3), None)]),
    "moe_top1_no_shared": config([(mingru(), moe(experts=3, top=1, shared=None))]),
    "moe_all_experts": config([(mingru(), moe(experts=4, top=4))]),
    "loop_everything_twice": config([(mingru(), dense()), (attn(), None)], loop=(0, 2, 2)),
    "loop_once_no_cap": config([(attn(), None), (mamba(), dense())], loop=(1, 2, 1), logit_cap=None, mult=1.0),
}


# ---------------------------------------------------------------- scenarios made so that one fault shows
def _attention_probe(n, key_pos, chunk, H=2, dk=8, dv=6, width=16, vocab=32, scale=3.0, dims=0):
    """One attention layer whose first score map makes every query point along one direction: the key of the marked token
    (token 1) points the same way, all other keys are orthogonal to it; the marked token's value fills the first half of a head's
    output, the ordinary tokens' values the second half.  The second map's queries are zero (uniform weights).  Queries and keys
    are RMS-normed, so `scale` alone sets how far the marked score (scale * dk) stands above the others (0).  The input
    convolution is switched off so that only the marked position carries the mark."""
    cfg = config([(attn(heads=H, kv_heads=1, dim=dk, vdim=dv, dims=dims, chunk=chunk, scale=scale), None)], width=width, vocab=vocab,
                 groups=1, logit_cap=None, taps=2)
    t = O.random_tensors(cfg, seed=11, dtype=torch.float32)
    t["embed"] = torch.randn(vocab, width, generator=torch.Generator().manual_seed(1)) * 0.1
    t["embed"][:, 0] = 1.0                       # every query reads this constant ...
    t["embed"][:, 1] = 0.0
    t["embed"][:, 2] = 1.0                       # ... every ordinary key this one ...
    t["embed"][1, 1] = 4.0                       # ... and only the marked token carries these
    t["embed"][1, 2] = 0.0
    t["l0.norm1"] = torch.ones(width)
    t["l0.canon1"] = torch.zeros(width, 2)
    q = torch.zeros(H, 2, dk, width); q[:, 0, :, 0] = 2.0              # map 0: all entries equal, direction (1, ..., 1)
    k = torch.zeros(2, dk, width)
    k[0, :, 1] = 2.0                                                   # marked key: along the queries
    k[0, : dk // 2, 2], k[0, dk // 2:, 2] = 1.0, -1.0                  # ordinary keys: orthogonal to the queries
    v = torch.zeros(dv, width); v[: dv // 2, 1] = 3.0; v[dv // 2:, 2] = 3.0
    t["l0.mix.q"], t["l0.mix.k"], t["l0.mix.v"] = q.reshape(H * 2 * dk, width), k.reshape(2 * dk, width), v
    for name in ("q.b", "k.b", "v.b"):
        t[f"l0.mix.{name}"] = torch.zeros_like(t[f"l0.mix.{name}"])
    t["l0.mix.q.norm"], t["l0.mix.k.norm"] = torch.ones(dk), torch.ones(dk)
    toks = [2 + (i % (vocab - 2)) for i in range(n)]
    toks[key_pos] = 1
    return cfg, t, toks


def case_far_key(make):
    """A marked key hundreds of positions back among keys that all score the same, in a chunk longer than the sequence: every
    later position must still see it, across blocks, in prompt portions and when decoding."""
    cfg, t, toks = _attention_probe(n=390, key_pos=3, chunk=512)
    ref = O.forward(cfg, t, toks)
    plain = list(toks); plain[3] = 5
    assert rel_err(O.forward(cfg, t, plain)[-1], ref[-1]) > 0.05
    model = make_worker(make, cfg, t, block_size=8, num_blocks=50)
    got = run_portions(model, toks, 0, [200, 150, 38, 1, 1])
    assert rel_err(got[-8:], ref[-8:]) < TOL and rel_err(got, ref) < TOL


def case_chunk_edges(make):
    """The marked key at the last position of a chunk, at the first of the next and in its middle: queries up to the chunk's end
    see it, the next chunk's first query does not - in a prompt, decoded, and with portions cut at, before and after the edge.
    Chunks are counted from the sequence's start, not from a portion's."""
    c = 12
    for key_pos in (c - 1, c, c + 5, 2 * c - 1):
        cfg, t, toks = _attention_probe(n=3 * c + 2, key_pos=key_pos, chunk=c, dims=4)
        ref = O.forward(cfg, t, toks)
        for off in (-1, 1):                       # a chunk that is one position longer or shorter gives other logits
            other = {**cfg, "layers": [{**cfg["layers"][0], "mixer": {**cfg["layers"][0]["mixer"], "mask": {"size": c + off}}}]}
            assert rel_err(O.forward(other, t, toks), ref) > 0.01
        for cuts in ([3 * c + 2], [c, c, c + 2], [c - 1, 2, c - 1, 1, 1, c], [c + 1, c - 2, 1, c + 2], [5] + [1] * (3 * c - 3),
                     [2] * (c + c // 2) + [2]):
            model = make_worker(make, cfg, t, block_size=8, num_blocks=8)
            got = run_portions(model, toks, 1, cuts)
            assert rel_err(got, ref) < TOL, (key_pos, cuts)
            # just inside and just outside, one by one
            for p in (key_pos, (key_pos // c + 1) * c - 1, (key_pos // c + 1) * c):
                assert rel_err(got[p], ref[p]) < TOL, (key_pos, cuts, p)


def case_first_tokens_and_block_borders(make):
    """The marked key at the first position, at the last slot of a block and at the first slot of the next one; queries right
    behind it, in a prompt and decoded."""
    for key_pos in (0, 7, 8):
        cfg, t, toks = _attention_probe(n=20, key_pos=key_pos, chunk=32)
        ref = O.forward(cfg, t, toks)
        for cuts in ([20], [key_pos + 1, 1, 1, 17 - key_pos], [2] + [1] * 18, [8, 8, 4]):
            model = make_worker(make, cfg, t, block_size=8, num_blocks=6)
            assert rel_err(run_portions(model, toks, 1, cuts), ref) < TOL, (key_pos, cuts)


def case_lambda_and_head_norm(make):
    """Learned vectors that make lambda large, so that the second map dominates the difference, and a value projection whose
    heads differ a hundredfold in size: the per-head normalisation brings them to the same size."""
    cfg = config([(attn(heads=4, kv_heads=2, dim=6, vdim=5, diff=0.8), dense())])
    t = O.random_tensors(cfg, seed=21, dtype=torch.float32)
    t["l0.mix.lq1"], t["l0.mix.lk1"] = torch.full((6,), 0.6), torch.full((6,), 0.5)      # exp(1.8)
    t["l0.mix.lq2"], t["l0.mix.lk2"] = torch.full((6,), -0.5), torch.full((6,), 0.5)     # exp(-1.5)
    assert O.differential_factor(O.sub(t, "l0.mix."), 0.8) > 6.0
    t["l0.mix.v"][:5] *= 100.0
    toks = tokens_for(cfg, 25, 21)
    ref = O.forward(cfg, t, toks)
    small = dict(t); small["l0.mix.lq1"] = torch.zeros(6)
    assert rel_err(O.forward(cfg, small, toks), ref) > 0.01
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [11, 1, 1, 12]), ref) < TOL


def case_slow_recurrences_remember(make):
    """A minGRU whose gate is nearly shut and a scan with tiny steps and slow decays: what the first tokens wrote is still in the
    state hundreds of tokens later, through portions and decoding."""
    cfg = config([(mingru(width=16), None), (mamba(inner=12, state=6, dt_rank=2, conv=3), None)], width=32, groups=2)
    t = O.random_tensors(cfg, seed=14, dtype=torch.float32)
    t["l0.mix.z.b"] = torch.full((16,), -6.0)
    t["l0.mix.z"] *= 0.1
    t["l1.mix.dt.b"] = torch.full((12,), -5.0)
    t["l1.mix.dt"] *= 0.1
    t["l1.mix.A_log"] = torch.full((12, 6), -2.0)
    toks = tokens_for(cfg, 300, 14)
    ref = O.forward(cfg, t, toks, dtype=torch.float64)
    other = list(toks); other[0] = (toks[0] + 1) % cfg["vocab"]; other[1] = (toks[1] + 3) % cfg["vocab"]
    assert rel_err(O.forward(cfg, t, other, dtype=torch.float64)[-1], ref[-1]) > 1e-3     # the start still matters at the end
    model = make_worker(make, cfg, t, block_size=16, num_blocks=20)
    got = run_portions(model, toks, 2, [130, 2, 100, 3, 1, 1] + [1] * 63)
    assert rel_err(got, ref) < TOL and rel_err(got[-1], ref[-1]) < TOL


def case_convolutions_across_short_portions(make):
    """Portions shorter than the convolutions' reach (four taps on every sublayer's input and in the scan): their inputs come from
    the step, from the previous step and from the one before, in every mix."""
    cfg = config([(mamba(inner=12, state=3, dt_rank=2, conv=4), dense()), (mingru(width=8), None)], width=24, taps=4)
    t = O.random_tensors(cfg, seed=15, dtype=torch.float32)
    t["l0.mix.conv"] = torch.tensor([[1.5, -1.0, 0.75, 0.5]]).repeat(12, 1)   # old inputs weigh as much as the current one
    t["l0.canon1"] = torch.tensor([[0.9, -1.1, 0.7, 0.4]]).repeat(24, 1)
    t["l0.canon2"] = torch.tensor([[-0.8, 0.6, 1.2, -0.3]]).repeat(24, 1)
    toks = tokens_for(cfg, 19, 15)
    ref = O.forward(cfg, t, toks)
    model = make_worker(make, cfg, t)
    for cuts in ([1] * 19, [2, 1, 2, 1, 1, 2, 10], [1, 2, 3, 4, 9], [3, 1, 1, 1, 13], [19]):
        assert rel_err(run_portions(model, toks, 3, cuts), ref) < TOL, cuts
        model.free_seqs_resources([3])
        assert rel_err(run_portions(model, toks, 3, cuts, decode_single=False), ref) < TOL, cuts
        model.free_seqs_resources([3])


def case_router_scores_are_not_renormalised(make):
    """Router logits that leave the chosen experts a small share of the softmax: their weights are those small scores (the
    feed-forward's normed output keeps its direction but the shared expert's share of it grows); a tie goes to the lower index."""
    cfg = config([(mingru(), moe(experts=6, top=2))])
    t = O.random_tensors(cfg, seed=16, dtype=torch.float32)
    t["l0.mlp.router"] *= 0.05                    # nearly uniform scores: the two chosen experts weigh about 1/6 each
    t["l0.mlp.router"][3] = t["l0.mlp.router"][1]         # experts 1 and 3 tie everywhere
    toks = tokens_for(cfg, 14, 16)
    ref = O.forward(cfg, t, toks)
    h = torch.randn(5, 48, generator=torch.Generator().manual_seed(3))
    chosen, weights = O.softmax_route(h, t["l0.mlp.router"], 2)
    assert float(weights.sum(-1).max()) < 0.5 and not ((chosen == 3).any(-1) & ~(chosen == 1).any(-1)).any()
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [6, 1, 7]), ref) < TOL


def case_state_rows_used_again(make):
    """A row whose previous sequence left recurrent states and convolution tails of every kind: the next sequence in that row
    starts from nothing, also when its first portion is a single token."""
    cfg = config([(mingru(), None), (mamba(), dense()), (attn(), None)], loop=(0, 2, 2))
    t = O.random_tensors(cfg, seed=17, dtype=torch.float32)
    model = make_worker(make, cfg, t, block_size=4, num_blocks=24, rows=2)
    a, b, c = tokens_for(cfg, 30, 50), tokens_for(cfg, 9, 51), tokens_for(cfg, 12, 52)
    ra, rb, rc = (O.forward(cfg, t, s) for s in (a, b, c))
    assert rel_err(run_portions(model, a, 1, [30]), ra) < TOL
    model.free_seqs_resources([1])
    assert rel_err(run_portions(model, b, 1, [1, 1, 7]), rb) < TOL            # one-token first portion in the used row
    model.free_seqs_resources([1])
    assert rel_err(run_portions(model, c, 1, [5, 7]), rc) < TOL
    assert rel_err(run_portions(model, a[:10], 0, [10]), ra[:10]) < TOL       # the other row, never used before


def case_passes_keep_their_own_state(make):
    """A repeated range with an attention and a recurrence: the second pass must not read the first pass's keys or state.  The
    reference is the same model written out as six layers without a repeated range (the pass's additions folded into the
    oracle's loop handling are checked by the whole-prompt scenarios)."""
    cfg = config([(attn(chunk=9), None), (mingru(), dense())], loop=(0, 2, 3))
    t = O.random_tensors(cfg, seed=18, dtype=torch.float32)
    toks = tokens_for(cfg, 31, 18)
    ref = O.forward(cfg, t, toks)
    once = {**cfg, "loop": {"start": 0, "stop": 2, "times": 1}}
    t1 = dict(t); t1["loop.step"] = t["loop.step"][:1]
    assert rel_err(O.forward(once, t1, toks), ref) > 0.01
    model = make_worker(make, cfg, t, block_size=4, num_blocks=12)
    assert len(model.layers) == 6 and sum(model.model_config.cache_slots_per_width.values()) == 3
    assert rel_err(run_portions(model, toks, 0, [8, 1, 1, 2, 19]), ref) < TOL

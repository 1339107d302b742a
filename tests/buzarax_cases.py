"""Configurations and scenarios for the Buzarax worker (swiftllm_b200.worker.buzarax_model) against the plain restatement of the
design in oracle/buzarax.py.  The schedule scenarios (whole prompts, decoding, portions, mixed batches, reused blocks and rows,
greedy generation) are the ones of tests/bupozen_cases.py; here are the design's own configurations and the scenarios whose
weights are made so that one particular fault would show.  They run on the CPU (kernels replaced by tests/cpu_shim.py) and on a
GPU (the CUDA kernels): tests/test_buzarax_cpu.py and tests/test_buzarax_gpu.py call them with the `make` factory of their world.

All configurations are small and deliberately irregular: head sizes that are not multiples of 32 or of each other, value sizes
different from key sizes, rotary on a part of a head / all of it / none, with and without stretched frequencies, one / several /
as many key-value heads as query heads, one to four convolution taps, one gate block and several, layers without feed-forward,
top-1 routing, weights of 1 in the sum of the two mixers, models without the pair table or the logit cap."""
import math

import torch

from bupozen_cases import TOL, make_worker, rel_err, run_portions, tokens_for
from oracle import buzarax as O


def attn(heads=6, kv_heads=2, dim=10, vdim=6, base=100.0, dims=6, scaling=(3.0, 40, 8.0, 1.0), scale=None, softcap=5.0):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    a = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot,
         "scale": scale if scale is not None else 2.0 / math.sqrt(dim)}
    if softcap:
        a["softcap"] = softcap
    return a


def lin(heads=3, dim=5, vdim=7, decay=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay or [0.5 + 0.49 * (h + 1) / heads for h in range(heads)]}


def parallel(left=None, right=None, left_scale=0.7, right_scale=1.3):
    return "parallel", {"left": left or attn(), "right": right or lin(), "left_scale": left_scale, "right_scale": right_scale}


def rglru(width=24, blocks=3, conv=4):
    return "rglru", {"width": width, "blocks": blocks, "conv": conv}


def dense(ff=40, limit=0.75):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, top=2, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, width=48, vocab=97, eps=1e-5, pair=(53, 31, 5), logit_cap=6.0):
    cfg = {"architecture": "Buzarax", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [{"type": kind, "mixer": m, "mlp": f} for (kind, m), f in layers]}
    if pair is not None:
        cfg["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), pair))}
    if logit_cap:
        cfg["logit_softcap"] = logit_cap
    return cfg


def full_config():
    """Every branch at once."""
    return config([
        (rglru(), moe()),
        (parallel(), dense()),
        (parallel(attn(heads=4, kv_heads=4, dim=8, vdim=12, dims=8, scaling=None, softcap=None), lin(heads=1, dim=9, vdim=4),
                  left_scale=1.0, right_scale=1.0), None),
        (rglru(width=20, blocks=1, conv=2), dense(ff=17, limit=2.5)),
        (parallel(attn(heads=5, kv_heads=1, dim=6, vdim=20, dims=0, scaling=None), lin(heads=4, dim=12, vdim=3)), moe(experts=5, top=1)),
        (rglru(width=33, blocks=11, conv=1), None),
        (parallel(attn(heads=9, kv_heads=3, dim=12, vdim=4, dims=12, scaling=(8.0, 16, 4.0, 0.5))), moe(experts=33, top=4, ff=8)),
    ])


SINGLE = {
    "recurrence_moe": config([(rglru(), moe())]),
    "recurrence_no_ff": config([(rglru(conv=3), None)]),
    "recurrence_one_tap_one_block": config([(rglru(width=10, blocks=1, conv=1), dense())]),
    "parallel_dense": config([(parallel(), dense())]),
    "parallel_no_ff": config([(parallel(), None)]),
    "parallel_top1": config([(parallel(), moe(experts=3, top=1))]),
    "mha_plain_rotary": config([(parallel(attn(heads=3, kv_heads=3, dims=10, scaling=None)), dense())]),
    "mqa_wide_value_no_rotary": config([(parallel(attn(heads=5, kv_heads=1, dim=4, vdim=70, dims=0, scaling=None)), dense())]),
    "no_cap_unit_weights": config([(parallel(attn(softcap=None), left_scale=1.0, right_scale=1.0), dense())], logit_cap=None),
    "no_pair_table": config([(rglru(), dense()), (parallel(), None)], pair=None),
    "one_decay_large_state": config([(parallel(right=lin(heads=2, dim=40, vdim=36)), None)]),
}


# ---------------------------------------------------------------- scenarios made so that one fault shows
def _attention_probe(n, key_pos, H=2, dk=8, dv=6, width=16, vocab=32, scale=3.0, softcap=None, k_sign=1.0):
    """One parallel mixer whose linear-attention half is switched off (weight 0) and whose attention weights make every query
    point along one direction: the key of the marked token (token 1) points the same way (cosine 1), all other keys are
    orthogonal to it; the marked token's value fills the first half of a head's output, the ordinary tokens' values the second
    half (so the split between them survives the norm on the mixer's output).  Queries and keys have unit RMS, so `scale` alone
    sets how far the marked score (scale * dk) stands above the others (0)."""
    a = attn(heads=H, kv_heads=1, dim=dk, vdim=dv, dims=0, scaling=None, scale=scale, softcap=softcap)
    cfg = config([(parallel(a, lin(heads=1, dim=4, vdim=4), left_scale=1.0, right_scale=0.0), None)], width=width, vocab=vocab,
                 pair=None, logit_cap=None)
    t = O.random_tensors(cfg, seed=11, dtype=torch.float32)
    t["embed"] = torch.randn(vocab, width, generator=torch.Generator().manual_seed(1)) * 0.1
    t["embed"][:, 0] = 1.0                       # every query reads this constant ...
    t["embed"][:, 1] = 0.0
    t["embed"][:, 2] = 1.0                       # ... every ordinary key this one ...
    t["embed"][1, 1] = 4.0                       # ... and only the marked token carries these
    t["embed"][1, 2] = 0.0
    q = torch.zeros(H * dk, width); q[:, 0] = 2.0                    # all entries equal: direction (1, 1, ..., 1)
    k = torch.zeros(dk, width)
    k[:, 1] = 2.0 * k_sign                                           # marked key: along (or against) the queries
    k[: dk // 2, 2], k[dk // 2:, 2] = 1.0, -1.0                      # ordinary keys: orthogonal to the queries
    v = torch.zeros(dv, width); v[: dv // 2, 1] = 3.0; v[dv // 2:, 2] = 3.0
    t["l0.mix.left.q"], t["l0.mix.left.k"], t["l0.mix.left.v"] = q, k, v
    t["l0.dwa"] = torch.tensor([0.0, 1.0])
    toks = [2 + (i % (vocab - 2)) for i in range(n)]
    toks[key_pos] = 1
    return cfg, t, toks


def case_far_key(make):
    """A marked key hundreds of positions back among keys that all score the same: every later position must still see it,
    across blocks, in prompt portions and when decoding."""
    cfg, t, toks = _attention_probe(n=390, key_pos=3)
    ref = O.forward(cfg, t, toks)
    model = make_worker(make, cfg, t, block_size=8, num_blocks=50)
    got = run_portions(model, toks, 0, [200, 150, 38, 1, 1])
    assert rel_err(got[-8:], ref[-8:]) < TOL
    blind = dict(t); blind["l0.mix.left.v"] = torch.zeros_like(t["l0.mix.left.v"])
    assert rel_err(O.forward(cfg, blind, toks)[-1], ref[-1]) > 0.05


def case_first_tokens_and_block_borders(make):
    """The marked key at the first position, at the last slot of a block and at the first slot of the next one; queries right
    behind it, in a prompt and decoded."""
    for key_pos in (0, 7, 8):
        cfg, t, toks = _attention_probe(n=20, key_pos=key_pos)
        ref = O.forward(cfg, t, toks)
        for cuts in ([20], [key_pos + 1, 1, 1, 17 - key_pos], [2] + [1] * 18, [8, 8, 4]):
            model = make_worker(make, cfg, t, block_size=8, num_blocks=6)
            assert rel_err(run_portions(model, toks, 1, cuts), ref) < TOL, (key_pos, cuts)


def case_sink(make):
    """Every score far below zero: with the extra 1 in the denominator the weights are tiny and the mixer's output nearly
    vanishes; a plain softmax would return the mean of the values."""
    cfg, t, toks = _attention_probe(n=15, key_pos=2, k_sign=-1.0)
    toks = [1] * 15                              # every key is a marked one: all scores = -scale * dk
    ref, layers = O.forward(cfg, t, toks, keep_layers=True)
    x0 = O.embed(toks, {k: v.float() for k, v in t.items()}, cfg)
    # the post-norm would blow a tiny output up again: look at the mixer itself
    h = x0
    y = O.capped_sink_attention(h, list(range(15)), O.sub(O.sub(t, "l0."), "mix.left."), cfg["layers"][0]["mixer"]["left"], 1e-5)
    v_only = (h @ t["l0.mix.left.v"].T) @ t["l0.mix.left.o"][:, :6].T
    assert float(y.abs().max()) < 1e-6 * float(v_only.abs().max())
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [9, 1, 5]), ref) < TOL
    # and large positive scores leave the 1 negligible
    cfg, t, toks = _attention_probe(n=15, key_pos=2)
    ref = O.forward(cfg, t, toks)
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [15]), ref) < TOL


def case_score_cap_binds(make):
    """Scores of 24 against a cap of 4: the marked key keeps a bounded lead (e^4 against e^0 per ordinary key), so the ordinary
    keys still carry weight; without the cap they would carry none."""
    cfg, t, toks = _attention_probe(n=40, key_pos=5, softcap=4.0)
    ref = O.forward(cfg, t, toks)
    free = {**cfg, "layers": [{**cfg["layers"][0], "mixer": {**cfg["layers"][0]["mixer"],
                                                              "left": {**cfg["layers"][0]["mixer"]["left"], "softcap": 400.0}}}]}
    assert rel_err(O.forward(free, t, toks)[10:], ref[10:]) > 0.02
    model = make_worker(make, cfg, t, block_size=8, num_blocks=8)
    assert rel_err(run_portions(model, toks, 0, [17, 2, 1, 20]), ref) < TOL


def case_slow_recurrence_remembers(make):
    """Decays close to 1 (a recurrence whose state fades over thousands of steps, a linear attention with decay 0.9999): what
    the first tokens wrote is still the bulk of the state hundreds of tokens later, through portions and decoding."""
    cfg = config([(rglru(width=16, blocks=2, conv=3), None), (parallel(right=lin(heads=2, dim=6, vdim=5, decay=[0.9999, 0.97])), None)],
                 width=32)
    t = O.random_tensors(cfg, seed=14, dtype=torch.float32)
    t["l0.mix.lam"] = torch.full((16,), -9.0)            # a = exp(-8 r softplus(-9)) ~ 1 - 1e-3 r
    toks = tokens_for(cfg, 300, 14)
    # the reference in fp64: near a = 1 an fp32 evaluation of 1 - a^2 keeps only three or four digits
    ref = O.forward(cfg, t, toks, dtype=torch.float64)
    other = list(toks); other[0] = (toks[0] + 1) % cfg["vocab"]; other[1] = (toks[1] + 3) % cfg["vocab"]
    assert rel_err(O.forward(cfg, t, other, dtype=torch.float64)[-1], ref[-1]) > 1e-3     # the start still matters at the end
    model = make_worker(make, cfg, t, block_size=16, num_blocks=20)
    got = run_portions(model, toks, 2, [130, 2, 100, 3, 1, 1] + [1] * 63)
    assert rel_err(got, ref) < TOL and rel_err(got[-1], ref[-1]) < TOL


def case_convolution_across_short_portions(make):
    """Portions shorter than the convolution's reach: its inputs come from the step, from the previous step and from the one
    before, in every mix."""
    cfg = config([(rglru(width=12, blocks=2, conv=4), None), (rglru(width=8, blocks=1, conv=2), dense())], width=24)
    t = O.random_tensors(cfg, seed=15, dtype=torch.float32)
    t["l0.mix.conv"] = torch.tensor([[1.5, -1.0, 0.75, 0.5]]).repeat(12, 1)   # old inputs weigh as much as the current one
    toks = tokens_for(cfg, 19, 15)
    ref = O.forward(cfg, t, toks)
    model = make_worker(make, cfg, t)
    for cuts in ([1] * 19, [2, 1, 2, 1, 1, 2, 10], [1, 2, 3, 4, 9], [3, 1, 1, 1, 13], [19]):
        assert rel_err(run_portions(model, toks, 3, cuts), ref) < TOL, cuts
        model.free_seqs_resources([3])
        assert rel_err(run_portions(model, toks, 3, cuts, decode_single=False), ref) < TOL, cuts
        model.free_seqs_resources([3])


def case_correction_changes_the_choice_only(make):
    """A correction that lifts an expert with a low score into the chosen set: it is chosen, and weighted by its (low) plain
    score; a router that added the correction to the weights, or ignored it, gives other logits."""
    cfg = config([(rglru(), moe(experts=6, top=2))])
    t = O.random_tensors(cfg, seed=16, dtype=torch.float32)
    t["l0.mlp.correction"] = torch.tensor([0.0, 0.0, 5.0, 0.0, 0.0, 0.0])
    toks = tokens_for(cfg, 14, 16)
    ref = O.forward(cfg, t, toks)
    none = dict(t); none["l0.mlp.correction"] = torch.zeros(6)
    assert rel_err(O.forward(cfg, none, toks), ref) > 0.01
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [6, 1, 7]), ref) < TOL


def case_state_rows_used_again(make):
    """A row whose previous sequence left a large recurrent state, a convolution tail and a last token: the next sequence in
    that row starts from nothing, also when its first portion is a single token."""
    cfg = config([(rglru(), None), (parallel(), dense())])
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

"""Scenarios that compare the Bupozen worker (swiftllm_b200.worker.bupozen_model) with the plain restatement of the design in
oracle/bupozen.py.  The same scenarios run on the CPU (host path, kernels replaced by tests/cpu_shim.py) and on a GPU (the CUDA
kernels): tests/test_bupozen_cpu.py and tests/test_bupozen_gpu.py call them with the `make` factory of their world.

All configurations are small and deliberately irregular: sizes that are not multiples of 32 or of each other, rotary on a part
of the rotated entries only, a layer without feed-forward, layers that borrow another layer's latent with other head counts
and windows, two latent widths (two cache tensors), more heads than one CTA takes, top-1 and top-k routing."""
import numpy as np
import torch

from oracle import bupozen as O
from oracle import buzarax as _buzarax
from oracle import naforax as _naforax
from oracle import rivudra as _rivudra

_ORACLES = {"Bupozen": O, "Rivudra": _rivudra, "Buzarax": _buzarax, "Naforax": _naforax}


def oracle_of(cfg):
    """The plain restatement of the design a configuration names (the scenarios below serve every parallel-block design)."""
    return _ORACLES[cfg["architecture"]]


def mixer(heads=3, dim=8, rot_dim=6, vdim=5, kv_rank=24, q_rank=12, window=7, base=100.0, dims=4, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "mask": {"size": window}, "rot": {"base": base, "dims": dims}, "scale": 1.0 / (dim + rot_dim) ** 0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


DENSE = {"kind": "dense", "ff": 40}


def moe(experts=6, top=2, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, width=48, vocab=97, eps=1e-5):
    return {"architecture": "Bupozen", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{"type": "latent_attention", "mixer": m, "mlp": f} for m, f in layers]}


def full_config():
    """Every branch at once."""
    return config([
        (mixer(), DENSE),
        (mixer(heads=2, dim=4, vdim=9, window=5, kv_from=0), moe()),                  # borrows layer 0's latent, other heads / window
        (mixer(heads=11, kv_rank=72, rot_dim=4, dims=4, window=13), None),            # second latent width, > 8 heads, no feed-forward
        (mixer(heads=11, kv_rank=72, rot_dim=4, dims=4, window=3, kv_from=2), moe(experts=5, top=1)),
        (mixer(window=64, dims=6), moe(experts=33, top=4, ff=8)),                     # window longer than the sequences
    ])


SINGLE = {
    "dense": config([(mixer(), DENSE)]),
    "no_ff": config([(mixer(), None)]),
    "moe": config([(mixer(), moe())]),
    "top1": config([(mixer(), moe(experts=3, top=1))]),
    "full_rotary_window1": config([(mixer(dims=6, window=1), DENSE)]),
    "no_rotary_wide": config([(mixer(dims=0, kv_rank=136, heads=9, window=9), DENSE)]),
}


def make_worker(make, cfg, tensors, dtype="float32", block_size=4, num_blocks=40, rows=4):
    """`make(cfg, tensors, engine kwargs)` -> initialised worker."""
    return make(cfg, tensors, dict(dtype=dtype, block_size=block_size, num_blocks=num_blocks, rows=rows))


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())


def run_portions(model, tokens, row, cuts, decode_single=True):
    """Feed one sequence in the portions given by `cuts` (lengths); single tokens after the first portion go in as decode
    entries.  Returns logits [len(tokens), vocab]."""
    out, at = [], 0
    for n in cuts:
        part = tokens[at:at + n]
        if n == 1 and at > 0 and decode_single:
            model.forward([part], [row], [at + 1], logit_rows=[0])
        else:
            model.forward([part], [row], [], prefill_prefix_lens_list=[at], logit_rows=list(range(n)))
        out.append(model.last_logits.cpu())
        at += n
    assert at == len(tokens)
    return torch.cat(out)


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


TOL = 2e-4     # fp32 worker against the fp32 oracle: relative rms error of the logits


# ---------------------------------------------------------------- scenarios
def case_whole_prompt(make, cfg, n=23, seed=0):
    t = oracle_of(cfg).random_tensors(cfg, seed=seed)
    model = make_worker(make, cfg, t)
    toks = tokens_for(cfg, n, seed)
    ref, layers = oracle_of(cfg).forward(cfg, t, toks, keep_layers=True)
    model.keep_residuals = True
    got = run_portions(model, toks, 1, [n])
    for i, r in enumerate(model.last_residuals):
        assert rel_err(r, layers[i]) < TOL, f"residual after layer {i}"
    assert rel_err(got, ref) < TOL


def case_prefill_vs_decode(make, cfg, n=30, first=3, seed=1):
    """The first tokens as one portion, every other token decoded alone (windows slide past their start while decoding)."""
    t = oracle_of(cfg).random_tensors(cfg, seed=seed)
    model = make_worker(make, cfg, t)
    toks = tokens_for(cfg, n, seed)
    ref = oracle_of(cfg).forward(cfg, t, toks)
    got = run_portions(model, toks, 2, [first] + [1] * (n - first))
    assert rel_err(got, ref) < TOL
    # token by token from the very first one (position 0 alone is a one-token prompt)
    model.free_seqs_resources([2])
    got = run_portions(model, toks[:12], 2, [1] * 12)
    assert rel_err(got, ref[:12]) < TOL


def case_portions(make, cfg, seed=2):
    t = oracle_of(cfg).random_tensors(cfg, seed=seed)
    toks = tokens_for(cfg, 37, seed)
    ref = oracle_of(cfg).forward(cfg, t, toks)
    model = make_worker(make, cfg, t)
    for cuts in ([2, 2, 2, 31], [5, 7, 1, 3, 2, 19], [36, 1], [4] * 9 + [1], [13, 2, 22]):
        got = run_portions(model, toks, 0, cuts)
        assert rel_err(got, ref) < TOL, cuts
        model.free_seqs_resources([0])
    # one-token portions that are sent as PROMPT portions (not as decode entries) take the same path as longer ones
    got = run_portions(model, toks[:9], 0, [3, 1, 1, 4], decode_single=False)
    assert rel_err(got, ref[:9]) < TOL


def case_mixed_batch(make, cfg, seed=3):
    """Unequal requests in one batch - portions of some beside decoded tokens of others - against each alone."""
    t = oracle_of(cfg).random_tensors(cfg, seed=seed)
    lens = [19, 6, 31, 1]
    seqs = [tokens_for(cfg, n, seed * 10 + k) for k, n in enumerate(lens)]
    refs = [oracle_of(cfg).forward(cfg, t, s) for s in seqs]
    model = make_worker(make, cfg, t)
    rows = [3, 0, 2, 1]
    got = [[None] * n for n in lens]
    # step 1: seq0 portion [0,7), seq2 portion [0,20), seq3 whole (1 token)
    # step 2: seq0 portion [7,18), seq1 whole, seq2 decode 20
    # step 3: seq0 decode 18, seq2 portion [21,31), seq1 nothing
    plan = [
        [(0, 0, 7), (2, 0, 20), (3, 0, 1)],
        [(0, 7, 18), (1, 0, 6), (2, 20, 21)],
        [(2, 21, 31), (0, 18, 19)],
    ]
    for step in plan:
        pre = [(k, lo, hi) for k, lo, hi in step if not (hi - lo == 1 and lo > 0)]
        dec = [(k, lo, hi) for k, lo, hi in step if hi - lo == 1 and lo > 0]
        order = pre + dec
        want, at = [], 0
        for k, lo, hi in order:
            want += list(range(at, at + hi - lo)); at += hi - lo
        model.forward([seqs[k][lo:hi] for k, lo, hi in order], [rows[k] for k, _, _ in order], [hi for _, _, hi in dec],
                      prefill_prefix_lens_list=[lo for _, lo, _ in pre], logit_rows=want)
        lg, at = model.last_logits.cpu(), 0
        for k, lo, hi in order:
            for p in range(lo, hi):
                got[k][p] = lg[at]; at += 1
    for k in range(4):
        assert rel_err(torch.stack(got[k]), refs[k]) < TOL, f"sequence {k}"


def case_blocks_and_rows_reused(make, cfg, seed=4):
    """A pool that only fits the live requests: blocks and block-table rows of finished requests are handed out again, in
    another order, while they still hold the old rows."""
    t = oracle_of(cfg).random_tensors(cfg, seed=seed)
    model = make_worker(make, cfg, t, block_size=4, num_blocks=12, rows=2)
    a, b, c = tokens_for(cfg, 22, 40), tokens_for(cfg, 17, 41), tokens_for(cfg, 26, 42)
    ra, rb, rc = (oracle_of(cfg).forward(cfg, t, s) for s in (a, b, c))
    ga = run_portions(model, a, 0, [10, 12])                 # 6 blocks
    gb = run_portions(model, b, 1, [17])                     # 5 blocks: 1 left
    assert model.gpu_block_manager.num_free_blocks == 1
    model.free_seqs_resources([0])
    gc = run_portions(model, c, 0, [3, 1, 1, 21])            # 7 blocks: a's six and the spare, row 0 again
    assert model.gpu_block_manager.num_free_blocks == 0
    model.free_seqs_resources([1])
    ga2 = run_portions(model, a[:20], 1, [20])               # b's blocks and row
    for got, ref in ((ga, ra), (gb, rb), (gc, rc), (ga2, ra[:20])):
        assert rel_err(got, ref) < TOL


def case_long_decode(make, cfg, seed=5, n=60):
    t = oracle_of(cfg).random_tensors(cfg, seed=seed)
    toks = tokens_for(cfg, n, seed)
    ref = oracle_of(cfg).forward(cfg, t, toks)
    model = make_worker(make, cfg, t, block_size=8, num_blocks=8)
    got = run_portions(model, toks, 3, [2] + [1] * (n - 2))
    assert rel_err(got, ref) < TOL
    assert rel_err(got[-1], ref[-1]) < TOL


def oracle_greedy(cfg, t, prompt, new_tokens):
    toks, out = list(prompt), []
    for _ in range(new_tokens):
        nxt = int(torch.argmax(oracle_of(cfg).forward(cfg, t, toks)[-1]))
        out.append(nxt); toks.append(nxt)
    return out


def case_greedy_generation(make, cfg, seed=6):
    """Through the worker's scheduler loop (worker/chunking.py: prompts in portions beside running decodes)."""
    from swiftllm_b200.worker.chunking import run_greedy
    # sharpen the head so that greedy choices do not hinge on rounding
    t = oracle_of(cfg).random_tensors(cfg, seed=seed)
    t["head"] = (t["head"].float() * 4).to(t["head"].dtype)
    prompts = [tokens_for(cfg, n, 60 + k) for k, n in enumerate((11, 3, 17))]
    model = make_worker(make, cfg, t, block_size=4, num_blocks=30, rows=4)
    got = run_greedy(model, prompts, new_tokens=5, max_tokens_in_step=9, max_chunk=6, seq_ids=[2, 0, 3])
    assert got == [oracle_greedy(cfg, t, p, 5) for p in prompts]
    assert model.gpu_block_manager.num_free_blocks == 30

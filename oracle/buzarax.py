"""Plain, slow restatement of the Buzarax design, one function per mechanism.

TEST INFRASTRUCTURE ONLY: shares no code with `swiftllm_b200/`.  Everything is computed per sequence, over the whole sequence at
once, in one floating-point type (float32 or float64), token by token where the rule is a recurrence.

The design.  A decoder-only model on a residual stream x [n, width]:
  * embedding: token row + a row of a hashed table of (previous token, token) pairs;
  * layers of two kinds of mixer, each followed by an optional feed-forward; BOTH sublayers read x itself and their OUTPUT is
    normalised (RMS norm with ONE scalar gain) before it is added:  x <- x + g1 * rms(mixer(x)),  x <- x + g2 * rms(ff(x));
  * after layer i the stream that goes on is a learned weighted sum of the embedding output and the results of layers 0 .. i;
  * mixer "rglru": a gated linear recurrence per channel behind a short causal convolution, times a GELU branch;
  * mixer "parallel": softmax attention with grouped key/value heads (rotary with stretched frequencies on the first entries
    of a head, unit-RMS queries and keys, values turned by their own position and the output turned back, a capped score, one
    extra 1 in the softmax denominator) BESIDE a linear attention with a constant decay per head, a group norm and a sigmoid gate;
  * feed-forwards: a clamped gated linear unit, or a mixture of SiLU-gated experts chosen by sigmoid scores plus a bias that
    only takes part in the choice;
  * output: scalar-gain RMS norm, head, tanh cap of the logits.
"""
from __future__ import annotations

import math

import torch

GATE_SLOPE = 1.702          # slope of the sigmoid in the clamped gated linear unit
RGLRU_C = 8.0               # log a = -RGLRU_C * r * softplus(lam)


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


# ---------------------------------------------------------------- small pieces
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def tanh_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


# ---------------------------------------------------------------- embedding
def bigram_rows(tokens, e: dict) -> list:
    """Row of the pair table for every token: (previous * mul_prev + token * mul_cur) mod buckets; the first token of a sequence
    has no previous one and takes the table's extra last row."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(e["buckets"] if i == 0 else (tokens[i - 1] * e["mul_prev"] + t * e["mul_cur"]) % e["buckets"])
    return rows


def embed(tokens, tensors: dict, config: dict) -> torch.Tensor:
    x = tensors["embed"][torch.tensor(tokens)]
    e = (config.get("embedding") or {}).get("bigram")
    if e:
        x = x + tensors["bigram"][torch.tensor(bigram_rows(tokens, e))]
    return x


# ---------------------------------------------------------------- rotations
def stretched_frequencies(rot: dict) -> tuple:
    """-> (frequency of every pair, factor on cos and sin).  Plain frequencies f_i = base^(-2i/dims); with `scaling`, pairs whose
    wavelength is long against the original context are slowed by `factor`, fast pairs are kept, with a linear ramp between."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_of(turns):         # the (fractional) pair index whose wavelength makes `turns` turns over the original context
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate_halves(v: torch.Tensor, positions, freqs, dims: int, amp: float = 1.0, sign: float = 1.0) -> torch.Tensor:
    """Entry i and entry i + dims/2 (i < dims/2) of the last axis of v [n, ..., d] turn together by the angle
    sign * p * freqs[i]; cos and sin are multiplied by amp; entries from `dims` on pass through."""
    out = v.clone()
    half = dims // 2
    for t, p in enumerate(positions):
        for i in range(half):
            a = sign * p * freqs[i]
            c, s = math.cos(a) * amp, math.sin(a) * amp
            u, w = v[t, ..., i].clone(), v[t, ..., i + half].clone()
            out[t, ..., i] = u * c - w * s
            out[t, ..., i + half] = w * c + u * s
    return out


# ---------------------------------------------------------------- mixers
def capped_sink_attention(h: torch.Tensor, positions, p: dict, m: dict, eps: float) -> torch.Tensor:
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    rot = m.get("rot") or {"base": 10000.0, "dims": 0}
    freqs, amp = stretched_frequencies(rot) if rot["dims"] else ([], 1.0)
    q = unit_rms(rotate_halves((h @ p["q"].T).reshape(n, H, dk), positions, freqs, rot["dims"], amp), eps)
    k = unit_rms(rotate_halves((h @ p["k"].T).reshape(n, G, dk), positions, freqs, rot["dims"], amp), eps)
    vfreq = [rot["base"] ** (-2.0 * i / dv) for i in range(dv // 2)]
    v = rotate_halves((h @ p["v"].T).reshape(n, G, dv), positions, vfreq, dv)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    cap = m.get("softcap")
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]                        # [n, n]
        if cap:
            s = tanh_cap(s, cap)
        for i in range(n):
            e = torch.exp(s[i, :i + 1])
            w = e / (1.0 + e.sum())                                     # the 1: a key of score 0 without a value
            out[i, hd] = w @ v[:i + 1, g]
    out = rotate_halves(out, positions, vfreq, dv, sign=-1.0)
    return out.reshape(n, H * dv) @ p["o"].T


def decayed_linear_attention(h: torch.Tensor, p: dict, m: dict, eps: float) -> torch.Tensor:
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q, k = silu(h @ p["q"].T).reshape(n, H, dk), silu(h @ p["k"].T).reshape(n, H, dk)
    v = silu(h @ p["v"].T).reshape(n, H, dv)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(n):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    y = unit_rms(out.reshape(n, H * dv), eps) * p["norm"]
    return (y * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


def parallel_mixer(h: torch.Tensor, positions, p: dict, m: dict, eps: float) -> torch.Tensor:
    left = capped_sink_attention(h, positions, sub(p, "left."), m["left"], eps)
    right = decayed_linear_attention(h, sub(p, "right."), m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Per channel c: y[t, c] = b[c] + sum_k w[c, K - 1 - k] * x[t - k, c], inputs before the start count as zero."""
    n, K = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(n):
        acc = b.clone()
        for k in range(K):
            if t - k >= 0:
                acc = acc + w[:, K - 1 - k] * x[t - k]
        y[t] = acc
    return y


def gated_linear_recurrence(h: torch.Tensor, p: dict, m: dict) -> torch.Tensor:
    n, C, B = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ p["y"].T + p["y.b"])
    u = causal_conv(h @ p["x"].T + p["x.b"], p["conv"], p["conv.b"])
    ub = u.reshape(n, B, C // B)
    r = torch.sigmoid(torch.einsum("boi,nbi->nbo", p["ra"], ub) + p["ra.b"]).reshape(n, C)
    i = torch.sigmoid(torch.einsum("boi,nbi->nbo", p["ri"], ub) + p["ri.b"]).reshape(n, C)
    log_a = -RGLRU_C * r * torch.nn.functional.softplus(p["lam"])
    a = torch.exp(log_a)
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.zeros(n, C, dtype=h.dtype)
    for t in range(n):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * (i[t] * u[t])
        out[t] = S
    return (out * y) @ p["o"].T


# ---------------------------------------------------------------- feed-forwards
def clamped_glu(h: torch.Tensor, p: dict, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ p["gate"].T, max=limit)
    u = torch.clamp(h @ p["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ p["down"].T


def silu_glu(h: torch.Tensor, p: dict) -> torch.Tensor:
    return (silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def sigmoid_route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int):
    """Per token: scores s = sigmoid(router h); the `top` experts with the largest s + correction are chosen; their weights
    are their plain scores s (no renormalisation)."""
    s = torch.sigmoid(h.float() @ router.float().T)
    idx, wts = [], []
    for t in range(s.shape[0]):
        choice = s[t] + correction.float()
        chosen = sorted(range(s.shape[1]), key=lambda e: (-float(choice[e]), e))[:top]
        idx.append(chosen)
        wts.append([s[t, e] for e in chosen])
    return idx, wts


def moe_ff(h: torch.Tensor, p: dict, f: dict) -> torch.Tensor:
    idx, wts = sigmoid_route(h, p["router"], p["correction"], f["router"]["top"])
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            out[t] += w.to(h.dtype) * silu_glu(h[t:t + 1], sub(p, f"e{e}."))[0]
    return out


# ---------------------------------------------------------------- the model
def forward(config: dict, tensors: dict, tokens, dtype=torch.float32, keep_layers: bool = False):
    """Logits [n, vocab] of one whole sequence (and the stream that leaves every layer, after the weighted sum over depth, when
    keep_layers)."""
    tensors = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    n = len(tokens)
    positions = list(range(n))
    x = embed(tokens, tensors, config)
    history, layers = [x], []
    for i, layer in enumerate(config["layers"]):
        p = sub(tensors, f"l{i}.")
        if layer["type"] == "rglru":
            y = gated_linear_recurrence(x, sub(p, "mix."), layer["mixer"])
        else:
            assert layer["type"] == "parallel", layer["type"]
            y = parallel_mixer(x, positions, sub(p, "mix."), layer["mixer"], eps)
        x = x + unit_rms(y, eps) * p["norm1"]
        f = layer.get("mlp")
        if f is not None:
            y = clamped_glu(x, sub(p, "mlp."), f["limit"]) if f["kind"] == "dense" else moe_ff(x, sub(p, "mlp."), f)
            x = x + unit_rms(y, eps) * p["norm2"]
        history.append(x)
        if "dwa" in p:
            x = sum(p["dwa"][j] * history[j] for j in range(i + 2))
        layers.append(x.clone())
    logits = (unit_rms(x, eps) * tensors["final.norm"]) @ tensors["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = tanh_cap(logits, cap)
    return (logits, torch.stack(layers)) if keep_layers else logits


# ---------------------------------------------------------------- random weights
def random_tensors(config: dict, seed: int = 0, std: float = 0.5, dtype=torch.bfloat16) -> dict:
    """Random weights with the design's tensor names and shapes."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * (gain * std / math.sqrt(i))).to(dtype)

    def vec(n, mean=0.0, dev=0.1):
        return (mean + dev * torch.randn(n, generator=g)).to(dtype)

    def scalar(mean=1.0):
        return (mean + 0.2 * torch.randn((), generator=g)).to(dtype)

    t = {"embed": torch.randn(config["vocab"], W, generator=g).to(dtype), "final.norm": scalar(), "head": lin(config["vocab"], W, 2.0)}
    e = (config.get("embedding") or {}).get("bigram")
    if e:
        t["bigram"] = (0.7 * torch.randn(e["buckets"] + 1, W, generator=g)).to(dtype)
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        t[p + "norm1"] = scalar()
        if layer["type"] == "rglru":
            C, B, K = m["width"], m["blocks"], m["conv"]
            t[p + "mix.y"], t[p + "mix.y.b"] = lin(C, W, 3.0), vec(C)
            t[p + "mix.x"], t[p + "mix.x.b"] = lin(C, W, 3.0), vec(C)
            t[p + "mix.conv"], t[p + "mix.conv.b"] = (0.5 * torch.randn(C, K, generator=g)).to(dtype), vec(C)
            for name in ("ra", "ri"):
                t[p + f"mix.{name}"] = (torch.randn(B, C // B, C // B, generator=g) * (2.0 / math.sqrt(C // B))).to(dtype)
                t[p + f"mix.{name}.b"] = vec(C, dev=0.5).reshape(B, C // B)
            t[p + "mix.lam"] = vec(C, mean=-2.0, dev=1.5)               # decays from fast to slow
            t[p + "mix.o"] = lin(W, C, 2.0)
        else:
            a, b = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            t[p + "mix.left.q"], t[p + "mix.left.k"] = lin(H * dk, W, 4.0), lin(G * dk, W, 4.0)
            t[p + "mix.left.v"], t[p + "mix.left.o"] = lin(G * dv, W, 2.0), lin(W, H * dv, 2.0)
            H, dk, dv = b["heads"], b["dim"], b["vdim"]
            t[p + "mix.right.q"], t[p + "mix.right.k"] = lin(H * dk, W, 2.0), lin(H * dk, W, 2.0)
            t[p + "mix.right.v"], t[p + "mix.right.g"] = lin(H * dv, W, 2.0), lin(H * dv, W, 2.0)
            t[p + "mix.right.o"], t[p + "mix.right.norm"] = lin(W, H * dv, 2.0), vec(H * dv, mean=1.0, dev=0.2)
        f = layer.get("mlp")
        if f is not None:
            t[p + "norm2"] = scalar()
            if f["kind"] == "dense":
                # gains large enough that the clamps bite for a good share of the entries
                t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = lin(f["ff"], W, 3.0), lin(f["ff"], W, 3.0), lin(W, f["ff"], 2.0)
            else:
                E, ff = f["router"]["experts"], f["expert"]["ff"]
                t[p + "mlp.router"], t[p + "mlp.correction"] = lin(E, W, 4.0), vec(E, dev=0.3)
                for e_ in range(E):
                    t[p + f"mlp.e{e_}.gate"], t[p + f"mlp.e{e_}.up"] = lin(ff, W, 3.0), lin(ff, W, 3.0)
                    t[p + f"mlp.e{e_}.down"] = lin(W, ff, 2.0)
        t[p + "dwa"] = (torch.softmax(torch.randn(i + 2, generator=g), 0) * 1.2).to(dtype)
    return t

"""Plain, slow restatement of the Naforax design, one function per mechanism.

TEST INFRASTRUCTURE ONLY: shares no code with `swiftllm_b200/`.  Everything is computed per sequence, over the whole sequence at
once, in one floating-point type (float32 or float64), token by token where the rule is a recurrence.

The design.  A decoder-only model on a residual stream x [n, width]:
  * embedding: x = embed[token]; this x is also re-injected at the start of every repeated pass;
  * a list of layers of which a range [start, stop) runs `times` times in a row with the same weights (every pass with its own
    keys / values and recurrent state); before every pass but the first the embedding output is added to x, and before every pass
    the pass's row of the table `loop.step` is added;
  * a layer:  x <- x + m * norm1b(mixer(c1(norm1(x)))),  x <- x + m * norm2b(ff(c2(norm2(x))))  with m a constant, every norm
    an RMS norm over equal consecutive groups of the vector with one weight vector, and c(h) = h + causal per-channel
    convolution of h over time;
  * mixer "attention": two softmax attentions ("maps") per head over the same values, whose outputs are subtracted with a
    learned factor, normalised over the head, gated by a sigmoid of a projection; per-head RMS norm (with weight) of queries and
    keys, then rotary on the leading entries of every map in interleaved pairs; a query sees earlier keys of its own chunk of
    `mask.size` positions only;
  * mixer "mingru": S <- (1 - z) S + z c per channel with z, c functions of the current token only; output gated by a SiLU;
  * mixer "mamba1": a selective state-space scan behind a causal convolution with SiLU;
  * feed-forwards: a GELU (tanh form) gated linear unit, or a mixture of clamped-GLU experts chosen by the largest softmax scores
    (weights: those scores, not renormalised) plus a shared expert with a per-token sigmoid gate;
  * output: group RMS norm, head, tanh cap of the logits.
"""
from __future__ import annotations

import math

import torch

GATE_SLOPE = 1.702          # slope of the sigmoid in the clamped gated linear unit


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


# ---------------------------------------------------------------- small pieces
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last axis in `groups` equal consecutive parts, each divided by its own root mean square; then times w."""
    n = x.shape[-1]
    parts = x.reshape(x.shape[:-1] + (groups, n // groups))
    return unit_rms(parts, eps).reshape(x.shape) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def tanh_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def causal_conv(x: torch.Tensor, w: torch.Tensor, b=None) -> torch.Tensor:
    """x [n, C], w [C, taps] (last column: the current token): out_t = sum_j w[:, j] x_(t - taps + 1 + j) (+ b), zeros before 0."""
    n, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * x[s]
        if b is not None:
            out[t] += b
    return out


def input_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """What a sublayer reads: its normed input plus that input's causal convolution."""
    return h + causal_conv(h, w)


# ---------------------------------------------------------------- attention
def rotate_pairs(v: torch.Tensor, positions, base: float, dims: int) -> torch.Tensor:
    """v [n, ..., d]: entries (2i, 2i + 1), i < dims / 2, turn by position * base^(-2i / dims); the rest pass."""
    out = v.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            x, y = v[t, ..., 2 * i].clone(), v[t, ..., 2 * i + 1].clone()
            out[t, ..., 2 * i] = x * c - y * s
            out[t, ..., 2 * i + 1] = y * c + x * s
    return out


def differential_factor(p: dict, diff: float) -> float:
    return float(torch.exp((p["lq1"] * p["lk1"]).sum()) - torch.exp((p["lq2"] * p["lk2"]).sum()) + diff)


def differential_attention(h: torch.Tensor, positions, p: dict, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).reshape(n, H, 2, dk)
    k = (h @ p["k"].T + p["k.b"]).reshape(n, G, 2, dk)
    v = (h @ p["v"].T + p["v.b"]).reshape(n, G, dv)
    q = unit_rms(q, eps) * p["q.norm"]
    k = unit_rms(k, eps) * p["k.norm"]
    rot = m.get("rot") or {}
    if rot.get("dims", 0) > 0:
        q = rotate_pairs(q, positions, rot["base"], rot["dims"])
        k = rotate_pairs(k, positions, rot["base"], rot["dims"])
    chunk = (m.get("mask") or {}).get("size", 0)
    lam = differential_factor(p, m["diff"])
    pos = torch.tensor(positions)
    visible = pos[None, :] <= pos[:, None]
    if chunk > 0:
        visible = visible & ((pos[None, :] // chunk) == (pos[:, None] // chunk))
    out = torch.zeros((n, H, dv), dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        maps = []
        for mp in range(2):
            s = (q[:, hh, mp] @ k[:, g, mp].T) * m["scale"]                 # [query, key]
            w = torch.softmax(s.masked_fill(~visible, -math.inf), dim=1)
            maps.append(w @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, hh] = unit_rms(o, eps) * (1.0 - m["diff"])
    gate = torch.sigmoid(h @ p["g"].T)
    return (out.reshape(n, H * dv) * gate) @ p["o"].T + p["o.b"]


# ---------------------------------------------------------------- recurrences
def min_gru(h: torch.Tensor, p: dict, m: dict) -> torch.Tensor:
    n = h.shape[0]
    z = torch.sigmoid(h @ p["z"].T + p["z.b"])
    u = h @ p["x"].T + p["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(m["width"], dtype=h.dtype)
    states = []
    for t in range(n):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        states.append(S)
    return (torch.stack(states) * silu(h @ p["g"].T)) @ p["o"].T


def selective_scan(h: torch.Tensor, p: dict, m: dict) -> torch.Tensor:
    n, C, N, R = h.shape[0], m["inner"], m["state"], m["dt_rank"]
    xz = h @ p["in"].T
    x, z = xz[:, :C], xz[:, C:]
    x = silu(causal_conv(x, p["conv"], p["conv.b"]))
    proj = x @ p["x"].T
    dt, B, Cm = proj[:, :R], proj[:, R:R + N], proj[:, R + N:]
    dt = softplus(dt @ p["dt"].T + p["dt.b"])                  # [n, C]
    A = -torch.exp(p["A_log"])                                  # [C, N]
    S = torch.zeros((C, N), dtype=h.dtype)
    ys = []
    for t in range(n):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append((S * Cm[t][None, :]).sum(dim=1) + p["D"] * x[t])
    return (torch.stack(ys) * silu(z)) @ p["o"].T


# ---------------------------------------------------------------- feed-forwards
def gelu_glu(h: torch.Tensor, p: dict) -> torch.Tensor:
    return (gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def clamped_glu(h: torch.Tensor, p: dict, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ p["gate"].T, max=limit)
    u = torch.clamp(h @ p["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ p["down"].T


def softmax_route(h: torch.Tensor, router: torch.Tensor, top: int):
    """-> (chosen experts [n, top], their softmax scores [n, top]); ties go to the lower index."""
    s = torch.softmax(h @ router.T, dim=-1)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def moe_ff(h: torch.Tensor, p: dict, f: dict) -> torch.Tensor:
    chosen, weights = softmax_route(h, p["router"], f["router"]["top"])
    out = torch.zeros((h.shape[0], p["e0.down"].shape[0]), dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            out[t] += w * clamped_glu(h[t:t + 1], sub(p, f"e{e}."), f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + torch.sigmoid(h @ p["shared.sg"].T) * clamped_glu(h, sub(p, "shared."), f["shared"]["limit"])
    return out


# ---------------------------------------------------------------- the model
def layer_runs(config: dict) -> list:
    """-> [(layer, pass)] in the order the layers run; layers outside the repeated range have pass 0."""
    L = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, 0) for i in range(L)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return [(i, 0) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + [(i, 0) for i in range(b, L)]


def forward(config: dict, tensors: dict, tokens, dtype=torch.float32, keep_layers: bool = False):
    """-> logits [n, vocab] (and the stream after every layer run, [runs, n, width])."""
    tens = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, groups, mult = config["norm"]["eps"], config["norm"].get("groups", 1), config.get("residual_mult", 1.0)
    positions = list(range(len(tokens)))
    x = tens["embed"][torch.tensor(tokens, dtype=torch.long)]
    x0 = x.clone()
    loop = config.get("loop")
    kept = []
    for i, t in layer_runs(config):
        layer, p = config["layers"][i], sub(tens, f"l{i}.")
        if loop and i == loop["start"]:
            if t > 0:
                x = x + x0
            x = x + tens["loop.step"][t]
        h = input_conv(group_norm(x, p["norm1"], groups, eps), p["canon1"])
        mp, m = sub(p, "mix."), layer["mixer"]
        if layer["type"] == "attention":
            y = differential_attention(h, positions, mp, m, eps)
        elif layer["type"] == "mingru":
            y = min_gru(h, mp, m)
        else:
            assert layer["type"] == "mamba1"
            y = selective_scan(h, mp, m)
        x = x + mult * group_norm(y, p["norm1b"], groups, eps)
        f = layer.get("mlp")
        if f is not None:
            h = input_conv(group_norm(x, p["norm2"], groups, eps), p["canon2"])
            y = gelu_glu(h, sub(p, "mlp.")) if f["kind"] == "dense" else moe_ff(h, sub(p, "mlp."), f)
            x = x + mult * group_norm(y, p["norm2b"], groups, eps)
        kept.append(x.clone())
    logits = group_norm(x, tens["final.norm"], groups, eps) @ tens["head"].T
    cap = config.get("logit_softcap") or 0.0
    if cap > 0:
        logits = tanh_cap(logits, cap)
    return (logits, torch.stack(kept)) if keep_layers else logits


def tensor_shapes(config: dict) -> dict:
    """name -> shape of every tensor of a checkpoint of this configuration."""
    W, V = config["width"], config["vocab"]
    taps = config["canon"]["taps"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if config.get("loop"):
        out["loop.step"] = (config["loop"]["times"], W)
    for i, layer in enumerate(config["layers"]):
        m, f, pre = layer["mixer"], layer.get("mlp"), f"l{i}."
        for nm in ("norm1", "norm1b"):
            out[pre + nm] = (W,)
        out[pre + "canon1"] = (W, taps)
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
            out.update({pre + "mix.q": (H * 2 * dk, W), pre + "mix.q.b": (H * 2 * dk,), pre + "mix.k": (G * 2 * dk, W),
                        pre + "mix.k.b": (G * 2 * dk,), pre + "mix.v": (G * dv, W), pre + "mix.v.b": (G * dv,),
                        pre + "mix.q.norm": (dk,), pre + "mix.k.norm": (dk,), pre + "mix.lq1": (dk,), pre + "mix.lk1": (dk,),
                        pre + "mix.lq2": (dk,), pre + "mix.lk2": (dk,), pre + "mix.g": (H * dv, W), pre + "mix.o": (W, H * dv),
                        pre + "mix.o.b": (W,)})
        elif layer["type"] == "mingru":
            C = m["width"]
            out.update({pre + "mix.z": (C, W), pre + "mix.z.b": (C,), pre + "mix.x": (C, W), pre + "mix.x.b": (C,),
                        pre + "mix.g": (C, W), pre + "mix.o": (W, C)})
        else:
            C, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            out.update({pre + "mix.in": (2 * C, W), pre + "mix.conv": (C, K), pre + "mix.conv.b": (C,), pre + "mix.x": (R + 2 * N, C),
                        pre + "mix.dt": (C, R), pre + "mix.dt.b": (C,), pre + "mix.A_log": (C, N), pre + "mix.D": (C,),
                        pre + "mix.o": (W, C)})
        if f is None:
            continue
        for nm in ("norm2", "norm2b"):
            out[pre + nm] = (W,)
        out[pre + "canon2"] = (W, taps)
        if f["kind"] == "dense":
            out.update({pre + "mlp.gate": (f["ff"], W), pre + "mlp.up": (f["ff"], W), pre + "mlp.down": (W, f["ff"])})
        else:
            names = [(f"e{e}", f["expert"]["ff"]) for e in range(f["router"]["experts"])]
            if f.get("shared"):
                names.append(("shared", f["shared"]["ff"]))
                out[pre + "mlp.shared.sg"] = (1, W)
            out[pre + "mlp.router"] = (f["router"]["experts"], W)
            for nm, ff in names:
                out.update({pre + f"mlp.{nm}.gate": (ff, W), pre + f"mlp.{nm}.up": (ff, W), pre + f"mlp.{nm}.down": (W, ff)})
    return out


def random_tensors(config: dict, seed: int = 0, std: float = 0.5, dtype=torch.bfloat16) -> dict:
    """Random weights for tests: projections N(0, std / sqrt(fan-in)) so that every mechanism contributes, norm weights around 1,
    A_log around log(1 .. state), step biases around softplus^-1 of small steps."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if leaf.endswith(("norm1", "norm2", "norm1b", "norm2b", ".norm")) or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "mix.A_log":
            t = torch.log(1.0 + torch.rand(shape, generator=g) * (shape[1] - 1))
        elif leaf == "mix.dt.b":
            t = -2.0 + torch.randn(shape, generator=g)
        elif leaf in ("mix.D",):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif leaf in ("mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf in ("canon1", "canon2", "mix.conv"):
            t = 0.4 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
        elif name in ("embed", "loop.step"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (std * 2.0 / math.sqrt(shape[-1]))
        out[name] = t.to(dtype)
    return out

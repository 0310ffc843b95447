"""Plain, slow restatement of the Rivudra design (a decoder-only model whose layers are PARALLEL blocks: one RMS norm with a
weight stored around zero feeds a gated sliding-window attention mixer and a mixture-of-experts feed-forward, and both are added
to the residual), one function per mechanism.

TEST INFRASTRUCTURE ONLY: shares no code with `swiftllm_b200/`.  Everything is computed per sequence, over the whole sequence at
once, in float32 (or float64), with explicit loops where a loop is the clearest statement of the rule.

Notation.  x: residual [n, width]; h = norm(x); per mixer: H query heads, G key/value heads, dk query/key and dv value entries per
head, w window; per feed-forward: E experts in groups, `top` of them per token.
"""
from __future__ import annotations

import math

import torch

GATE_SLOPE = 1.702
RENORM_EPS = 1e-20


def offset_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * (1 + weight)   (eps under the root; the weight is stored around zero)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (1.0 + weight.to(x.dtype))


def rotate_pairs(v: torch.Tensor, positions, base: float, dims: int) -> torch.Tensor:
    """Interleaved rotary embedding: entries (2i, 2i+1), i < dims/2, of the last axis of v [n, ..., d] turn by the angle
    p * base^(-2i/dims) for the token at position p; entries from `dims` on pass through."""
    out = v.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, w = v[t, ..., 2 * i].clone(), v[t, ..., 2 * i + 1].clone()
            out[t, ..., 2 * i] = u * c - w * s
            out[t, ..., 2 * i + 1] = w * c + u * s
    return out


def window_visible(i: int, j: int, window: int) -> bool:
    """Query position i sees key position j iff 0 <= i - j < window (itself and the window - 1 positions before it)."""
    return 0 <= i - j < window


def sink_softmax(s: torch.Tensor) -> torch.Tensor:
    """p_j = exp(s_j) / (1 + sum_j exp(s_j)): a softmax with one more key of score 0 that has no value."""
    m = torch.clamp(s.max(), min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum())


def gated_window_attention(h: torch.Tensor, positions, p: dict, m: dict) -> torch.Tensor:
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    q = rotate_pairs((h @ p["q"].T).reshape(n, H, dk), positions, rot["base"], rot["dims"])
    k = rotate_pairs((h @ p["k"].T).reshape(n, G, dk), positions, rot["base"], rot["dims"])
    v = (h @ p["v"].T).reshape(n, G, dv)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for i in range(n):
        js = [j for j in range(n) if window_visible(positions[i], positions[j], m["mask"]["size"])]
        for hd in range(H):
            g = hd // (H // G)
            s = torch.stack([(q[i, hd] @ k[j, g]) * m["scale"] for j in js])
            w = sink_softmax(s)
            out[i, hd] = sum(w[a] * v[j, g] for a, j in enumerate(js))
    gate = torch.sigmoid(h @ p["g"].T)                               # [n, H * dv], element by element
    return (out.reshape(n, H * dv) * gate) @ p["o"].T


def clamped_glu_expert(h: torch.Tensor, p: dict, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ p["gate"].T, max=limit)
    u = torch.clamp(h @ p["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ p["down"].T


def route(h: torch.Tensor, router: torch.Tensor, r: dict):
    """Per token: scores = softmax over all experts; experts of the best `keep` groups (a group's score: its largest score) may
    be chosen, the `top` largest of those are; weights = chosen scores / (their sum + 1e-20) * scale."""
    z = h.float() @ router.float().T
    s = torch.softmax(z, dim=-1)
    E = s.shape[1]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = E // groups["count"]
    idx, wts = [], []
    for t in range(s.shape[0]):
        gscore = [float(s[t, g * per:(g + 1) * per].max()) for g in range(groups["count"])]
        kept = sorted(range(groups["count"]), key=lambda g: (-gscore[g], g))[:groups["keep"]]
        allowed = [e for e in range(E) if e // per in kept]
        chosen = sorted(allowed, key=lambda e: (-float(s[t, e]), e))[:r["top"]]
        w = torch.stack([s[t, e] for e in chosen])
        idx.append(chosen)
        wts.append(w / (w.sum() + RENORM_EPS) * r.get("scale", 1.0))
    return idx, wts


def moe_ff(h: torch.Tensor, p: dict, f: dict) -> torch.Tensor:
    idx, wts = route(h, p["router"], f["router"])
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            out[t] += w.to(h.dtype) * clamped_glu_expert(h[t:t + 1], sub(p, f"e{e}."), f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + clamped_glu_expert(h, sub(p, "shared."), f["shared"]["limit"])
    return out


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens, dtype=torch.float32, keep_layers: bool = False):
    """Logits [n, vocab] of one whole sequence (and the residual after every layer when keep_layers)."""
    tensors = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    n = len(tokens)
    positions = list(range(n))
    x = tensors["embed"][torch.tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    layers = []
    for i, layer in enumerate(config["layers"]):
        assert layer["type"] == "attention"
        h = offset_rms_norm(x, tensors[f"l{i}.norm1"], eps)
        y = gated_window_attention(h, positions, sub(tensors, f"l{i}.mix."), layer["mixer"])
        if layer.get("mlp") is not None:
            y = y + moe_ff(h, sub(tensors, f"l{i}.mlp."), layer["mlp"])
        x = x + y
        layers.append(x.clone())
    logits = offset_rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    return (logits, torch.stack(layers)) if keep_layers else logits


def random_tensors(config: dict, seed: int = 0, std: float = 0.5, dtype=torch.bfloat16) -> dict:
    """Random weights with the design's tensor names and shapes; projections ~ N(0, std / sqrt(fan_in)), norms ~ N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * (gain * std / math.sqrt(i))).to(dtype)

    def nrm(n):
        return (0.1 * torch.randn(n, generator=g)).to(dtype)

    t = {"embed": torch.randn(config["vocab"], W, generator=g).to(dtype), "final.norm": nrm(W), "head": lin(config["vocab"], W, 2.0)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = nrm(W)
        t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = lin(H * dk, W, 4.0), lin(G * dk, W, 4.0), lin(G * dv, W, 2.0)
        t[p + "mix.g"], t[p + "mix.o"] = lin(H * dv, W, 2.0), lin(W, H * dv, 2.0)
        f = layer.get("mlp")
        if f is None:
            continue
        t[p + "mlp.router"] = lin(f["router"]["experts"], W, 4.0)
        names = [(f"e{e}", f["expert"]["ff"]) for e in range(f["router"]["experts"])]
        if f.get("shared"):
            names.append(("shared", f["shared"]["ff"]))
        for name, ff in names:
            # gains large enough that the clamps bite for a good share of the entries
            t[p + f"mlp.{name}.gate"], t[p + f"mlp.{name}.up"] = lin(ff, W, 3.0), lin(ff, W, 3.0)
            t[p + f"mlp.{name}.down"] = lin(W, ff, 2.0)
    return t

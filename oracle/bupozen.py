"""Plain, slow restatement of the Bupozen design (a decoder-only model whose layers are PARALLEL blocks: one RMS norm feeds a
latent-attention mixer and a feed-forward, and both are added to the residual), one function per mechanism.

TEST INFRASTRUCTURE ONLY: shares no code with `swiftllm_b200/`.  Everything is computed per sequence, over the whole
sequence at once, in float32 (or float64) with explicit loops where a loop is the clearest statement of the rule.

Notation.  x: residual [n, width]; h = norm(x); per mixer: H heads, dn = unrotated and dr = rotated query/key size per head,
dv value size, r latent size, w window.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * weight   (eps under the root)."""
    x = x.to(weight.dtype) if weight.dtype == torch.float64 else x.float()
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype)


def rotate_pairs(v: torch.Tensor, positions, base: float, dims: int) -> torch.Tensor:
    """Interleaved rotary embedding of the first `dims` entries of the last axis of v [n, ..., d]: entries (2i, 2i+1) of the
    token at position p turn by the angle p * base^(-2i/dims); entries from `dims` on pass through."""
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
    """Query position i sees key position j iff 0 <= i - j < window."""
    return 0 <= i - j < window


def latent_kv(h: torch.Tensor, positions, p: dict, m: dict, eps: float):
    """What a latent-attention layer caches for its tokens: the normed latent c [n, r] and the shared rotated key part [n, dr]."""
    r, dr = m["kv_rank"], m["rot_dim"]
    d = h @ p["dkv"].T
    c = rms_norm(d[:, :r], p["dkv.norm"], eps)
    kr = rotate_pairs(d[:, r:r + dr], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h: torch.Tensor, positions, p: dict, m: dict, eps: float, c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    """The mixer's output for the tokens h [n, width] of ONE sequence at `positions` (0..n-1 here), given the latents c and
    rotated key parts kr of the same positions (its own or the ones of the layer named by `kv_from`)."""
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = h.shape[0]
    cq = rms_norm(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).reshape(n, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate_pairs(q[..., dn:], positions, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ p["uk"].T).reshape(n, H, dn)
    v = (c @ p["uv"].T).reshape(n, H, dv)
    gate = torch.sigmoid(h @ p["g"].T)                                # [n, H]
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for i in range(n):
        js = [j for j in range(n) if window_visible(positions[i], positions[j], m["mask"]["size"])]
        for hd in range(H):
            s = torch.stack([(qn[i, hd] @ kn[j, hd] + qr[i, hd] @ kr[j]) * m["scale"] for j in js])
            w = torch.softmax(s, dim=0)
            out[i, hd] = sum(w[k] * v[j, hd] for k, j in enumerate(js)) * gate[i, hd]
    return out.reshape(n, H * dv) @ p["o"].T


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def dense_ff(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return relu_squared(h @ up.T) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, top: int):
    """Per token: the `top` experts with the largest router logits and softmax weights over those logits only."""
    z = h.float() @ router.float().T
    vals, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(vals, dim=-1)


def moe_ff(h: torch.Tensor, p: dict, top: int) -> torch.Tensor:
    idx, w = route(h, p["router"], top)
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += w[t, k].to(h.dtype) * dense_ff(h[t:t + 1], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    return out


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens, dtype=torch.float32, keep_layers: bool = False):
    """Logits [n, vocab] of one whole sequence (and the residual after every layer when keep_layers)."""
    tensors = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    n = len(tokens)
    positions = list(range(n))
    x = tensors["embed"][torch.tensor(tokens)]
    held, layers = {}, []
    for i, layer in enumerate(config["layers"]):
        assert layer["type"] == "latent_attention"
        m = layer["mixer"]
        h = rms_norm(x, tensors[f"l{i}.norm1"], eps)
        pm = sub(tensors, f"l{i}.mix.")
        if "kv_from" in m and m["kv_from"] is not None:
            c, kr = held[m["kv_from"]]
        else:
            c, kr = held[i] = latent_kv(h, positions, pm, m, eps)
        y = latent_attention(h, positions, pm, m, eps, c, kr)
        ff = layer.get("mlp")
        if ff is not None:
            pf = sub(tensors, f"l{i}.mlp.")
            if ff["kind"] == "dense":
                y = y + dense_ff(h, pf["up"], pf["down"])
            else:
                y = y + moe_ff(h, pf, ff["router"]["top"])
        x = x + y
        layers.append(x.clone())
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    return (logits, torch.stack(layers)) if keep_layers else logits


def random_tensors(config: dict, seed: int = 0, std: float = 0.5, dtype=torch.bfloat16) -> dict:
    """Random weights with the design's tensor names and shapes; projections ~ N(0, std / sqrt(fan_in))."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * (gain * std / math.sqrt(i))).to(dtype)

    def nrm(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)

    t = {"embed": torch.randn(config["vocab"], W, generator=g).to(dtype), "final.norm": nrm(W), "head": lin(config["vocab"], W, 2.0)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, dn, dr, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        t[p + "norm1"] = nrm(W)
        t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = lin(qr, W, 2.0), nrm(qr), lin(H * (dn + dr), qr, 4.0)
        if m.get("kv_from") is None:
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = lin(r + dr, W, 2.0), nrm(r)
        t[p + "mix.uk"], t[p + "mix.uv"] = lin(H * dn, r, 4.0), lin(H * dv, r, 2.0)
        t[p + "mix.g"], t[p + "mix.o"] = lin(H, W, 2.0), lin(W, H * dv, 2.0)
        ff = layer.get("mlp")
        if ff is None:
            continue
        if ff["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"] = lin(ff["ff"], W, 2.0), lin(W, ff["ff"], 2.0)
        else:
            t[p + "mlp.router"] = lin(ff["router"]["experts"], W, 4.0)
            for e in range(ff["router"]["experts"]):
                t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = lin(ff["expert"]["ff"], W, 2.0), lin(W, ff["expert"]["ff"], 2.0)
    return t

"""Configurations and scenarios for the Rivudra worker (swiftllm_b200.worker.rivudra_model) against the plain restatement of the
design in oracle/rivudra.py.  The schedule scenarios (whole prompts, decoding, portions, mixed batches, reused blocks and rows,
greedy generation) are the ones of tests/bupozen_cases.py; here are the design's own configurations and the scenarios whose
weights are made so that one particular fault would show.  They run on the CPU (kernels replaced by tests/cpu_shim.py) and on a
GPU (the CUDA kernels): tests/test_rivudra_cpu.py and tests/test_rivudra_gpu.py call them with the `make` factory of their world.

All configurations are small and deliberately irregular: head sizes that are not multiples of 32 or of each other, value size
different from the key size, rotary on a part of a head, one / several / as many key-value heads as query heads, layers of
different cache row widths, a layer without feed-forward, one group / all groups kept / fewer, top-1, with and without a shared
expert, limits that differ between the routed and the shared experts."""
import math

import torch

from bupozen_cases import TOL, make_worker, rel_err, run_portions, tokens_for
from oracle import rivudra as O


def mixer(heads=6, kv_heads=2, dim=10, vdim=7, window=7, base=100.0, dims=6, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
            "rot": {"base": base, "dims": dims}, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}


def moe(experts=6, top=2, ff=12, limit=0.75, groups=3, keep=2, scale=1.25, shared=(9, 1.5)):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
    if shared is not None:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def config(layers, width=48, vocab=97, eps=1e-5, embed_scale=0.7):
    return {"architecture": "Rivudra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "layers": [{"type": "attention", "mixer": m, "mlp": f} for m, f in layers]}


def full_config():
    """Every branch at once."""
    return config([
        (mixer(), moe()),
        (mixer(heads=4, kv_heads=4, dim=8, vdim=12, window=5, dims=8), moe(experts=8, top=3, groups=2, keep=1, shared=None)),
        (mixer(heads=11, kv_heads=1, dim=6, vdim=40, window=13, dims=2), None),       # another row width, 11 heads on one kv head
        (mixer(window=3, dims=0), moe(experts=5, top=1, groups=1, keep=1, scale=1.0)),  # same row width as layer 0, no rotary
        (mixer(heads=9, kv_heads=3, dim=12, vdim=5, window=64, dims=12), moe(experts=33, top=4, ff=8, groups=11, keep=4)),
    ])


SINGLE = {
    "moe": config([(mixer(), moe())]),
    "no_ff": config([(mixer(), None)]),
    "top1_one_group": config([(mixer(), moe(experts=3, top=1, groups=1, keep=1))]),
    "all_groups_kept": config([(mixer(), moe(experts=8, top=3, groups=4, keep=4, shared=None))]),
    "one_group_kept": config([(mixer(), moe(experts=12, top=2, groups=4, keep=1))]),
    "mha_window1": config([(mixer(heads=3, kv_heads=3, window=1), moe())]),
    "mqa_wide_value": config([(mixer(heads=5, kv_heads=1, dim=4, vdim=70, dims=4, window=9), moe())]),
    "no_rotary": config([(mixer(dims=0), moe())]),
    "unit_scales": config([(mixer(scale=1.0), moe(scale=1.0))], embed_scale=1.0),
}


# ---------------------------------------------------------------- scenarios made so that one fault shows
def _one_layer_probe(window, n, key_pos, H=2, dk=8, dv=6, width=16, vocab=32):
    """One attention-only layer whose weights make every query score ~0 against every key except the key at `key_pos`, which
    scores high, and whose value alone is large: the logits at a query position tell at once whether that key was seen."""
    cfg = config([(mixer(heads=H, kv_heads=1, dim=dk, vdim=dv, window=window, dims=0, scale=1.0), None)], width=width, vocab=vocab,
                 embed_scale=1.0)
    t = O.random_tensors(cfg, seed=11, dtype=torch.float32)
    # token `1` marks the special key: its embedding has a large entry in a dimension that no other token uses
    t["embed"] = torch.randn(vocab, width, generator=torch.Generator().manual_seed(1)) * 0.1
    t["embed"][:, 0] = 1.0                       # every query reads this constant ...
    t["embed"][:, 1] = 0.0
    t["embed"][1, 1] = 4.0                       # ... and only the marked token carries this
    t["l0.norm1"] = torch.zeros(width)
    q = torch.zeros(H * dk, width); q[:, 0] = 2.0
    k = torch.zeros(dk, width); k[:, 1] = 2.0    # only the marked key has a non-zero key
    v = torch.zeros(dv, width); v[:, 1] = 3.0    # and a large value
    t["l0.mix.q"], t["l0.mix.k"], t["l0.mix.v"] = q, k, v
    toks = [2 + (i % (vocab - 2)) for i in range(n)]
    toks[key_pos] = 1
    return cfg, t, toks


def case_window_edges(make, cuts_of=lambda n: [n]):
    """A marked key just inside and just outside the window of the last position, in a prompt and when decoding, with the window
    crossing block borders; the first positions of a sequence (windows that are not full yet)."""
    for window in (5, 8, 9):
        for n in (window + 7,):
            for back in (window - 1, window):                       # distance of the marked key from the last position
                cfg, t, toks = _one_layer_probe(window, n, n - 1 - back)
                ref = O.forward(cfg, t, toks)
                seen = O.forward(cfg, t, toks[n - 1 - back:])[-1]    # the marked key first in a sequence of its own
                # the oracle itself tells the two apart: inside the window the marked value dominates the last position
                inside = back < window
                for cuts in (cuts_of(n), [n - 1, 1], [2] + [1] * (n - 2), [n - 3, 2, 1]):
                    model = make_worker(make, cfg, t, block_size=4, num_blocks=16)
                    got = run_portions(model, toks, 1, cuts)
                    assert rel_err(got, ref) < TOL, (window, back, cuts)
                    # the difference between "seen" and "not seen" is far above the tolerance
                    blind = dict(t); blind["l0.mix.v"] = torch.zeros_like(t["l0.mix.v"])
                    gap = rel_err(O.forward(cfg, blind, toks)[-1], ref[-1])
                    assert (gap > 0.05) == inside, (window, back, gap)
                del seen


def case_far_key(make):
    """A marked key hundreds of positions back, inside a long window, among keys that all score the same."""
    cfg, t, toks = _one_layer_probe(window=400, n=390, key_pos=3)
    ref = O.forward(cfg, t, toks)
    model = make_worker(make, cfg, t, block_size=8, num_blocks=50)
    got = run_portions(model, toks, 0, [200, 150, 38, 1, 1])
    assert rel_err(got[-8:], ref[-8:]) < TOL
    blind = dict(t); blind["l0.mix.v"] = torch.zeros_like(t["l0.mix.v"])
    assert rel_err(O.forward(cfg, blind, toks)[-1], ref[-1]) > 0.05


def case_sink(make):
    """Scores far below zero: without the extra 1 in the denominator the weights would sum to one and the output would be the
    plain mean of the values; with it they are tiny."""
    cfg = config([(mixer(heads=2, kv_heads=1, dim=8, vdim=6, window=6, dims=0, scale=1.0), None)], width=16, vocab=32, embed_scale=1.0)
    t = O.random_tensors(cfg, seed=12, dtype=torch.float32)
    t["embed"][:, 0] = 1.0
    t["l0.norm1"] = torch.zeros(16)
    q = torch.zeros(16, 16); q[:, 0] = 3.0
    k = torch.zeros(8, 16); k[:, 0] = -3.0
    t["l0.mix.q"], t["l0.mix.k"] = q, k
    toks = tokens_for(cfg, 15, 12)
    ref = O.forward(cfg, t, toks)
    nomix = dict(t); nomix["l0.mix.o"] = torch.zeros_like(t["l0.mix.o"])
    assert rel_err(O.forward(cfg, nomix, toks), ref) < 1e-3          # the sink takes nearly all the weight
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [9, 1, 5]), ref) < TOL
    # and large positive scores leave the sink negligible
    t["l0.mix.k"] = -k
    ref = O.forward(cfg, t, toks)
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [15]), ref) < TOL


def case_group_limit_binds(make):
    """Router weights such that the second-best expert overall lies in a group that is not kept: a router without the group limit
    picks another pair."""
    cfg = config([(mixer(), moe(experts=6, top=2, groups=3, keep=1, shared=None))])
    t = O.random_tensors(cfg, seed=13, dtype=torch.float32)
    r = torch.zeros(6, 48)
    r[0, :] = 0.30; r[1, :] = -0.30; r[2, :] = 0.25; r[3, :] = 0.1; r[4, :] = 0.0; r[5, :] = -0.1
    t["l0.mlp.router"] = r + 0.01 * t["l0.mlp.router"]
    toks = tokens_for(cfg, 12, 13)
    ref = O.forward(cfg, t, toks)
    free = {**cfg, "layers": [{**cfg["layers"][0], "mlp": moe(experts=6, top=2, groups=1, keep=1, shared=None)}]}
    assert rel_err(O.forward(free, t, toks), ref) > 0.02
    model = make_worker(make, cfg, t)
    assert rel_err(run_portions(model, toks, 0, [12]), ref) < TOL

"""GPU: the Rivudra worker and its CUDA kernels (csrc/window_attn.cu, the router / expert / norm kernels of
csrc/parallel_block.cu) against oracle/rivudra.py - every kernel alone, then the scenarios of tests/bupozen_cases.py and
tests/rivudra_cases.py through the worker (fp32 tight, bf16 loose)."""
import types

import pytest
import torch

import bupozen_cases as B
import rivudra_cases as C
from oracle import rivudra as O
from test_bupozen_gpu import _make, tol

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_add_rmsnorm_with_fp32_unit_offset_weight(dtype):
    from swiftllm_b200.worker.kernels.parallel_block import add_rmsnorm_f32
    from swiftllm_b200.worker.weight import unit_offset_norm
    g = torch.Generator().manual_seed(3)
    x = torch.randn(7, 1000, generator=g) * 3
    a, b = (torch.randn(7, 1000, generator=g).to(dtype) for _ in range(2))
    w = (0.1 * torch.randn(1000, generator=g)).to(torch.bfloat16)
    res = x.clone().to(DEV)
    out = add_rmsnorm_f32(res, a.to(DEV), b.to(DEV), unit_offset_norm(w.to(DEV)), 1e-5, out_dtype=dtype)
    xs = x + a.float() + b.float()
    assert out.dtype == dtype and torch.allclose(res.cpu(), xs, rtol=0, atol=1e-6)
    assert B.rel_err(out, O.offset_rms_norm(xs, w.float(), 1e-5)) < tol(dtype)


@pytest.mark.parametrize("experts,top,groups,keep", [(6, 2, 3, 2), (8, 3, 2, 1), (3, 1, 1, 1), (33, 4, 11, 4), (64, 8, 8, 3),
                                                     (256, 8, 8, 4), (5, 5, 1, 1), (12, 3, 4, 4), (200, 32, 2, 1)])
def test_moe_route_grouped(experts, top, groups, keep):
    from swiftllm_b200.worker.kernels.parallel_block import moe_route_grouped
    g = torch.Generator().manual_seed(experts + top)
    h = torch.randn(37, 24, generator=g)
    router = torch.randn(experts, 24, generator=g)
    router[-1] = router[0]                                   # equal scores: the lower index wins
    r = {"experts": experts, "top": top, "scale": 1.75, "groups": {"count": groups, "keep": keep}}
    idx, wts = O.route(h, router, r)
    ref = torch.zeros(37, experts)
    for t in range(37):
        for e, w in zip(idx[t], wts[t]):
            ref[t, e] = w
    got = moe_route_grouped((h @ router.T).contiguous().to(DEV), top, groups, keep, 1.75, 1e-20).cpu()
    assert torch.equal(got != 0, ref != 0)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,ff,sff", [(5, 7, 9), (3, 16, 0), (0, 0, 11), (4, 33, 33)])
def test_clamped_glu_experts(dtype, experts, ff, sff):
    from swiftllm_b200.worker.kernels.parallel_block import moe_clamped_glu_scale
    g = torch.Generator().manual_seed(ff + sff)
    T, cols = 9, experts * ff + sff
    u = (torch.randn(T, 2 * cols, generator=g) * 2).to(dtype)
    w = torch.rand(T, experts, generator=g)
    w[w < 0.5] = 0.0
    y = moe_clamped_glu_scale(u.to(DEV), w.to(DEV) if experts else None, experts, ff, 0.75, sff, 1.5, 1.702).cpu().float()
    uf = u.float()

    def act(gate, up, lim):
        gate, up = gate.clamp(max=lim), up.clamp(-lim, lim)
        return gate * torch.sigmoid(1.702 * gate) * (up + 1)
    ref = torch.zeros(T, cols)
    for e in range(experts):
        blk = uf[:, 2 * ff * e:2 * ff * (e + 1)]
        ref[:, e * ff:(e + 1) * ff] = act(blk[:, :ff], blk[:, ff:], 0.75) * w[:, e:e + 1]
    if sff:
        blk = uf[:, 2 * ff * experts:]
        ref[:, experts * ff:] = act(blk[:, :sff], blk[:, sff:], 1.5)
    assert B.rel_err(y, ref) < tol(dtype)
    if experts:
        assert bool((y[:, :experts * ff].view(T, experts, ff)[w == 0] == 0).all())       # unused experts: exact zeros


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dk,dv,dims,window,bs,sink", [
    (6, 2, 10, 7, 6, 7, 4, True), (8, 2, 48, 32, 48, 40, 16, True), (4, 4, 16, 48, 8, 0, 8, False), (12, 3, 32, 130, 0, 100, 16, True),
    (16, 1, 8, 8, 8, 5, 4, True), (3, 1, 128, 256, 64, 33, 32, False)])
def test_window_attention_standout_keys(dtype, H, G, dk, dv, dims, window, bs, sink):
    """Store + attention kernels on scattered blocks against the plain rule; some keys are scaled so that single scores stand
    out (a far key inside the window, the key just outside it), and token rows are shuffled sequences at unequal positions."""
    from swiftllm_b200.worker.kernels.window_attn import window_attention, window_kv_store
    g = torch.Generator().manual_seed(H * 100 + dk)
    lens = [61, 9, 1, 38]
    nb = sum((n + bs - 1) // bs for n in lens) + 3
    perm = torch.randperm(nb, generator=g).tolist()
    table = torch.full((4, 20), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for b in range((n + bs - 1) // bs):
            table[s, b] = perm.pop()
    tok_seq = [s for s, n in enumerate(lens) for _ in range(n)]
    tok_pos = [p for n in lens for p in range(n)]
    T = len(tok_seq)
    q = torch.randn(T, H * dk, generator=g)
    k = torch.randn(T, G * dk, generator=g)
    v = torch.randn(T, G * dv, generator=g)
    gate = torch.randn(T, H * dv, generator=g)
    w_eff = window if window > 0 else 10 ** 6
    for s0 in (0, 70):                                        # sequences 0 and 3: last query's far key in, next one out
        n = lens[0] if s0 == 0 else lens[3]
        inside, outside = max(0, n - w_eff), n - w_eff - 1
        k[s0 + inside] *= 3.0
        if outside >= 0:
            k[s0 + outside] *= 5.0
    q, k, v, gate = (x.to(dtype) for x in (q, k, v, gate))
    base, scale = 1000.0, 1.0 / dk ** 0.5
    pos = torch.tensor(tok_pos, dtype=torch.float64)
    ang = pos[:, None] * torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)[None] if dims else None
    cos, sin = (torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)) if dims else (None, None)
    st = types.SimpleNamespace(token_seq_ids=torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
                               token_positions=torch.tensor(tok_pos, dtype=torch.int32, device=DEV))
    cache = torch.full((nb, 2, bs, G * (dk + dv)), float("nan"), dtype=dtype, device=DEV)
    fused = torch.cat([q, k, v, gate], dim=1).to(DEV)         # slices of one wide matrix, as the mixer passes them
    qd, kd, vd, gd = fused[:, :H * dk], fused[:, H * dk:(H + G) * dk], fused[:, (H + G) * dk:(H + G) * dk + G * dv], fused[:, (H + G) * dk + G * dv:]
    window_kv_store(kd, vd, cache, 1, table.to(DEV), st, G, dk, dv, dims, cos, sin)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    window_attention(qd, gd, cache, 1, table.to(DEV), st, out, H, G, dk, dv, dims, window, scale, sink, cos, sin)
    assert bool(torch.isnan(cache[:, 0]).all())                # the other slot is untouched
    # the plain rule, per sequence
    ref = torch.zeros(T, H * dv)
    at = 0
    for n in lens:
        positions = list(range(n))
        qq = O.rotate_pairs(q[at:at + n].float().view(n, H, dk), positions, base, dims)
        kk = O.rotate_pairs(k[at:at + n].float().view(n, G, dk), positions, base, dims).to(dtype).float()   # the cache rounds
        vv = v[at:at + n].float().view(n, G, dv)
        for i in range(n):
            js = [j for j in range(n) if O.window_visible(i, j, w_eff)]
            for h in range(H):
                s = torch.stack([(qq[i, h] @ kk[j, h // (H // G)]) * scale for j in js])
                p = O.sink_softmax(s) if sink else torch.softmax(s, dim=0)
                o = sum(p[a] * vv[j, h // (H // G)] for a, j in enumerate(js))
                ref[at + i, h * dv:(h + 1) * dv] = o * torch.sigmoid(gate[at + i, h * dv:(h + 1) * dv].float())
        at += n
    assert B.rel_err(out, ref) < tol(dtype)


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


def test_long_decode():
    B.case_long_decode(_make, C.config([(C.mixer(window=9), C.moe()), (C.mixer(window=4, kv_heads=1), None)]))


def test_greedy_generation():
    B.case_greedy_generation(_make, C.config([(C.mixer(), C.moe()), (C.mixer(window=5), C.moe(shared=None))]))


def test_window_edges():
    C.case_window_edges(_make)


def test_far_key():
    C.case_far_key(_make)


def test_sink():
    C.case_sink(_make)


def test_group_limit_binds():
    C.case_group_limit_binds(_make)


def _tc_config():
    """Head sizes that are multiples of 16 (the shapes the 16-bit tensor-core path takes), windows over several key tiles."""
    return C.config([(C.mixer(heads=8, kv_heads=2, dim=32, vdim=16, dims=32, window=70), C.moe()),
                     (C.mixer(heads=6, kv_heads=1, dim=64, vdim=64, dims=16, window=9), C.moe(shared=None)),
                     (C.mixer(heads=4, kv_heads=4, dim=16, vdim=48, dims=0, window=100), None)], width=64)


def test_bfloat16_worker_close_to_fp32_oracle():
    """bf16 projections / cache, fp32 residual: the logits stay within bf16 rounding of the fp32 oracle on the same weights,
    and do not depend on how the prompt was cut beyond that."""
    for cfg, n, cuts, bs, nb in ((C.full_config(), 33, [5, 2, 1, 1, 24], 4, 40), (_tc_config(), 150, [61, 4, 64, 2, 1, 1, 17], 8, 60)):
        t = O.random_tensors(cfg, seed=11)
        toks = B.tokens_for(cfg, n, 11)
        ref = O.forward(cfg, t, toks)[-40:]
        m = B.make_worker(_make, cfg, t, dtype="bfloat16", block_size=bs, num_blocks=nb)
        whole = B.run_portions(m, toks, 0, [n])[-40:]
        cut = B.run_portions(m, toks, 1, cuts)[-40:]
        assert B.rel_err(whole, ref) < 3e-2 and B.rel_err(cut, ref) < 3e-2 and B.rel_err(cut, whole) < 2e-2


def test_cuda_graph_decode_matches_eager():
    cfg = C.config([(C.mixer(window=11), C.moe()), (C.mixer(heads=5, kv_heads=5, window=6), C.moe(shared=None))], width=64)
    t = O.random_tensors(cfg, seed=13)
    t["head"] = (t["head"].float() * 4).to(t["head"].dtype)
    prompts = [B.tokens_for(cfg, n, 70 + k) for k, n in enumerate((7, 3, 12))]
    runs = []
    for graph in (False, True):
        m = B.make_worker(_make, cfg, t, dtype="bfloat16", block_size=4, num_blocks=40)
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


def test_trace_replay_command_line(tmp_path):
    """bin/trace_run on a checkpoint folder of this design: a mixed schedule (portions beside decoded tokens, requests that end
    and whose rows and blocks are used again) in both dtypes, against the oracle run on each whole sequence."""
    import json
    import os
    import subprocess
    import numpy as np
    from safetensors.torch import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = C.config([
        (C.mixer(heads=10, kv_heads=2, dim=16, vdim=24, window=21, base=5000.0, dims=16), C.moe(experts=9, top=3, ff=24, groups=3, keep=2)),
        (C.mixer(heads=3, kv_heads=3, dim=8, vdim=8, window=9, base=300.0, dims=6), None),
        (C.mixer(heads=18, kv_heads=1, dim=16, vdim=8, window=33, base=5000.0, dims=16), C.moe(shared=None)),
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
    for dtype, limit in (("float32", 2e-4), ("bfloat16", 4e-2)):
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


@pytest.mark.parametrize("H,G,dk,dv,window", [(16, 2, 64, 48, 90), (6, 2, 32, 16, 40), (16, 1, 16, 16, 7), (4, 4, 128, 128, 0),
                                              (12, 4, 48, 80, 150), (64, 1, 16, 32, 33)])
def test_tensor_core_and_cuda_core_attention_agree(H, G, dk, dv, window):
    """The same mixed step (two prompt portions that start inside a sequence, a one-token prompt, three decoded tokens) through
    the tensor-core kernel and through the fp32 CUDA-core kernel: bf16 storage, heads per group that are not a power of two,
    several key tiles, token runs that end inside a CTA's token range."""
    from swiftllm_b200.worker.kernels import window_attn as WA
    g = torch.Generator().manual_seed(H + dk)
    bs, lens = 16, [300, 77, 1, 200, 130, 65]                 # cached lengths after this step
    new = [150, 40, 1, 1, 1, 1]                              # tokens of this step per sequence (the last ones)
    nb = sum((n + bs - 1) // bs for n in lens)
    perm = torch.randperm(nb, generator=g).tolist()
    table = torch.full((6, 32), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for b in range((n + bs - 1) // bs):
            table[s, b] = perm.pop()
    cache = (torch.randn(nb, 1, bs, G * (dk + dv), generator=g)).to(torch.bfloat16).to(DEV)
    tok_seq = [s for s, n in enumerate(new) for _ in range(n)]
    tok_pos = [lens[s] - n + p for s, n in enumerate(new) for p in range(n)]
    T = len(tok_seq)
    q = torch.randn(T, H * dk, generator=g).to(torch.bfloat16).to(DEV)
    gate = torch.randn(T, H * dv, generator=g).to(torch.bfloat16).to(DEV)
    dims = dk // 2
    ang = torch.tensor(tok_pos, dtype=torch.float64)[:, None] * torch.tensor([100.0 ** (-2.0 * i / dims) for i in range(dims // 2)],
                                                                             dtype=torch.float64)[None]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    st = types.SimpleNamespace(token_seq_ids=torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
                               token_positions=torch.tensor(tok_pos, dtype=torch.int32, device=DEV), num_prefill_tokens=191)
    outs = []
    for simt in (True, False):
        old = WA.set_simt(simt)
        try:
            out = torch.zeros(T, H * dv, dtype=torch.bfloat16, device=DEV)
            WA.window_attention(q, gate, cache, 0, table.to(DEV), st, out, H, G, dk, dv, dims, window, dk ** -0.5, True, cos, sin)
            outs.append(out.float().cpu())
        finally:
            WA.set_simt(old)
    assert B.rel_err(outs[1], outs[0]) < 1.5e-2
    # every row on its own is close too (a row that saw a wrong window would stand out)
    row_err = (outs[1] - outs[0]).pow(2).mean(-1).sqrt() / outs[0].pow(2).mean(-1).sqrt()
    assert float(row_err.max()) < 4e-2

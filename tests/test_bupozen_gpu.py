"""GPU: the Bupozen worker and its CUDA kernels (csrc/parallel_block.cu, csrc/latent_attn.cu) against oracle/bupozen.py -
every kernel alone, then the scenarios of tests/bupozen_cases.py through the worker (fp32 tight, bf16 loose)."""
import types

import pytest
import torch

import bupozen_cases as C
from oracle import bupozen as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.5e-2


def _make(cfg, tensors, eng):
    import swiftllm_b200
    from swiftllm_b200.worker.weight import dict_getter
    torch.cuda.set_device(0)
    ec = swiftllm_b200.EngineConfig(model_path="", use_dummy=False, block_size=eng["block_size"], gpu_mem_utilization=0.9,
                                    num_cpu_blocks=0, max_seqs_in_block_table=eng["rows"], max_blocks_per_seq=eng["num_blocks"],
                                    max_batch_size=4, max_tokens_in_batch=256, dtype=eng["dtype"])
    m = swiftllm_b200.create_model(ec, swiftllm_b200.registry.model_config_from_dict(cfg))
    m.load_weights(dict_getter(tensors))
    m.init_kvcache_and_swap(eng["num_blocks"])
    return m


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 1000, 4096])
def test_add_rmsnorm_f32(dtype, width):
    from swiftllm_b200.worker.kernels.parallel_block import add_rmsnorm_f32
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3
    a, b = (torch.randn(7, width, generator=g).to(dtype) for _ in range(2))
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(dtype)
    for aa, bb in ((None, None), (a, None), (None, b), (a, b)):
        xs = x.clone()
        if aa is not None or bb is not None:
            xs = xs + ((aa.float() if aa is not None else 0) + (bb.float() if bb is not None else 0))
        res = x.clone().to(DEV)
        out = add_rmsnorm_f32(res, None if aa is None else aa.to(DEV), None if bb is None else bb.to(DEV), w.to(DEV), 1e-5)
        assert out.dtype == dtype and torch.allclose(res.cpu(), xs, rtol=0, atol=1e-6)        # the residual itself stays fp32
        assert C.rel_err(out, O.rms_norm(xs, w.float(), 1e-5)) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_strided_slice_of_a_wider_matrix(dtype):
    from swiftllm_b200.worker.kernels.parallel_block import rmsnorm_strided
    g = torch.Generator().manual_seed(1)
    big = (torch.randn(5, 77, generator=g) * 2).to(dtype)
    w = (1 + 0.1 * torch.randn(21, generator=g)).to(dtype)
    out = rmsnorm_strided(big.to(DEV)[:, 13:34], w.to(DEV), 1e-3)
    assert out.is_contiguous() and C.rel_err(out, O.rms_norm(big[:, 13:34].float(), w.float(), 1e-3)) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_relu2_and_expert_scaling(dtype):
    from swiftllm_b200.worker.kernels.parallel_block import moe_relu2_scale_inplace, relu2_inplace
    g = torch.Generator().manual_seed(2)
    u = torch.randn(9, 5 * 7, generator=g).to(dtype)
    x = u.clone().to(DEV)
    relu2_inplace(x)
    assert C.rel_err(x, O.relu_squared(u.float())) < tol(dtype)
    w = torch.rand(9, 5, generator=g)
    w[w < 0.5] = 0.0
    x = u.clone().to(DEV)
    moe_relu2_scale_inplace(x, w.to(DEV), 7)
    ref = (O.relu_squared(u.float()).view(9, 5, 7) * w[:, :, None]).view(9, 35)
    assert C.rel_err(x, ref) < tol(dtype)
    assert bool((x.cpu().view(9, 5, 7)[w == 0] == 0).all())              # unused experts: exact zeros


@pytest.mark.parametrize("experts,top", [(6, 2), (3, 1), (33, 4), (64, 8), (200, 32), (5, 5)])
def test_moe_route(experts, top):
    from swiftllm_b200.worker.kernels.parallel_block import moe_route
    g = torch.Generator().manual_seed(experts)
    h = torch.randn(37, 16, generator=g)
    router = torch.randn(experts, 16, generator=g)
    idx, wts = O.route(h, router, top)
    got = moe_route((h @ router.T).to(DEV).contiguous(), top).cpu()
    ref = torch.zeros(37, experts).scatter_(1, idx, wts)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6)
    assert bool(((got > 0).sum(1) == top).all()) and torch.allclose(got.sum(1), torch.ones(37), atol=1e-5)


def _paged(rows_by_seq, block_size, width, dtype, seed=0, shuffle=True):
    """A cache with one slot of interest (slot 1 of 3) whose blocks are scattered; returns cache, block_table, fill function."""
    nseq = len(rows_by_seq)
    per = [(n + block_size - 1) // block_size for n in rows_by_seq]
    nb = sum(per) + 3
    g = torch.Generator().manual_seed(seed)
    ids = torch.randperm(nb, generator=g).tolist() if shuffle else list(range(nb))
    bt = torch.full((nseq, max(per) + 1), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(per):
        bt[s, :n] = torch.tensor(ids[at:at + n], dtype=torch.int32); at += n
    cache = torch.zeros(nb, 3, block_size, width, dtype=dtype)
    return cache, bt


def _row_index(bt, s, p, bs):
    return int(bt[s, p // bs]), p % bs


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_kv_store(dtype):
    """norm + rotary + scatter to the tokens' cache rows; nothing else of the cache is touched."""
    from swiftllm_b200.worker.kernels.latent_attn import latent_kv_store
    r, dr, dims, bs, base = 24, 6, 4, 4, 100.0
    cache, bt = _paged([11, 6], bs, r + dr, dtype)
    cache.fill_(7.0)
    g = torch.Generator().manual_seed(3)
    tok_seq, tok_pos = [0, 0, 0, 1, 0, 1], [3, 4, 5, 5, 10, 0]           # crosses a block border; last and first rows
    wide = torch.randn(6, 50, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(r, generator=g)).to(dtype)
    m = {"kv_rank": r, "rot_dim": dr, "rot": {"base": base, "dims": dims}}
    ang = torch.tensor(tok_pos, dtype=torch.float64)[:, None] * torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)],
                                                                            dtype=torch.float64)
    st = types.SimpleNamespace(token_seq_ids=torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
                               token_positions=torch.tensor(tok_pos, dtype=torch.int32, device=DEV))
    dcache = cache.to(DEV)
    latent_kv_store(wide.to(DEV)[:, 9:9 + r + dr], w.to(DEV), dcache, 1, bt.to(DEV), st, r, dr, dims, 1e-5,
                    torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV))
    got = dcache.cpu()
    touched = torch.zeros(cache.shape[:3], dtype=torch.bool)
    for t, (s, p) in enumerate(zip(tok_seq, tok_pos)):
        x = wide[t:t + 1, 9:9 + r + dr].float()
        c = O.rms_norm(x[:, :r], w.float(), 1e-5)
        kr = O.rotate_pairs(x[:, r:], [p], base, dims)
        b, o = _row_index(bt, s, p, bs)
        touched[b, 1, o] = True
        assert C.rel_err(got[b, 1, o], torch.cat([c[0], kr[0]])) < tol(dtype), (t, s, p)
    assert bool((got[~touched] == 7.0).all())


def _plain_attention(q_lat, q_rot, gate, rows, pos, window, scale, base, dims, r):
    """One query (all heads) against the cached rows of positions 0..pos: visibility by the window rule, plain softmax."""
    H = q_lat.shape[0]
    qr = O.rotate_pairs(q_rot[None].double(), [pos], base, dims)[0]
    out = torch.zeros(H, r, dtype=torch.float64)
    js = [j for j in range(pos + 1) if window <= 0 or O.window_visible(pos, j, window)]
    for h in range(H):
        s = torch.stack([(q_lat[h].double() @ rows[j, :r].double() + qr[h] @ rows[j, r:].double()) * scale for j in js])
        p = torch.softmax(s, dim=0)
        out[h] = sum(p[k] * rows[j, :r].double() for k, j in enumerate(js)) * torch.sigmoid(gate[h].double())
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,r,dr,dims,window,bs", [
    (3, 24, 6, 4, 7, 4), (11, 72, 4, 4, 33, 16), (2, 136, 8, 8, 0, 8), (9, 40, 2, 0, 32, 32),      # CUDA-core kernel
    # 16-element-aligned rows: with 16-bit storage these take the tensor-core kernel (1, 2 and 3 head groups, whole and partial
    # column tiles per warp, windows that end inside / at the edge of / beyond a 64-key tile)
    (20, 64, 16, 16, 100, 16), (5, 128, 32, 24, 0, 8), (16, 512, 64, 64, 64, 16), (33, 208, 48, 48, 65, 4), (4, 16, 16, 0, 63, 32),
    (2, 528, 16, 16, 40, 16), (3, 1000, 6, 6, 20, 8)])                                                # latents wider than 512
def test_latent_attention_standout_keys(dtype, H, r, dr, dims, window, bs):
    """Among hundreds of small keys ONE key per query scores far above the rest, placed where an off-by-one shows: far back,
    the first and last position a window keeps, the position just outside it, both sides of a block border, position 0.  A
    query that wrongly sees (or misses) its stand-out key gets a completely different output."""
    from swiftllm_b200.worker.kernels.latent_attn import latent_attention
    n, base, scale = 300, 50.0, 0.3
    g = torch.Generator().manual_seed(H * 1000 + r)
    cache, bt = _paged([n, 40], bs, r + dr, dtype, seed=r)
    rows = [(torch.randn(m, r + dr, generator=g) * 0.2).to(dtype) for m in (n, 40)]
    for s, rr in enumerate(rows):
        for p in range(rr.shape[0]):
            b, o = _row_index(bt, s, p, bs)
            cache[b, 1, o] = rr[p]
    W = window if window > 0 else n
    queries = []                                                   # (seq, pos, stand-out key position)
    for pos in (n - 1, n - 2, 257, 2 * bs, 2 * bs - 1):
        for key in (pos - W + 1, pos - W, pos - W + 2, pos, 0, (pos // bs) * bs, (pos // bs) * bs - 1, pos - 1):
            if 0 <= key <= pos:
                queries.append((0, pos, key))
    queries += [(1, 0, 0), (1, 1, 0), (1, 39, 39 - min(W, 40) + 1), (1, 5, 3)]
    T = len(queries)
    q_lat = torch.randn(T, H, r, generator=g) * 0.3
    for t, (s, pos, key) in enumerate(queries):                    # point every head's query at its stand-out key's latent
        c = rows[s][key, :r].float()
        q_lat[t] += 40.0 * c / (c.norm() ** 2 * scale)
    q_lat = q_lat.to(dtype)
    q_wide = torch.randn(T, H, 5 + dr, generator=g).to(dtype)      # q_rot is a strided slice, as in the worker
    gate = torch.randn(T, H + 3, generator=g).to(dtype)
    ang = torch.tensor([p for _, p, _ in queries], dtype=torch.float64)[:, None] * \
        torch.tensor([base ** (-2.0 * i / max(dims, 1)) for i in range(dims // 2)], dtype=torch.float64)
    st = types.SimpleNamespace(token_seq_ids=torch.tensor([s for s, _, _ in queries], dtype=torch.int32, device=DEV),
                               token_positions=torch.tensor([p for _, p, _ in queries], dtype=torch.int32, device=DEV))
    out = torch.full((T, H, r + 2), 9.0, dtype=dtype, device=DEV)
    latent_attention(q_lat.to(DEV), q_wide.to(DEV)[:, :, 5:], gate.to(DEV)[:, 3:], cache.to(DEV), 1, bt.to(DEV), st,
                     out[:, :, :r], dims, window, scale, torch.cos(ang).float().to(DEV).contiguous(),
                     torch.sin(ang).float().to(DEV).contiguous())
    assert bool((out[:, :, r:] == 9.0).all())
    for t, (s, pos, key) in enumerate(queries):
        ref = _plain_attention(q_lat[t].float(), q_wide[t, :, 5:].float(), gate[t, 3:].float(), rows[s].float(), pos, window, scale,
                               base, dims, r)
        assert C.rel_err(out[t, :, :r], ref) < (1e-4 if dtype == torch.float32 else 3e-2), (s, pos, key)


def test_tensor_core_and_cuda_core_attention_agree():
    """The same bf16 inputs through both kernels (the library switch forces the CUDA-core one)."""
    from swiftllm_b200 import _lib
    from swiftllm_b200.worker.kernels.latent_attn import latent_attention
    H, r, dr, bs, n = 24, 96, 32, 16, 200
    g = torch.Generator().manual_seed(5)
    cache, bt = _paged([n], bs, r + dr, torch.bfloat16, seed=5)
    cache.copy_((torch.randn(cache.shape, generator=g) * 0.5).to(torch.bfloat16))
    pos = [0, 1, 15, 16, 63, 64, 65, 127, 128, 199]
    T = len(pos)
    q_lat, q_rot = (torch.randn(T, H, d, generator=g).to(torch.bfloat16).to(DEV) for d in (r, dr))
    gate = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    ang = torch.tensor(pos, dtype=torch.float64)[:, None] * torch.tensor([10.0 ** (-2.0 * i / 32) for i in range(16)], dtype=torch.float64)
    st = types.SimpleNamespace(token_seq_ids=torch.zeros(T, dtype=torch.int32, device=DEV),
                               token_positions=torch.tensor(pos, dtype=torch.int32, device=DEV))
    outs = []
    for simt in (0, 1):
        old = _lib.lib().sllm_latent_attention_set_simt(simt)
        try:
            out = torch.empty(T, H, r, dtype=torch.bfloat16, device=DEV)
            latent_attention(q_lat, q_rot, gate, cache.to(DEV), 1, bt.to(DEV), st, out, 32, 70, 0.2,
                             torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV))
            outs.append(out.float().cpu())
        finally:
            _lib.lib().sllm_latent_attention_set_simt(old)
    assert C.rel_err(outs[0], outs[1]) < 1e-2


# ---------------------------------------------------------------- the worker
@pytest.mark.parametrize("name", sorted(C.SINGLE))
def test_single_mechanisms(name):
    C.case_whole_prompt(_make, C.SINGLE[name], n=17)


def test_whole_prompt():
    C.case_whole_prompt(_make, C.full_config())


def test_prefill_vs_decode():
    C.case_prefill_vs_decode(_make, C.full_config())


def test_portions():
    C.case_portions(_make, C.full_config())


def test_mixed_batch():
    C.case_mixed_batch(_make, C.full_config())


def test_blocks_and_rows_reused():
    C.case_blocks_and_rows_reused(_make, C.full_config())


def test_long_decode():
    C.case_long_decode(_make, C.config([(C.mixer(window=9), C.DENSE), (C.mixer(window=4, kv_from=0), C.moe())]))


def test_greedy_generation():
    C.case_greedy_generation(_make, C.config([(C.mixer(), C.DENSE), (C.mixer(window=5, kv_from=0), C.moe())]))


def test_bfloat16_worker_close_to_fp32_oracle():
    """bf16 projections / cache, fp32 residual: the logits stay within bf16 rounding of the fp32 oracle on the same weights,
    and do not depend on how the prompt was cut beyond that."""
    cfg = C.full_config()
    t = O.random_tensors(cfg, seed=11)
    toks = C.tokens_for(cfg, 33, 11)
    ref = O.forward(cfg, t, toks)
    m = C.make_worker(_make, cfg, t, dtype="bfloat16")
    whole = C.run_portions(m, toks, 0, [33])
    cut = C.run_portions(m, toks, 1, [5, 2, 1, 1, 24])
    assert C.rel_err(whole, ref) < 3e-2 and C.rel_err(cut, ref) < 3e-2 and C.rel_err(cut, whole) < 2e-2


def test_bfloat16_worker_on_tensor_core_shapes():
    """Latent sizes that are multiples of 16 send the bf16 worker through the tensor-core attention kernel."""
    cfg = C.config([(C.mixer(heads=3, kv_rank=32, rot_dim=16, dims=16, window=70), C.DENSE),
                    (C.mixer(heads=18, kv_rank=32, rot_dim=16, dims=16, window=9, kv_from=0), C.moe()),
                    (C.mixer(heads=2, kv_rank=144, rot_dim=32, dims=20, window=100), None)], width=64)
    t = O.random_tensors(cfg, seed=12)
    toks = C.tokens_for(cfg, 150, 12)
    ref = O.forward(cfg, t, toks)[-40:]
    m = C.make_worker(_make, cfg, t, dtype="bfloat16", block_size=8, num_blocks=60)
    whole = C.run_portions(m, toks, 0, [150])[-40:]
    cut = C.run_portions(m, toks, 1, [61, 4, 64, 2, 1, 1, 17])[-40:]
    assert C.rel_err(whole, ref) < 3e-2 and C.rel_err(cut, ref) < 3e-2 and C.rel_err(cut, whole) < 2e-2


def test_cuda_graph_decode_matches_eager():
    """Pure-decode steps replayed from a CUDA graph (EngineConfig.use_cuda_graph) give the eager path's tokens, across block
    borders, for two batch sizes, and leave the allocator's host mirror in step with the device."""
    cfg = C.config([(C.mixer(heads=3, kv_rank=32, rot_dim=16, dims=16, window=11), C.DENSE),
                    (C.mixer(heads=5, kv_rank=32, rot_dim=16, dims=16, window=6, kv_from=0), C.moe())], width=64)
    t = O.random_tensors(cfg, seed=13)
    t["head"] = (t["head"].float() * 4).to(t["head"].dtype)
    prompts = [C.tokens_for(cfg, n, 70 + k) for k, n in enumerate((7, 3, 12))]
    runs = []
    for graph in (False, True):
        m = C.make_worker(_make, cfg, t, dtype="bfloat16", block_size=4, num_blocks=40)
        m.engine_config.use_cuda_graph = graph
        last = m.forward(prompts, [0, 1, 2], [])
        lens, toks = [len(p) for p in prompts], [list(last)]
        for step in range(9):
            live = [0, 1, 2] if step < 6 else [0, 2]                # the batch shrinks: a second graph
            for i in live:
                lens[i] += 1
            out = m.forward([[toks[-1][i]] for i in live], live, [lens[i] for i in live])
            nxt = list(toks[-1])
            for i, o in zip(live, out):
                nxt[i] = o
            toks.append(nxt)
        assert m.gpu_block_manager.check_device_status() >= 0
        free = m.gpu_block_manager.num_free_blocks
        assert free == 40 - sum((n + 3) // 4 for n in lens) and int(m.gpu_block_manager.is_block_free.sum()) == free
        runs.append(toks)
    assert runs[0] == runs[1]


def test_trace_replay_command_line(tmp_path):
    """bin/trace_run on a checkpoint folder: a mixed schedule (portions beside decoded tokens, requests that end and whose rows
    and blocks are used again) in both dtypes, against the oracle run on each whole sequence."""
    import json
    import os
    import subprocess
    import numpy as np
    from safetensors.torch import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = C.config([
        (C.mixer(heads=5, dim=16, rot_dim=16, vdim=24, kv_rank=48, q_rank=40, window=21, base=5000.0, dims=16), C.moe(experts=7, top=3, ff=24)),
        (C.mixer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=40, q_rank=24, window=9, base=300.0, dims=6), C.DENSE),
        (C.mixer(heads=18, dim=16, rot_dim=16, vdim=8, kv_rank=48, q_rank=40, window=33, base=5000.0, dims=16, kv_from=0), None),
    ], width=72, vocab=131, eps=1e-6)
    t = O.random_tensors(cfg, seed=21)
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in t.items()}, str(model_dir / "model.safetensors"))
    reqs = {k: C.tokens_for(cfg, n, s) for s, (k, n) in enumerate((("a", 70), ("b", 41), ("c", 17), ("d", 5), ("e", 30)))}
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
        # the pool is smaller than the sum of all requests: 70 + 41 + 30 live at most, rounded up per request
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True, cwd=root)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
        for n, rr in enumerate(rows):
            got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rr), -1)
            for j, (k, pos) in enumerate(rr):
                err = np.sqrt(((got[j] - ref[k][pos]) ** 2).mean() / (ref[k][pos] ** 2).mean())
                assert err < limit, (dtype, n, k, pos, err)

"""The Pesivik path on the GPU against the plain restatement in ``pesivik_oracle`` (float64, token loops): every
mechanism alone through its kernel, then whole models through ``ModelRunner.forward_ragged`` and the engine -- whole
prompts against token-by-token decoding, portions down to two tokens, unequal batches against each request alone,
pool rows and slots that change hands, keys just inside and just outside the window in prompts and in decoding, far
keys, the first tokens, long decoding, sizes that differ from one another.  fp32 runs are held to 1e-4 of the logits'
spread; bf16 runs to a few bf16 roundings."""

from __future__ import annotations

import math
import random

import numpy as np
import pytest
import torch

import pesivik_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]
DEV = "cuda"


def _i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def _close(got, ref, tol):
    got = got.double().cpu()
    ref = torch.as_tensor(np.asarray(ref)).double()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = (got - ref).abs().max().item()
    spread = max(ref.abs().max().item(), 1e-6)
    assert err <= tol * spread, f"max abs err {err:.3e} on values up to {spread:.3e} (tol {tol})"


# ------------------------------------------------------------------------------------------- mechanisms alone #
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
def test_layer_norms_layer_scale_and_the_fused_input_norm(dtype, tol):
    from lite_llama_b200.kernels import embed_positions, post_norm_residual, rmsnorm_from_f32

    n, vocab, eps = 44, 30, 1e-3
    embed = torch.randn(vocab, n).to(dtype)
    toks = [3, 29, 0, 7, 7]
    r, act = embed_positions(_i32(toks), _i32(range(5)), embed.to(DEV), None, want_act=False, scale=0.3)
    ref = embed.double().numpy()[toks] * 0.3
    assert act is None
    _close(r, ref, 1e-6)
    y = (torch.randn(5, n) * 3 + 2).to(dtype)                 # a mean far from zero: the variance is of the deviations
    w, ls, wn = ((1 + 0.2 * torch.randn(n)).to(dtype) for _ in range(3))
    act = post_norm_residual(r, y.to(DEV), w.to(DEV), eps, 0.0, kind="layer", layer_scale=ls.to(DEV),
                             next_weight=wn.to(DEV), next_kind="layer")
    ref = ref + np.stack([O.layer_norm(O.f64(y[t]), O.f64(w), eps) * O.f64(ls) for t in range(5)])
    _close(r, ref, 3e-6)
    _close(act, np.stack([O.layer_norm(ref[t], O.f64(wn), eps) for t in range(5)]), tol)
    out = rmsnorm_from_f32(r, w.to(DEV), eps, 0.0, _i32([4, 1]), kind="layer")
    _close(out, np.stack([O.layer_norm(ref[t], O.f64(w), eps) for t in (4, 1)]), tol)
    # without the fused norm the call hands back the plain copy (or nothing in fp32), as for the post-norm designs
    act = post_norm_residual(r, y.to(DEV), w.to(DEV), eps, 0.0, kind="layer")
    assert (act is None) == (dtype == torch.float32)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_gelu_forms_and_soft_cap(dtype, tol):
    from lite_llama_b200.kernels import gelu, softcap_to_f32

    x = (torch.randn(7, 33) * 3).to(dtype)
    _close(gelu(x.to(DEV)), O.gelu_erf(O.f64(x)), tol)
    z = O.f64(x)
    _close(gelu(x.to(DEV), "tanh"), 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))), tol)
    big = (torch.randn(4, 50) * 40).to(dtype)
    capped = softcap_to_f32(big.to(DEV), 9.0)
    assert capped.dtype == torch.float32
    _close(capped, O.soft_cap(O.f64(big), 9.0), 2e-6)
    _close(softcap_to_f32(big.to(DEV), 0.0), O.f64(big), 0)


@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,rot_dims,heads", [(20, 12, 4, 4, 3), (16, 24, 8, 8, 2), (9, 5, 6, 2, 1),
                                                                   (8, 8, 0, 0, 2)])
def test_latent_prepare_and_query_rotation(q_rank, kv_rank, rot_dim, rot_dims, heads):
    from lite_llama_b200.kernels import latent_prepare, rope_heads, rope_table

    T, eps, base = 6, 1e-4, 300.0
    cols = q_rank + kv_rank + rot_dim + heads
    proj = torch.randn(T, cols + 3)
    wq, wkv = 1 + 0.3 * torch.randn(q_rank), 1 + 0.3 * torch.randn(kv_rank)
    pos = [0, 1, 977, 40, 3, 2500]
    rows = [5, 0, 7, 2, 9, 1]
    pool = torch.full((10, kv_rank + rot_dim + 2), 9.0, device=DEV)
    dev = proj.to(DEV)
    cs = rope_table(_i32(pos), rot_dims, base)
    assert (cs is None) == (rot_dims == 0)
    latent_prepare(dev, pool, _i32(rows), cs, wq.to(DEV), wkv.to(DEV), q_rank, kv_rank, rot_dim, rot_dims, eps)
    p64 = O.f64(proj)
    _close(dev[:, :q_rank], np.stack([O.rms_norm(p64[t, :q_rank], O.f64(wq), eps) for t in range(T)]), 2e-6)
    _close(dev[:, q_rank:], p64[:, q_rank:], 0)                       # the rest of the row is left alone
    want = np.stack([np.concatenate([O.rms_norm(p64[t, q_rank:q_rank + kv_rank], O.f64(wkv), eps),
                                     O.rotate(p64[t, q_rank + kv_rank:q_rank + kv_rank + rot_dim], pos[t], rot_dims, base)])
                     for t in range(T)])
    _close(pool[torch.tensor(rows, device=DEV).long(), :kv_rank + rot_dim], want, 3e-6)
    assert (pool[:, kv_rank + rot_dim:] == 9.0).all() and (pool[[3, 4, 6, 8]] == 9.0).all()
    if rot_dim:
        dim = 5
        q = torch.randn(T, heads * (dim + rot_dim))
        dst = torch.zeros(T, heads * (kv_rank + rot_dim), device=DEV)
        qd = q.to(DEV)
        rope_heads(dst[:, kv_rank:], kv_rank + rot_dim, qd[:, dim:], dim + rot_dim, cs, heads, rot_dim, rot_dims)
        for h in range(heads):
            ref = np.stack([O.rotate(O.f64(q[t, h * (dim + rot_dim) + dim:(h + 1) * (dim + rot_dim)]), pos[t], rot_dims, base)
                            for t in range(T)])
            _close(dst[:, h * (kv_rank + rot_dim) + kv_rank:(h + 1) * (kv_rank + rot_dim)], ref, 3e-6)
            assert (dst[:, h * (kv_rank + rot_dim):h * (kv_rank + rot_dim) + kv_rank] == 0).all()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("m,heads,n,k", [(1, 1, 1, 1), (37, 3, 12, 8), (70, 2, 65, 20)])
def test_per_head_products_with_the_sigmoid_gate(dtype, tol, m, heads, n, k):
    from lite_llama_b200.kernels import head_linear

    x = torch.randn(m, heads * k + 2).to(dtype)
    w = torch.randn(heads, n, k).to(dtype)
    gate = torch.randn(m, heads + 3).to(dtype)
    out = torch.zeros(m, heads * n, dtype=dtype, device=DEV)
    head_linear(out, n, x.to(DEV), k, w.to(DEV))
    ref = torch.einsum("thk,hnk->thn", x[:, :heads * k].double().view(m, heads, k), w.double())
    _close(out, ref.reshape(m, heads * n), tol)
    head_linear(out, n, x.to(DEV), k, w.to(DEV), gate.to(DEV)[:, 2:])
    ref = ref * torch.sigmoid(gate[:, 2:2 + heads].double()).unsqueeze(-1)
    _close(out, ref.reshape(m, heads * n), tol)


def _window_case(heads, rank, rot, seqs, window, dtype, boost=None, seed=0):
    """Attention over cached rows [latent | rotated part] as one key/value head whose values are the latent:
    ``seqs = [(new tokens, cached tokens)]``; returns (kernel output, plain softmax over each token's window)."""
    from lite_llama_b200.kernels import sink_attention

    g = torch.Generator().manual_seed(seed)
    D, scale = rank + rot, 0.3
    width = -(-D // 8) * 8
    total = sum(n + c for n, c in seqs)
    perm = torch.randperm(total + 5, generator=g)[:total].tolist()         # scattered pool rows
    pool = torch.randn(total + 5, width, generator=g).to(dtype)
    max_len = max(n + c for n, c in seqs)
    table = torch.zeros(len(seqs), max_len, dtype=torch.int32)
    q = torch.randn(sum(n for n, _ in seqs), heads * D, generator=g).to(dtype)
    starts, at, used = [0], 0, 0
    for s, (n, c) in enumerate(seqs):
        table[s, :n + c] = torch.tensor(perm[used:used + n + c], dtype=torch.int32)
        used += n + c
        starts.append(starts[-1] + n)
    if boost is not None:                                   # (sequence, query token, key position, gain): one score stands out
        s, t, key, gain = boost
        row = table[s, key].item()
        qi = starts[s] + t
        pool[row, :D] = (q[qi, :D].float() / q[qi, :D].float().norm() * gain).to(dtype)
    ref = torch.zeros(q.shape[0], heads * rank, dtype=torch.float64)
    for s, (n, c) in enumerate(seqs):
        for t in range(n):
            p = c + t
            keys = [j for j in range(p + 1) if window <= 0 or p - j < window]
            kv = pool[table[s, keys].long()].double()
            for h in range(heads):
                sc = (kv[:, :D] @ q[starts[s] + t, h * D:(h + 1) * D].double()) * scale
                pr = torch.softmax(sc, 0)
                ref[starts[s] + t, h * rank:(h + 1) * rank] = pr @ kv[:, :rank]
    out = torch.zeros(q.shape[0], heads * rank, dtype=dtype, device=DEV)
    lens, ctxs = [n for n, _ in seqs], [c for _, c in seqs]
    portions = [i for i, n in enumerate(lens) if n > 1]
    singles = [i for i, n in enumerate(lens) if n == 1]
    args = (q.to(DEV), pool.to(DEV), table.to(DEV), _i32(starts), _i32(ctxs), _i32(range(len(seqs))))
    if portions:
        sink_attention(out, *args, _i32(portions), len(portions), max(lens), None, heads, 1, D, rank, scale, 0.0,
                       window=window, v_col0=0)
    if singles:
        keys = max(ctxs[i] for i in singles) + 1
        keys = min(keys, window) if window > 0 else keys
        splits = max(1, -(-keys // 128))
        per = -(-(-(-keys // splits)) // 32) * 32
        sink_attention(out, *args, _i32(singles), len(singles), 1, None, heads, 1, D, rank, scale, 0.0,
                       num_splits=splits, split_keys=per, window=window, v_col0=0)
    return out, ref


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("heads,rank,rot,window", [(3, 12, 4, 7), (2, 24, 8, 70), (5, 10, 3, 1), (2, 16, 16, 150),
                                                   (1, 40, 8, 0), (20, 8, 8, 33), (70, 16, 8, 140), (6, 64, 16, 0)])
def test_windowed_attention_on_the_latent_rows(dtype, tol, heads, rank, rot, window):
    """Portions with and without a cached prefix, single tokens, windows shorter and longer than a key tile (32 / 64)
    and than a key range of the single-token kernel (128); the values are the leading columns of the keys."""
    out, ref = _window_case(heads, rank, rot, [(70, 0), (1, 0), (9, 200), (1, 333), (130, 61), (1, 5), (2, 149)], window,
                            dtype, seed=heads)
    _close(out, ref, tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads", [2, 6])          # 6 heads on one cached row: single tokens take the heads-as-rows tiles
@pytest.mark.parametrize("window,ctx", [(37, 100), (64, 64), (65, 300), (129, 400)])
def test_the_key_at_the_window_edge_counts_and_the_next_one_does_not(dtype, heads, window, ctx):
    """One key is made to dominate its query's scores.  Just inside the window (distance window - 1) the output is
    that key's latent; one step further out it must have no influence at all -- for a token inside a portion and for
    a token decoded alone."""
    rank, rot = 16, 8
    for new, t in ((12, 7), (1, 0)):                        # a portion's 8th token; a single token
        p = ctx + t
        inside, ref_in = _window_case(heads, rank, rot, [(3, 10), (new, ctx)], window, dtype, boost=(1, t, p - window + 1, 60.0))
        _close(inside, ref_in, 1e-5 if dtype == torch.float32 else 2e-2)
        outside, ref_out = _window_case(heads, rank, rot, [(3, 10), (new, ctx)], window, dtype, boost=(1, t, p - window, 60.0))
        _close(outside, ref_out, 1e-5 if dtype == torch.float32 else 2e-2)
        row = 3 + t
        assert (ref_in[row] - ref_out[row]).abs().max() > 0.5          # the case does tell the two apart


@pytest.mark.parametrize("experts,top,groups,keep", [(8, 3, 4, 2), (15, 4, 5, 3), (6, 1, 6, 1), (5, 2, 1, 1), (64, 8, 8, 4),
                                                     (4, 4, 2, 2), (40, 34, 2, 2)])
def test_router_with_selection_bias_and_group_limit(experts, top, groups, keep):
    from lite_llama_b200.kernels import route_sigmoid_groups

    T, k = 23, 37
    x = torch.randn(T, k)
    wr = torch.randn(experts, k) * 0.5
    bias = torch.randn(experts) * 0.8 - 0.9                  # mostly negative choice scores: a dropped group is not "0"
    wts, ids = route_sigmoid_groups(x.to(DEV), wr.to(DEV), bias.to(DEV), top, groups, keep)
    spec = {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}
    for t in range(T):
        chosen, weights = O.route(O.f64(x[t]), O.f64(wr), O.f64(bias), spec)
        assert ids[t].tolist() == chosen
        _close(wts[t], weights, 2e-6)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-6), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("experts,top,ff,hidden,shared", [(8, 3, 12, 48, 20), (3, 1, 70, 33, 0), (16, 4, 8, 16, 8)])
def test_routed_experts_and_the_shared_one(dtype, tol, experts, top, ff, hidden, shared):
    from lite_llama_b200.kernels import gelu, grouped_experts, linear_simt

    T = 41
    x = torch.randn(T, hidden).to(dtype)
    up = (torch.randn(experts, ff, hidden) / math.sqrt(hidden)).to(dtype)
    down = (torch.randn(experts, hidden, ff) / math.sqrt(ff)).to(dtype)
    ids = torch.stack([torch.randperm(experts)[:top] for _ in range(T)]).to(torch.int32)
    ids[:5] = torch.arange(top, dtype=torch.int32)            # one expert with many tokens, some with none
    wts = torch.rand(T, top)
    add = None
    ref = np.zeros((T, hidden))
    for t in range(T):
        for j in range(top):
            e = int(ids[t, j])
            ref[t] += float(wts[t, j]) * O.expert(O.f64(x[t]), O.f64(up[e]), O.f64(down[e]))
    if shared:
        su, sd = (torch.randn(shared, hidden) / math.sqrt(hidden)).to(dtype), (torch.randn(hidden, shared) / 4).to(dtype)
        add = linear_simt(gelu(linear_simt(x.to(DEV), su.to(DEV))), sd.to(DEV))
        ref += np.stack([O.expert(O.f64(x[t]), O.f64(su), O.f64(sd)) for t in range(T)])
    out = grouped_experts(x.to(DEV), up.to(DEV), down.to(DEV), wts.to(DEV), ids.to(DEV), addend=add)
    _close(out, ref, tol)
    # a token's result does not depend on the rest of the batch
    alone = grouped_experts(x[7:8].to(DEV), up.to(DEV), down.to(DEV), wts[7:8].to(DEV), ids[7:8].to(DEV),
                            addend=None if add is None else add[7:8])
    assert torch.equal(alone, out[7:8])


# ------------------------------------------------------------------------------------------------ whole models #
def _small():
    a = O.mixer_entry()                                                     # nothing equal to anything else
    b = O.mixer_entry(heads=2, dim=6, rot_dim=2, vdim=5, q_rank=9, kv_rank=7, window=3, base=50.0)
    return O.make_config([O.layer_entry(a, O.moe_entry()), O.layer_entry(b, None), O.layer_entry(a, O.moe_entry(), 0),
                          O.layer_entry(b, O.moe_entry(experts=6, top=1, groups=1, keep=1, ff=20, shared_ff=0)),
                          O.layer_entry(a, O.moe_entry(), 0)])


def _aligned(every_expert=False):
    # sizes in steps of 8: the tensor-core attention tiles in bf16; a window longer than a 64-key tile; the later
    # layer is the one that owns the weights
    a = O.mixer_entry(heads=4, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=24, window=70, base=1.0e6)
    b = O.mixer_entry(heads=2, dim=32, rot_dim=16, vdim=16, q_rank=32, kv_rank=48, window=16)
    big = O.moe_entry(experts=15, top=4, groups=5, keep=3, ff=24, shared_ff=32)
    little = O.moe_entry(experts=4, top=2, groups=2, keep=1, ff=16, shared_ff=8)
    if every_expert:                                        # top == experts: the router only weighs
        big = O.moe_entry(experts=3, top=3, groups=1, keep=1, ff=24, shared_ff=32)
        little = O.moe_entry(experts=2, top=2, groups=2, keep=2, ff=16, shared_ff=8)
    return O.make_config([O.layer_entry(a, big, 2), O.layer_entry(b, little), O.layer_entry(a, big)],
                         width=64, vocab=128, softcap=25.0)


def _ones():
    # one head, one expert, a window of one token, no rotated part, no soft cap
    a = O.mixer_entry(heads=1, dim=4, rot_dim=0, vdim=4, q_rank=4, kv_rank=4, window=1)
    b = O.mixer_entry(heads=1, dim=3, rot_dim=2, vdim=1, q_rank=1, kv_rank=1, window=2)
    return O.make_config([O.layer_entry(a, O.moe_entry(experts=1, top=1, groups=1, keep=1, ff=5, shared_ff=0)),
                          O.layer_entry(b, None)], width=10, vocab=17, softcap=0.0, embed_scale=1.0)


CONFIGS = {"small": _small, "aligned": _aligned, "ones": _ones, "aligned_every_expert": lambda: _aligned(True)}


def _runner(cfg, w, dtype=torch.float32, max_tokens=512, max_requests=4):
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.registry import lookup

    arch = lookup(cfg["architecture"])
    conf = arch.parse_config(cfg)
    return ModelRunner(conf, arch.map_weights(conf, w, DEV, dtype), max_tokens, device=DEV, dtype=dtype,
                       max_requests=max_requests)


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _feed(runner, req, toks, cuts):
    """Feed ``toks`` in portions of the given sizes (the rest one by one); logits of every position."""
    out, at = [], 0
    for n in list(cuts) + [1] * len(toks):
        if at >= len(toks):
            break
        part = toks[at:at + n]
        out.append(runner.forward_ragged([(req, part)], list(range(len(part)))))
        at += len(part)
    return torch.cat(out)


@pytest.mark.parametrize("name,length", [("small", 45), ("aligned", 150), ("ones", 20)])
def test_whole_prompt_portions_and_decoding_agree_with_the_restatement(name, length):
    cfg = CONFIGS[name]()
    w = O.random_model(cfg, seed=1)
    toks = _tokens(cfg, length, 2)
    ref = O.forward(cfg, w, toks)
    runner = _runner(cfg, w)
    for cuts in ([length], [length - 15], [], [2, 2, 3, 17, 2, 5], [1, length - 1], [7, 1, 1, 20], [64, 2, 63]):
        req = runner.open_request()
        _close(_feed(runner, req, toks, cuts), ref, 1e-4)
        runner.close_request(req)
    assert runner.kv_cache_manager.can_use_mem_size == runner.kv_cache_manager.max_num_tokens
    assert runner.state_manager.free_slots == 4


def test_layer_outputs_match_one_by_one():
    cfg = CONFIGS["small"]()
    w = O.random_model(cfg, seed=5)
    toks = _tokens(cfg, 12, 6)
    layers = []
    O.forward(cfg, w, toks, layers)
    runner = _runner(cfg, w)
    runner.model.layer_trace = []
    runner.forward_ragged([(runner.open_request(), toks)])
    assert len(runner.model.layer_trace) == len(layers) == 5
    for got, ref in zip(runner.model.layer_trace, layers):
        _close(got, ref, 2e-5)


def test_layers_that_share_weights_keep_caches_of_their_own():
    cfg = CONFIGS["small"]()
    from lite_llama_b200.executor.registry import lookup

    arch = lookup("Pesivik")
    conf = arch.parse_config(cfg)
    wts = arch.map_weights(conf, O.random_model(cfg, seed=2), DEV, torch.float32)
    assert wts.layers[2] is wts.layers[0] and wts.layers[4] is wts.layers[0] and wts.layers[1] is not wts.layers[3]
    runner = _runner(cfg, O.random_model(cfg, seed=2))
    pools = runner.kv_cache_manager.gpu_kv_buffer
    assert len(pools) == 5 and len({p.data_ptr() for p in pools}) == 5
    assert [p.shape[1] for p in pools] == [16, 16, 16, 16, 16]           # [latent | rotated part] padded to 8 columns


def test_unequal_batches_match_each_request_alone_and_reuse_rows_and_slots():
    """Six requests through four slots and a pool smaller than their sum: portions beside single tokens, requests
    leaving and joining, rows and slots changing hands; every logit equals the request's own restatement."""
    cfg = CONFIGS["small"]()
    w = O.random_model(cfg, seed=7)
    lens = [40, 3, 25, 1, 31, 18]
    toks = [_tokens(cfg, n, 10 + i) for i, n in enumerate(lens)]
    refs = [O.forward(cfg, w, t) for t in toks]
    runner = _runner(cfg, w, max_tokens=96, max_requests=4)
    plan = {0: [5, 2, 1, 1, 9, 1, 1, 1, 1, 1, 1, 16], 1: [2, 1], 2: [1, 1, 20, 1, 1, 1], 3: [1],
            4: [16, 2, 2, 1, 1, 1, 1, 1, 6], 5: [3, 3, 3, 3, 3, 3]}
    waiting, live, fed, got = [0, 1, 2, 3, 4, 5], {}, {i: 0 for i in plan}, {i: [] for i in plan}
    steps, seen_rows = 0, set()
    while waiting or live:
        while waiting and len(live) < 4 and runner.kv_cache_manager.can_use_mem_size >= sum(
                lens[i] - fed[i] for i in live) + lens[waiting[0]]:
            live[waiting.pop(0)] = runner.open_request()
        order = sorted(live, key=lambda i: (i * 7 + steps) % 5)               # the batch order changes every step
        entries, want, at, shape = [], [], 0, []
        for i in order:
            n = plan[i].pop(0) if plan[i] else 1
            n = min(n, lens[i] - fed[i])
            entries.append((live[i], toks[i][fed[i]:fed[i] + n]))
            want += list(range(at, at + n))
            at += n
            shape.append((i, n))
        logits = runner.forward_ragged(entries, want)
        at = 0
        for i, n in shape:
            got[i].append(logits[at:at + n])
            at += n
            fed[i] += n
            if fed[i] == lens[i]:
                seen_rows.update(live[i].rows)
                runner.close_request(live.pop(i))
        steps += 1
    for i in plan:
        _close(torch.cat(got[i]), refs[i], 1e-4)
    assert runner.kv_cache_manager.can_use_mem_size == 96 and sum(lens) > 96 >= len(seen_rows)


def test_long_decoding_carries_the_window_over_decoded_tokens_and_key_range_edges():
    a = O.mixer_entry(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=8, kv_rank=8, window=150)
    b = O.mixer_entry(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=8, kv_rank=8, window=33)
    cfg = O.make_config([O.layer_entry(a, None), O.layer_entry(b, O.moe_entry(experts=4, top=2, groups=2, keep=1, ff=8,
                                                                            shared_ff=0))], width=16, vocab=40)
    w = O.random_model(cfg, seed=9)
    toks = _tokens(cfg, 420, 3)
    ref = O.forward(cfg, w, toks)
    runner = _runner(cfg, w, max_tokens=448)
    got = _feed(runner, runner.open_request(), toks, [100])       # 320 tokens decoded one by one: 1 -> 2 key ranges
    _close(got, ref, 1e-4)


def test_rows_outside_every_window_return_to_the_pool_while_the_request_runs():
    """Every layer has a window, so a running request holds only the rows a later token can still see (the longest
    window and one key tile of slack): two sequences of 400 and 300 tokens run side by side through a pool of 256 rows,
    in portions and token by token, and every logit equals the restatement."""
    a = O.mixer_entry(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=8, kv_rank=12, window=33)
    b = O.mixer_entry(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=8, kv_rank=4, window=20)
    cfg = O.make_config([O.layer_entry(a, None), O.layer_entry(b, O.moe_entry(experts=4, top=2, groups=2, keep=1, ff=8,
                                                                            shared_ff=0))], width=16, vocab=40)
    w = O.random_model(cfg, seed=17)
    toks = [_tokens(cfg, 400, 5), _tokens(cfg, 300, 6)]
    refs = [O.forward(cfg, w, t) for t in toks]
    runner = _runner(cfg, w, max_tokens=256, max_requests=2)
    assert runner.keep_positions == 32 + 64
    reqs = [runner.open_request(), runner.open_request()]
    plans = [[20, 3, 17, 2] * 4 + [1] * 400, [1, 30, 1, 9] * 5 + [1] * 300]
    fed, got = [0, 0], [[], []]
    while fed[0] < 400 or fed[1] < 300:
        entries, want, at, shape = [], [], 0, []
        for i in (0, 1):
            if fed[i] < len(toks[i]):
                n = min(plans[i].pop(0), len(toks[i]) - fed[i])
                entries.append((reqs[i], toks[i][fed[i]:fed[i] + n]))
                want += list(range(at, at + n))
                at += n
                shape.append((i, n))
        logits = runner.forward_ragged(entries, want)
        at = 0
        for i, n in shape:
            got[i].append(logits[at:at + n])
            at += n
            fed[i] += n
            assert runner.rows_held(reqs[i]) <= 96 + n
    for i in (0, 1):
        _close(torch.cat(got[i]), refs[i], 1e-4)
        runner.close_request(reqs[i])
    assert runner.kv_cache_manager.can_use_mem_size == 256


def test_a_far_key_outside_the_window_is_forgotten_and_one_inside_is_found():
    """The model as a whole: changing a token that lies outside every layer's reach leaves the logits of the last
    position untouched, changing one inside the first layer's window does not."""
    a = O.mixer_entry(window=7)
    cfg = O.make_config([O.layer_entry(a, O.moe_entry()), O.layer_entry(a, O.moe_entry(), 0)])
    w = O.random_model(cfg, seed=4)
    toks = _tokens(cfg, 60, 8)
    runner = _runner(cfg, w)

    def last(seq, cuts):
        req = runner.open_request()
        out = _feed(runner, req, seq, cuts)[-1].double().cpu()
        runner.close_request(req)
        return out

    base = last(toks, [60])
    far = list(toks)
    far[59 - 13] = (far[59 - 13] + 1) % cfg["vocab"]            # two layers of window 7 reach back 12 positions at most
    near = list(toks)
    near[59 - 12] = (near[59 - 12] + 1) % cfg["vocab"]
    for cuts in ([60], [50], [30, 2, 20]):
        _close(last(far, cuts), base, 1e-5)
        assert (last(near, cuts) - base).abs().max().item() > 1e-4


@pytest.mark.parametrize("name,length,cuts", [("small", 40, [13, 2, 9]), ("aligned", 150, [70, 3, 66]),
                                              ("aligned_every_expert", 150, [70, 3, 66])])
def test_bf16_serving_precision_stays_within_a_few_roundings(name, length, cuts):
    """Where every expert is used there is no choice to make and every position stays within a few roundings.  With a
    real choice, a token whose best candidates lie closer together than the rounding of the router's input may take
    another expert (and the positions that see it follow): those few positions are allowed to differ."""
    cfg = CONFIGS[name]()
    w = O.random_model(cfg, seed=11)
    toks = _tokens(cfg, length, 12)
    ref = torch.as_tensor(O.forward(cfg, w, toks))
    for plan in (cuts, [length]):
        runner = _runner(cfg, w, dtype=torch.bfloat16)
        got = _feed(runner, runner.open_request(), toks, plan)
        assert got.dtype == torch.float32                    # soft-capped logits leave in fp32
        d = got.double().cpu() - ref
        rel = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / ref.std()
        assert rel.median().item() < 0.02, rel.median().item()
        if name.endswith("every_expert"):
            assert rel.max().item() < 0.06, rel.max().item()
        else:
            assert (rel > 0.06).double().mean().item() <= 0.1, rel


def test_captured_decode_steps_equal_eager_ones():
    cfg = CONFIGS["aligned"]()
    w = O.random_model(cfg, seed=21)
    prompts = [_tokens(cfg, n, 30 + n) for n in (70, 5, 33)]
    tails = [_tokens(cfg, 12, 40 + i) for i in range(3)]
    outs = []
    for graphs in (False, True):
        runner = _runner(cfg, w, max_tokens=256, max_requests=3)
        if graphs:
            runner.enable_ragged_decode_graphs(ctx_buckets=(64, 256))
            assert runner._ragged_graphs
        reqs = [runner.open_request() for _ in prompts]
        got = [runner.forward_ragged([(r, p) for r, p in zip(reqs, prompts)])]
        for step in range(12):
            live = [i for i in range(3) if not (i == 1 and step >= 6)]          # request 1 leaves half way
            if step == 6:
                runner.close_request(reqs[1])
            got.append(runner.forward_ragged([(reqs[i], [tails[i][step]]) for i in live]).clone())
        outs.append(torch.cat(got).float().cpu())
    _close(outs[1], outs[0], 1e-5)
    ref = O.forward(cfg, w, prompts[0] + tails[0])
    _close(outs[1][[0] + [3 + 3 * k for k in range(6)]], ref[[69] + [70 + k for k in range(6)]], 1e-4)


def test_checkpoint_directory_and_greedy_generation_through_the_engine(tmp_path):
    import json

    from lite_llama_b200.engine import Engine
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.checkpoint import write_safetensors

    cfg = CONFIGS["small"]()
    w = O.random_model(cfg, seed=13, spread=2.0)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    runner = ModelRunner.from_checkpoint(tmp_path, dtype=torch.float32, max_tokens=160, max_requests=3)
    prompts = [_tokens(cfg, n, 20 + n) for n in (9, 1, 30, 4, 17)]
    new = 12
    engine = Engine(runner, max_step_tokens=16, max_portion=7)        # portions of 7 beside decoding requests
    outs = engine.generate(prompts, new)
    for p, out in zip(prompts, outs):
        seq = list(p)
        for t in out:
            logits = torch.as_tensor(O.forward(cfg, w, seq)[-1])
            top2 = logits.topk(2).values
            if (top2[0] - top2[1]).item() < 1e-3:
                break                                                  # undecidable at fp32: stop comparing this one
            assert t == int(logits.argmax()), "greedy token differs from the restatement"
            seq.append(t)
    assert engine.steps > 12 and runner.state_manager.free_slots == 3
    assert runner.kv_cache_manager.can_use_mem_size == 160


@pytest.mark.parametrize("graphs", [False, True])
def test_engine_generates_past_the_pool_size_when_every_layer_has_a_window(graphs):
    """Two requests of 30 + 150 tokens each through a pool of 200 rows: admission counts what the windows keep, the
    runner gives unseen rows back, and the greedy tokens follow the restatement."""
    from lite_llama_b200.engine import Engine

    a = O.mixer_entry(window=7)
    cfg = O.make_config([O.layer_entry(a, O.moe_entry()), O.layer_entry(a, O.moe_entry(), 0)])
    w = O.random_model(cfg, seed=23, spread=2.0)
    runner = _runner(cfg, w, max_tokens=200, max_requests=2)
    engine = Engine(runner, max_step_tokens=32, max_portion=8, decode_graphs=graphs)      # replayed decode steps too
    prompts = [_tokens(cfg, 30, 50), _tokens(cfg, 30, 51)]
    outs = engine.generate(prompts, 150)
    assert [len(o) for o in outs] == [150, 150] and runner.kv_cache_manager.can_use_mem_size == 200
    for p, out in zip(prompts, outs):
        seq = list(p)
        for t in out[:40]:
            logits = torch.as_tensor(O.forward(cfg, w, seq)[-1])
            top2 = logits.topk(2).values
            if (top2[0] - top2[1]).item() < 1e-3:
                break
            assert t == int(logits.argmax())
            seq.append(t)


# ------------------------------------------------------------------------------------- random models and schedules #
def _random_config(rng, odd):
    def mixer():
        return O.mixer_entry(heads=rng.choice([1, 2, 3, 5, 6, 8]), dim=rng.choice([8, 12, 24, 32, 40, 64]),
                             rot_dim=rng.choice([0, 2, 4, 8, 16, 32]), vdim=rng.choice([8, 10, 24, 40, 80]),
                             q_rank=rng.choice([5, 30, 57] if odd else [8, 24, 56, 96]),
                             kv_rank=rng.choice([4, 8, 20, 40, 64, 72, 128]),
                             window=rng.choice([1, 2, 5, 16, 33, 64, 65, 100, 128, 200, 1000]),
                             base=rng.choice([100.0, 10000.0, 1.0e6]))

    def mlp():
        if rng.random() < 0.2:
            return None
        groups, per = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 4])
        keep = rng.randint(1, groups)
        return O.moe_entry(experts=groups * per, top=rng.randint(1, keep * per), groups=groups, keep=keep,
                           ff=rng.choice([8, 12, 40, 96]), shared_ff=rng.choice([0, 16, 40]))

    kinds = [(mixer(), mlp()) for _ in range(rng.randint(1, 2))]
    layers, owner = [], {}
    for i in range(rng.randint(2, 5)):
        k = rng.randrange(len(kinds))
        if k in owner and rng.random() < 0.7:
            layers.append(O.layer_entry(kinds[k][0], kinds[k][1], owner[k]))
        else:
            layers.append(O.layer_entry(kinds[k][0], kinds[k][1]))
            owner.setdefault(k, i)
    return O.make_config(layers, width=rng.choice([50, 92, 37, 129] if odd else [16, 40, 72, 136, 200]),
                         vocab=rng.choice([33, 1001] if odd else [17, 64, 300]), eps=rng.choice([1e-5, 1e-6, 1e-3]),
                         embed_scale=rng.choice([0.5, 1.0, 2.0]), softcap=rng.choice([0.0, 10.0, 30.0]))


@pytest.mark.parametrize("seed", range(8))
def test_random_models_under_random_mixed_schedules(seed):
    """Random sizes (odd widths, ranks and vocabularies on the odd seeds), layer orders with shared layers, windows from
    1 to beyond the sequences; up to four requests fed in random portions beside one another through a pool of exactly
    their size, the tails token by token.  fp32 logits equal the restatement; the bf16 run completes and stays close
    for the typical position (a token may take another expert where its best candidates nearly tie)."""
    rng = random.Random(seed)
    cfg = _random_config(rng, odd=seed % 2 == 1)
    w = O.random_model(cfg, seed=seed)
    lens = [rng.choice([1, 5, 23, 60, 97, 150])] + [rng.choice([30, 90, 130]) for _ in range(rng.randint(1, 3))]
    toks = [_tokens(cfg, n, seed * 10 + i) for i, n in enumerate(lens)]
    refs = [O.forward(cfg, w, t) for t in toks]
    plan, fed = [], [0] * len(lens)
    while any(f < n for f, n in zip(fed, lens)):
        step = []
        for i, n in enumerate(lens):
            if fed[i] < n and rng.random() < 0.8:
                left = n - fed[i]
                c = 1 if left <= 20 else min(left - 20, rng.choice([1, 2, 3, 7, 16, 29, 64, 66, 128]))
                step.append((i, c))
                fed[i] += c
        if step:
            plan.append(step)
    pool = -(-sum(lens) // 64) * 64
    for dtype in (torch.float32, torch.bfloat16):
        runner = _runner(cfg, w, dtype=dtype, max_tokens=pool)
        got, reqs, fed = [[] for _ in lens], {}, [0] * len(lens)
        for step in plan:
            entries, want, at = [], [], 0
            for i, c in step:
                if i not in reqs:
                    reqs[i] = runner.open_request()
                entries.append((reqs[i], toks[i][fed[i]:fed[i] + c]))
                want += list(range(at, at + c))
                at += c
            logits = runner.forward_ragged(entries, want).float().cpu()
            at = 0
            for i, c in step:
                got[i].append(logits[at:at + c])
                at += c
                fed[i] += c
                if fed[i] == lens[i]:
                    runner.close_request(reqs.pop(i))
        assert runner.kv_cache_manager.can_use_mem_size == pool
        for i in range(len(lens)):
            if dtype == torch.float32:
                _close(torch.cat(got[i]), refs[i], 1e-4)
            else:
                d = torch.cat(got[i]).double() - torch.as_tensor(refs[i])
                rel = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / max(float(refs[i].std()), 1e-9)
                assert rel.median().item() < 0.08, rel.median().item()

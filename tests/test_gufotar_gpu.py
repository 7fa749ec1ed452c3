"""The Gufotar path on the GPU against the plain restatement in ``gufotar_oracle`` (float64, token loops): every
mechanism alone through its kernel, then whole models through ``ModelRunner.forward_ragged`` and the engine --
prompts against token-by-token decoding, portions down to two tokens, unequal batches against each request alone,
pool rows and state slots that change hands, keys far back and at the split edges, long decoding, odd sizes.
fp32 runs are held to 1e-4 of the logits' spread; bf16 runs to a few bf16 roundings."""

from __future__ import annotations

import math

import pytest
import torch

import gufotar_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]
DEV = "cuda"


def _cuda(t, dtype):
    return t.to(device=DEV, dtype=dtype).contiguous()


def _i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def _close(got, ref, tol):
    got, ref = got.double().cpu(), ref.double()
    err = (got - ref).abs().max().item()
    spread = max(ref.abs().max().item(), 1e-6)
    assert err <= tol * spread, f"max abs err {err:.3e} on values up to {spread:.3e} (tol {tol})"


# ------------------------------------------------------------------------------------------- mechanisms alone #
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (37, 130, 36), (130, 65, 200)])
def test_simt_gemm(dtype, tol, m, n, k):
    from lite_llama_b200.kernels import linear_simt

    x, w = torch.randn(m, k).to(dtype), torch.randn(n, k).to(dtype)
    y = linear_simt(x.to(DEV), w.to(DEV))
    _close(y, x.double() @ w.double().t(), tol)
    # a row's result does not depend on the rest of the batch
    assert torch.equal(linear_simt(x[:1].to(DEV), w.to(DEV)), y[:1])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_residual_stream_ops(dtype, tol):
    from lite_llama_b200.kernels import embed_positions, post_norm_residual, relu_squared, rmsnorm_from_f32

    n, vocab, npos, eps = 44, 30, 20, 1e-5
    embed, pos = torch.randn(vocab, n).to(dtype), torch.randn(npos, n).to(dtype)
    toks, ps = [3, 29, 0, 7, 7], [0, 19, 5, 6, 1]
    r, act = embed_positions(_i32(toks), _i32(ps), embed.to(DEV), pos.to(DEV))
    ref = embed.double()[toks] + pos.double()[ps]
    _close(r, ref, 1e-6)
    assert (act is None) == (dtype == torch.float32)
    y, w = torch.randn(5, n).to(dtype), (torch.randn(n) * 0.3).to(dtype)
    post_norm_residual(r, y.to(DEV), w.to(DEV), eps)
    ref = ref + O.zero_centred_norm(y.double(), w.double(), eps)
    _close(r, ref, 2e-6)
    out = rmsnorm_from_f32(r, w.to(DEV), eps, 1.0, _i32([4, 1]))
    _close(out, O.zero_centred_norm(ref, w.double(), eps)[[4, 1]], tol)
    _close(relu_squared(y.to(DEV)), torch.relu(y.double()) ** 2, tol)


@pytest.mark.parametrize("taps,c,extra", [(1, 37, 5), (2, 37, 5), (4, 37, 5), (5, 37, 5), (4, 40, 8), (3, 8, 0)])
def test_causal_conv_with_tail_over_portions(taps, c, extra):
    """Odd channel counts take the scalar kernel, multiples of 4 with an aligned column window the 16-byte one."""
    from lite_llama_b200.kernels import causal_conv_silu

    w, b = torch.randn(c, taps) * 0.5, torch.randn(c) * 0.1
    seqs = {0: torch.randn(11, c), 2: torch.randn(6, c), 1: torch.randn(1, c)}        # slot -> inputs
    ref = {s: O.silu(O.causal_conv(u.double(), w.double(), b.double())[0]) for s, u in seqs.items()}
    tail = torch.full((3, max(taps - 1, 1), c), 7.0, device=DEV)        # stale contents must not leak in
    fed = {s: 0 for s in seqs}
    for portion in ({0: 1, 2: 2}, {0: 2, 2: 1, 1: 1}, {0: 5}, {2: 3, 0: 3}):
        slots = list(portion)
        rows = torch.cat([seqs[s][fed[s]:fed[s] + portion[s]] for s in slots])
        proj = torch.cat([torch.randn(rows.shape[0], extra), rows], 1).to(DEV)      # the conv input is a column window
        starts = [0]
        for s in slots:
            starts.append(starts[-1] + portion[s])
        out = causal_conv_silu(proj, extra, c, w.to(DEV), b.to(DEV), tail, _i32(starts), _i32(fed[s] for s in slots),
                               _i32(slots))
        want = torch.cat([ref[s][fed[s]:fed[s] + portion[s]] for s in slots])
        _close(out, want, 2e-6)
        for s in slots:
            fed[s] += portion[s]


@pytest.mark.parametrize("heads,groups,state,hd", [(4, 2, 12, 6), (3, 1, 48, 7), (2, 2, 100, 16), (2, 1, 130, 4),
                                                   (1, 1, 1, 1), (2, 1, 40, 70), (2, 2, 130, 40), (1, 1, 400, 33),
                                                   (2, 1, 16, 64)])
def test_ssm_scan_carries_state_between_steps(heads, groups, state, hd):
    from lite_llama_b200.kernels import ssm_scan

    T = 23
    inner, gn = heads * hd, groups * state
    xbc = torch.randn(T, inner + 2 * gn)
    dt_raw = torch.randn(T, heads) * 2
    dt_bias, a_log, d = torch.randn(heads), torch.randn(heads), torch.randn(heads)
    y_ref, s_ref = O.ssm_recurrence(xbc[:, :inner].double().view(T, heads, hd), O.softplus(dt_raw.double() + dt_bias.double()),
                                    a_log.double(), xbc[:, inner:inner + gn].double().view(T, groups, state),
                                    xbc[:, inner + gn:].double().view(T, groups, state), d.double())
    st = torch.full((2, heads, state, hd), 3.0, device=DEV)
    got, at = [], 0
    for n in (1, 2, 9, 1, 10):                         # slot 1; an unrelated one-token sequence shares every step
        other = torch.randn(1, inner + 2 * gn)
        step_x = torch.cat([other, xbc[at:at + n]]).to(DEV)
        step_dt = torch.cat([torch.randn(1, heads), dt_raw[at:at + n]]).to(DEV)
        y = ssm_scan(step_x, step_dt, dt_bias.to(DEV), a_log.to(DEV), d.to(DEV), st, _i32([0, 1, 1 + n]), _i32([0, at]),
                     _i32([0, 1]), heads, groups, state, hd)
        got.append(y[1:])
        at += n
    _close(torch.cat(got), y_ref.reshape(T, inner), 5e-6)
    _close(st[1], s_ref, 5e-6)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("groups", [1, 3])
def test_gated_group_norm(dtype, tol, groups):
    from lite_llama_b200.kernels import gated_group_norm

    y, z, w = torch.randn(5, 48), torch.randn(5, 48).to(dtype), torch.randn(48).to(dtype)
    proj = torch.cat([z, torch.zeros(5, 3, dtype=dtype)], 1).to(DEV)
    out = gated_group_norm(y.to(DEV), proj[:, :48], w.to(DEV), groups, 1e-5)
    _close(out, O.grouped_gated_norm(y.double(), z.double(), w.double(), groups, 1e-5), tol)


def _attention_case(H, G, D, Dv, lens_ctx, softcap, with_sink, dtype, scale=0.3, boost=None, seed=0):
    """Fill the pool for sequences with ``ctx`` cached tokens, run ``new`` more through prepare + attention, and return
    (kernel output, oracle output) for the new tokens.  ``boost`` = (seq, key position, factor) scales one cached key."""
    from lite_llama_b200.kernels import attn_prepare, sink_attention

    g = torch.Generator().manual_seed(seed)
    nseq = len(lens_ctx)
    max_seq = max(c + n for n, c in lens_ctx)
    total_rows = sum(c + n for n, c in lens_ctx)
    perm = torch.randperm(total_rows + 5, generator=g)              # scattered pool rows
    pool = torch.zeros(total_rows + 5, G * (D + Dv), dtype=dtype, device=DEV)
    table = torch.zeros(nseq + 1, max_seq, dtype=torch.int32, device=DEV)
    slots = list(range(nseq, 0, -1))                                 # slot != sequence index
    qn, kn, vn = H * D, G * D, G * Dv
    qw, kw = (1 + 0.2 * torch.randn(qn, generator=g)).to(dtype), (1 + 0.2 * torch.randn(kn, generator=g)).to(dtype)
    sink = (torch.randn(H, generator=g) * 2).to(dtype) if with_sink else None
    seqs, at = [], 0
    for i, (n, c) in enumerate(lens_ctx):
        qkv = torch.randn(c + n, qn + kn + vn, generator=g).to(dtype)
        if boost and boost[0] == i:
            qkv[boost[1], qn:qn + kn] *= boost[2]
        rows = perm[at:at + c + n].to(torch.int32)
        at += c + n
        table[slots[i], :c + n] = rows.to(DEV)
        seqs.append((qkv, rows))
    eps, coef, every = 1e-5, 0.5, 3.0

    def prep(qkv, rows, pos):
        buf = qkv.to(DEV).clone()
        attn_prepare(buf, pool, rows.to(DEV), _i32(pos), qn, kn, vn, qw.to(DEV), kw.to(DEV), eps, coef, every)
        return buf

    for (n, c), (qkv, rows) in zip(lens_ctx, seqs):                  # the cached part
        if c:
            prep(qkv[:c], rows[:c], range(c))
    new_q = torch.cat([prep(qkv[c:], rows[c:], range(c, c + n)) for (n, c), (qkv, rows) in zip(lens_ctx, seqs)])
    starts = [0]
    for n, _ in lens_ctx:
        starts.append(starts[-1] + n)
    out = torch.zeros(starts[-1], H * Dv, dtype=dtype, device=DEV)
    args = (_i32(starts), _i32(c for _, c in lens_ctx), _i32(slots))
    portions = [i for i, (n, _) in enumerate(lens_ctx) if n > 1]
    singles = [i for i, (n, _) in enumerate(lens_ctx) if n == 1]
    geo = (H, G, D, Dv, scale, softcap)
    if portions:
        sink_attention(out, new_q, pool, table, *args, _i32(portions), len(portions),
                       max(lens_ctx[i][0] for i in portions), _cuda(sink, dtype) if with_sink else None, *geo)
    if singles:
        keys = max(lens_ctx[i][1] for i in singles) + 1
        splits = max(1, -(-keys // 64))
        sink_attention(out, new_q, pool, table, *args, _i32(singles), len(singles), 1,
                       _cuda(sink, dtype) if with_sink else None, *geo, num_splits=splits, split_keys=64)
    refs = []
    for (n, c), (qkv, _) in zip(lens_ctx, seqs):
        x = qkv.double()
        pos = torch.arange(c + n)
        q = O.rms_unit(x[:, :qn], eps) * qw.double() * O.query_temperature(pos, {"coef": coef, "every": every})[:, None]
        k = O.rms_unit(x[:, qn:qn + kn], eps) * kw.double()
        if dtype != torch.float32:                                   # what the cache and the q buffer hold
            q, k = q.to(dtype).double(), k.to(dtype).double()
        v = x[:, qn + kn:]
        o = O.sink_attention(q[c:].view(n, H, D), k.view(-1, G, D), v.view(-1, G, Dv), pos[c:], pos, scale, softcap,
                             sink.double() if with_sink else None)
        refs.append(o.reshape(n, H * Dv))
    return out, torch.cat(refs)


@pytest.mark.parametrize("H,G,D,Dv", [(4, 4, 16, 16), (6, 2, 24, 40), (8, 1, 32, 20), (20, 1, 8, 72), (3, 3, 80, 130)])
@pytest.mark.parametrize("softcap,with_sink", [(0.0, False), (5.0, True)])
def test_sink_attention_portions_and_single_tokens(H, G, D, Dv, softcap, with_sink):
    # portions with and without a cached prefix, a first token, decode tokens right at and around the 64-key split edge
    cases = [(9, 0), (1, 0), (5, 30), (1, 63), (1, 64), (2, 17), (1, 130), (33, 31), (1, 5)]
    out, ref = _attention_case(H, G, D, Dv, cases, softcap, with_sink, torch.float32)
    _close(out, ref, 1e-5)


@pytest.mark.parametrize("H,G,D,Dv", [(8, 2, 32, 48), (8, 1, 64, 48), (4, 2, 128, 128), (4, 4, 16, 16), (6, 2, 24, 40),
                                      (2, 1, 72, 104), (3, 3, 20, 12)])
def test_sink_attention_bf16(H, G, D, Dv):
    """16-bit activations: the tensor-core tiled kernel where the head sizes allow it (steps of 8 up to 128), the
    CUDA-core one otherwise; tiles of 64 tokens and 64 keys are crossed with and without a cached prefix."""
    cases = [(7, 0), (1, 40), (12, 70), (70, 3), (130, 64), (64, 0), (65, 63), (1, 0)]
    out, ref = _attention_case(H, G, D, Dv, cases, 10.0, True, torch.bfloat16)
    _close(out, ref, 2e-2)
    out, ref = _attention_case(H, G, D, Dv, cases[:4], 0.0, False, torch.bfloat16, seed=4)
    _close(out, ref, 2e-2)


@pytest.mark.parametrize("new,ctx,key", [(1, 700, 3), (1, 700, 255), (1, 700, 256), (40, 600, 0), (40, 600, 599)])
def test_a_far_key_among_hundreds_is_found(new, ctx, key):
    """One cached key is scaled up so that (for the heads whose score with it is positive and soft-capped to the top)
    it owns the softmax; a kernel that skips it, or any key range, cannot match the restatement."""
    out, ref = _attention_case(4, 2, 16, 8, [(new, ctx), (1, 9)], 30.0, False, torch.float32, scale=1.0,
                               boost=(0, key, 40.0))
    _close(out, ref, 1e-5)


def test_the_sink_takes_its_share():
    """With a large sink most of the probability mass has no value: outputs shrink by the factor the restatement
    gives, both in the tiled and in the split kernel."""
    out, ref = _attention_case(2, 1, 16, 8, [(6, 0), (1, 100)], 0.0, True, torch.float32, scale=0.05, seed=3)
    _close(out, ref, 1e-5)
    plain, _ = _attention_case(2, 1, 16, 8, [(6, 0), (1, 100)], 0.0, False, torch.float32, scale=0.05, seed=3)
    assert (out.abs().mean() < 0.98 * plain.abs().mean()).item()


def test_value_mixing_and_unmixed_copy():
    from lite_llama_b200.kernels import attn_prepare

    qn, kn, vn, T = 16, 8, 12, 5
    qkv = torch.randn(T, qn + kn + vn)
    first = torch.randn(T, vn)
    lam = torch.tensor([0.3])
    pool = torch.zeros(9, kn + vn, device=DEV)
    rows = _i32([8, 2, 4, 0, 5])
    keep = torch.zeros(T, vn, device=DEV)
    attn_prepare(qkv.to(DEV), pool, rows, _i32(range(T)), qn, kn, vn, None, None, 1e-5, 0.0, 0.0, first.to(DEV), keep,
                 lam.to(DEV))
    v = qkv[:, qn + kn:]
    _close(keep, v, 0)
    _close(pool[rows.long(), kn:], 0.7 * v.double() + 0.3 * first.double(), 1e-6)
    _close(pool[rows.long(), :kn], qkv[:, qn:qn + kn], 0)            # no norm weight: keys are stored as they are


# ------------------------------------------------------------------------------------------------ whole models #
CONFIGS = {
    "mixed": lambda: O.make_config([O.mamba2_layer(), O.attention_layer(), O.attention_layer(heads=6, kv_heads=6, dim=8,
                                    vdim=8, every=4, ff=0), O.mamba2_layer(heads=2, vdim=20, state=40, groups=1,
                                    norm_groups=1, conv=2, ff=56), O.attention_layer(kv_heads=1, vdim=48, softcap=0.0)]),
    "odd_width": lambda: O.make_config([O.attention_layer(heads=3, kv_heads=1, dim=20, vdim=12, ff=50),
                                        O.mamba2_layer(heads=5, vdim=4, state=33, groups=5, norm_groups=5, conv=5),
                                        O.attention_layer(heads=2, kv_heads=2, dim=12, vdim=36, v_mix=False)],
                                       width=36, vocab=61),
    # sizes in steps of 8: the 16-byte kernels, the tensor-core attention tiles (bf16), two columns per lane in the scan
    "aligned": lambda: O.make_config([O.mamba2_layer(heads=4, vdim=40, state=24, groups=2, norm_groups=2, conv=4, ff=64),
                                      O.attention_layer(heads=4, kv_heads=2, dim=32, vdim=40, every=16),
                                      O.attention_layer(heads=8, kv_heads=1, dim=16, vdim=80, every=16, ff=0)],
                                     width=64, vocab=128),
    "recurrent_only": lambda: O.make_config([O.mamba2_layer(ff=32), O.mamba2_layer(groups=1, norm_groups=1, conv=4)]),
    "attention_only": lambda: O.make_config([O.attention_layer(), O.attention_layer(v_mix=False, ff=0),
                                             O.attention_layer()], width=48),
}


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


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_portions_and_decoding_agree_with_the_restatement(name):
    cfg = CONFIGS[name]()
    w = O.random_model(cfg, seed=1)
    toks = _tokens(cfg, 45, 2)
    ref = O.Oracle(cfg, w).forward(toks)
    runner = _runner(cfg, w)
    for cuts in ([45], [30], [], [2, 2, 3, 17, 2, 5], [1, 44], [7, 1, 1, 20]):
        req = runner.open_request()
        _close(_feed(runner, req, toks, cuts), ref, 1e-4)
        runner.close_request(req)
    assert runner.kv_cache_manager.can_use_mem_size == runner.kv_cache_manager.max_num_tokens
    assert runner.state_manager.free_slots == 4


def test_layer_outputs_match_one_by_one():
    cfg = CONFIGS["mixed"]()
    w = O.random_model(cfg, seed=5)
    toks = _tokens(cfg, 12, 6)
    _, layers = O.Oracle(cfg, w).forward(toks, keep_layers=True)
    runner = _runner(cfg, w)
    runner.model.layer_trace = []
    runner.forward_ragged([(runner.open_request(), toks)])
    for got, ref in zip(runner.model.layer_trace, layers):
        _close(got, ref, 2e-5)


def test_unequal_batches_match_each_request_alone_and_reuse_rows_and_slots():
    """Six requests through four slots and a pool smaller than their sum: portions beside single tokens, requests
    leaving and joining, rows and slots changing hands; every logit equals the request's own restatement."""
    cfg = CONFIGS["mixed"]()
    w = O.random_model(cfg, seed=7)
    lens = [40, 3, 25, 1, 31, 18]
    toks = [_tokens(cfg, n, 10 + i) for i, n in enumerate(lens)]
    orc = O.Oracle(cfg, w)
    refs = [orc.forward(t, seq=i) for i, t in enumerate(toks)]
    runner = _runner(cfg, w, max_tokens=96, max_requests=4)
    plan = {0: [5, 2, 1, 1, 9, 1, 1, 1, 1, 1, 1, 16], 1: [2, 1], 2: [1, 1, 20, 1, 1, 1], 3: [1],
            4: [16, 2, 2, 1, 1, 1, 1, 1, 6], 5: [3, 3, 3, 3, 3, 3]}
    waiting, live, fed, got = [0, 1, 2, 3, 4, 5], {}, {i: 0 for i in plan}, {i: [] for i in plan}
    steps = 0
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
                runner.close_request(live.pop(i))
        steps += 1
    for i in plan:
        _close(torch.cat(got[i]), refs[i], 1e-4)
    assert runner.kv_cache_manager.can_use_mem_size == 96


def test_long_decoding_crosses_key_split_edges():
    cfg = O.make_config([O.attention_layer(heads=2, kv_heads=1, dim=8, vdim=8, ff=0), O.mamba2_layer(heads=2, vdim=4,
                         state=8, groups=1, norm_groups=1)], width=16, vocab=40, max_positions=640)
    w = O.random_model(cfg, seed=9)
    toks = _tokens(cfg, 560, 3)
    ref = O.Oracle(cfg, w).forward(toks)
    runner = _runner(cfg, w, max_tokens=640)
    req = runner.open_request()
    got = _feed(runner, req, toks, [200])                    # 360 tokens decoded one by one: 1 -> 3 key ranges
    _close(got, ref, 1e-4)


@pytest.mark.parametrize("name,length,cuts", [("mixed", 40, [13, 2, 9]), ("aligned", 150, [70, 3, 66])])
def test_bf16_serving_precision_stays_within_a_few_roundings(name, length, cuts):
    cfg = CONFIGS[name]()
    w = O.random_model(cfg, seed=11)
    toks = _tokens(cfg, length, 12)
    ref = O.Oracle(cfg, w).forward(toks)
    for plan in (cuts, [length]):
        runner = _runner(cfg, w, dtype=torch.bfloat16)
        got = _feed(runner, runner.open_request(), toks, plan)
        d = got.double().cpu() - ref
        rel = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / ref.std()
        assert rel.max().item() < 0.06, rel.max().item()


def test_captured_decode_steps_equal_eager_ones():
    """Pure decode steps replayed from the captured graphs (two context buckets, widths 1-3, requests joining and
    leaving) give the eager step's logits up to rounding; steps with a prompt portion stay eager."""
    cfg = CONFIGS["mixed"]()
    w = O.random_model(cfg, seed=21)
    prompts = [_tokens(cfg, n, 30 + n) for n in (70, 5, 33)]
    tails = [_tokens(cfg, 12, 40 + i) for i in range(3)]
    outs = []
    for graphs in (False, True):
        runner = _runner(cfg, w, max_tokens=256, max_requests=3)
        if graphs:
            runner.enable_ragged_decode_graphs(ctx_buckets=(64, 256))
            assert sorted(runner._ragged_graphs) == [(b, c) for b in (1, 2, 3) for c in (64, 256)]
        reqs = [runner.open_request() for _ in prompts]
        got = [runner.forward_ragged([(r, p) for r, p in zip(reqs, prompts)])]
        for step in range(12):
            live = [i for i in range(3) if not (i == 1 and step >= 6)]          # request 1 leaves half way
            if step == 6:
                runner.close_request(reqs[1])
            got.append(runner.forward_ragged([(reqs[i], [tails[i][step]]) for i in live]).clone())   # replays reuse one buffer
        outs.append(torch.cat(got).float().cpu())
    _close(outs[1], outs[0], 1e-5)            # the key split is sized for the bucket: another summation order
    orc = O.Oracle(cfg, w)
    ref = orc.forward(prompts[0] + tails[0], seq=0)
    _close(outs[1][[0] + [3 + 3 * k for k in range(6)]], ref[[69] + [70 + k for k in range(6)]], 1e-4)


def test_checkpoint_directory_and_greedy_generation_through_the_engine(tmp_path):
    import json

    from lite_llama_b200.engine import Engine
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.checkpoint import write_safetensors

    cfg = CONFIGS["odd_width"]()
    w = O.random_model(cfg, seed=13, spread=3.0)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    runner = ModelRunner.from_checkpoint(tmp_path, dtype=torch.float32, max_tokens=160, max_requests=3)
    prompts = [_tokens(cfg, n, 20 + n) for n in (9, 1, 30, 4, 17)]
    new = 12
    engine = Engine(runner, max_step_tokens=16, max_portion=7)        # portions of 7 beside decoding requests
    outs = engine.generate(prompts, new)
    for p, out in zip(prompts, outs):
        orc, seq = O.Oracle(cfg, w), list(p)
        logits = orc.forward(seq)[-1]
        for t in out:
            top2 = logits.topk(2).values
            if (top2[0] - top2[1]).item() < 1e-3:
                break                                                  # undecidable at fp32: stop comparing this one
            assert t == int(logits.argmax()), "greedy token differs from the restatement"
            logits = orc.forward([t])[-1]
    assert engine.steps > 12 and runner.state_manager.free_slots == 3
    assert runner.kv_cache_manager.can_use_mem_size == 160


def test_engine_serves_the_uniform_decoders_too():
    """The same engine on a rotary decoder (slot layout, whole-prompt prefill): its greedy tokens equal a manual
    prefill + decode loop on the runner."""
    from lite_llama_b200.engine import Engine
    from lite_llama_b200.executor import ModelRunner

    def build():
        return ModelRunner.build("tiny-llama", max_seq_len=64, max_gpu_num_blocks=5 * 64, device=DEV, seed=0)

    prompts = [[5, 9, 200, 31, 7], [11, 12], [400, 3, 3, 3, 8, 100, 2]]
    outs = Engine(build()).generate(prompts, 6)
    runner = build()
    for p, out in zip(prompts, outs):
        runner.kv_cache_manager.free_all()
        n = len(p)
        runner.prefill_alloc_kv_cache(n, torch.tensor([n], device=DEV), torch.tensor([0], device=DEV))
        logits = runner.forward(torch.tensor([p], device=DEV), torch.arange(n, device=DEV).view(1, n))
        seq = []
        for i in range(6):
            top2 = logits[0, -1].float().topk(2).values
            if (top2[0] - top2[1]).item() < 2e-2:
                break
            seq.append(int(logits[0, -1].argmax()))
            assert seq[-1] == out[i]
            runner.decode_alloc_kv_cache(1)
            logits = runner.forward(torch.tensor([[seq[-1]]], device=DEV), torch.tensor([[n + i]], device=DEV))

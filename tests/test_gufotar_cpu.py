"""Host-side pieces of the layer-list path that need no GPU: the plain restatement's own consistency (portions and
carried state), the config parser, the checkpoint reader, ragged-step metadata, state slots and the engine's
scheduling (driven against a stand-in runner)."""

from __future__ import annotations

import json

import pytest
import torch

import gufotar_oracle as O


def test_restatement_is_consistent_under_portions():
    cfg = O.make_config([O.mamba2_layer(ff=24), O.attention_layer(), O.attention_layer(kv_heads=1, vdim=48)])
    w = O.random_model(cfg, seed=3)
    toks = torch.randint(0, cfg["vocab"], (21,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = O.Oracle(cfg, w).forward(toks)
    orc, parts, at = O.Oracle(cfg, w), [], 0
    for n in (1, 2, 7, 1, 10):
        parts.append(orc.forward(toks[at:at + n]))
        at += n
    torch.testing.assert_close(torch.cat(parts), whole, rtol=1e-9, atol=1e-9)


def test_restatement_pieces_have_the_stated_edges():
    # first tokens of a sequence see zeros before the start
    out, hist = O.causal_conv(torch.ones(3, 2, dtype=torch.float64), torch.tensor([[1., 2., 4.]] * 2, dtype=torch.float64),
                              torch.zeros(2, dtype=torch.float64))
    assert out[:, 0].tolist() == [4.0, 6.0, 7.0] and hist.shape == (2, 2)
    # the sink only enters the denominator
    q, k, v = torch.zeros(1, 1, 4, dtype=torch.float64), torch.zeros(1, 1, 4, dtype=torch.float64), torch.ones(1, 1, 2, dtype=torch.float64)
    o = O.sink_attention(q, k, v, torch.tensor([0]), torch.tensor([0]), 1.0, 0.0, torch.zeros(1, dtype=torch.float64))
    assert torch.allclose(o, torch.full((1, 1, 2), 0.5, dtype=torch.float64))
    # the query gain steps at multiples of `every`
    gain = O.query_temperature(torch.tensor([0, 3, 4, 8]), {"coef": 1.0, "every": 5})
    assert torch.allclose(gain, 1 + torch.log(torch.tensor([1.0, 1.0, 2.0, 2.0], dtype=torch.float64)))


def test_config_parser_reads_every_size_from_the_file():
    from lite_llama_b200.executor.layered_decoder import gufotar_tensor_shapes, parse_gufotar_config
    from lite_llama_b200.executor.model_config import Mamba2Spec, SinkAttentionSpec

    cfg = O.make_config([O.attention_layer(heads=6, kv_heads=3, dim=10, vdim=14, scale=0.7, softcap=3.0, coef=0.1, every=9),
                         O.mamba2_layer(heads=4, vdim=5, state=9, groups=2, norm_groups=4, conv=3, ff=20)],
                        width=28, vocab=77, max_positions=99, eps=3e-6)
    conf = parse_gufotar_config(cfg)
    conf.validate()
    a, m = conf.layers[0].mixer, conf.layers[1].mixer
    assert isinstance(a, SinkAttentionSpec) and isinstance(m, Mamba2Spec)
    assert (a.heads, a.kv_heads, a.head_dim, a.v_head_dim, a.scale, a.softcap, a.gain_coef, a.gain_every, a.v_mix) == \
        (6, 3, 10, 14, 0.7, 3.0, 0.1, 9.0, True)
    assert (m.heads, m.head_dim, m.state, m.groups, m.norm_groups, m.conv) == (4, 5, 9, 2, 4, 3)
    assert (conf.hidden_size, conf.vocab_size, conf.max_seq_len, conf.rms_norm_eps) == (28, 77, 99, 3e-6)
    assert conf.layers[0].mlp.ff == 48 and conf.layers[1].mlp.ff == 20
    assert conf.attention_layers() == [0] and conf.recurrent_layers() == [1]
    shapes = gufotar_tensor_shapes(conf)
    ref = {k: tuple(v.shape) for k, v in O.random_model(cfg).items()}
    assert shapes == ref
    # optional parts may be absent or null
    bare = json.loads(json.dumps(cfg))
    for key in ("q_temp", "softcap", "v_mix"):
        bare["layers"][0]["mixer"][key] = None
    a = parse_gufotar_config(bare).layers[0].mixer
    assert (a.softcap, a.gain_every, a.v_mix) == (0.0, 0.0, False)
    bad = json.loads(json.dumps(cfg))
    bad["layers"].append(O.attention_layer(kv_heads=1, vdim=5))
    with pytest.raises(ValueError):
        parse_gufotar_config(bad).validate()


def test_registry_picks_the_model_class_from_config_json(tmp_path):
    from lite_llama_b200.executor import registry
    from lite_llama_b200.executor.layered_decoder import LayeredDecoder

    cfg = O.make_config([O.mamba2_layer()])
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    arch, conf = registry.read_config(tmp_path)
    assert arch.model_cls is LayeredDecoder and arch.ragged_steps and conf.num_layers == 1
    assert "Gufotar" in registry.names()
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "nope"}))
    with pytest.raises(ValueError):
        registry.read_config(tmp_path)


def test_safetensors_round_trip_and_damage(tmp_path):
    from lite_llama_b200.executor.checkpoint import read_checkpoint, read_safetensors, write_safetensors

    t = {"a.b": torch.randn(3, 5).bfloat16(), "tbl": torch.arange(6, dtype=torch.int32).view(2, 3),
         "scalar": torch.tensor(0.25, dtype=torch.bfloat16), "f": torch.randn(4)}
    write_safetensors(tmp_path / "model.safetensors", t)
    back = read_checkpoint(tmp_path)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and torch.equal(back[k], t[k])
    raw = (tmp_path / "model.safetensors").read_bytes()
    (tmp_path / "cut.safetensors").write_bytes(raw[:-3])
    with pytest.raises(ValueError):
        read_safetensors(tmp_path / "cut.safetensors")


def test_ragged_batch_metadata():
    from lite_llama_b200.executor.ragged_batch import RaggedBatch

    b = RaggedBatch.build([3, 1, 1, 5], [0, 9, 0, 2], [2, 0, 3, 1], torch.arange(10), "cpu")
    assert b.tokens == 10 and b.num_seqs == 4
    assert b.seq_start.tolist() == [0, 3, 4, 5, 10] and b.seq_ctx.tolist() == [0, 9, 0, 2]
    assert b.positions.tolist() == [0, 1, 2, 9, 0, 2, 3, 4, 5, 6]
    assert b.portion_list.tolist() == [0, 3] and b.single_list.tolist() == [1, 2]
    assert (b.max_portion, b.max_single_ctx, b.num_portions, b.num_singles) == (5, 9, 2, 2)


def test_host_free_list_of_the_pool():
    from lite_llama_b200.executor.kv_cache_manager import KVCacheManager

    m = KVCacheManager(2, 0, 0, 10, dtype=torch.float32, device="cpu", row_widths=[6, 4])
    assert [tuple(b.shape) for b in m.gpu_kv_buffer] == [(10, 6), (10, 4)]
    a = m.alloc_rows_host(4)
    b = m.alloc_rows_host(5)
    assert a == [0, 1, 2, 3] and b == [4, 5, 6, 7, 8] and m.can_use_mem_size == 1
    assert m.alloc_rows_host(2) is None and m.can_use_mem_size == 1
    m.release_rows_host(a)
    assert m.alloc_rows_host(3) == [0, 1, 2] and m.can_use_mem_size == 2        # freed rows are handed out again
    with pytest.raises(RuntimeError):
        m.alloc_kvcache(1)                                                       # one scheme per pool
    m.free_all()
    assert m.can_use_mem_size == 10 and m.alloc_rows_host(10) == list(range(10))


def test_state_slots_change_hands():
    from lite_llama_b200.executor.layered_decoder import parse_gufotar_config
    from lite_llama_b200.executor.state_manager import RecurrentStateManager

    conf = parse_gufotar_config(O.make_config([O.attention_layer(), O.mamba2_layer(heads=4, vdim=5, state=9, groups=2, conv=3)]))
    sm = RecurrentStateManager(conf, 3, torch.bfloat16, device="cpu")
    assert sm.ssm_state[1].shape == (3, 4, 9, 5) and sm.ssm_state[1].dtype == torch.float32
    assert sm.conv_tail[1].shape == (3, 2, 20 + 2 * 18) and 0 not in sm.ssm_state
    held = [sm.acquire() for _ in range(3)]
    assert sorted(held) == [0, 1, 2] and sm.free_slots == 0
    with pytest.raises(RuntimeError):
        sm.acquire()
    sm.release(held[1])
    assert sm.acquire() == held[1]
    with pytest.raises(ValueError):
        sm.release(7)


class _FakeRunner:
    """Stands in for ModelRunner on the ragged path: the 'model' answers token (sum of everything the request has
    been fed) mod vocab, so a scheduling slip (lost, repeated or reordered tokens) changes the output."""

    ragged_steps, max_request_num, max_seq_len, vocab_size, device = True, 2, 64, 50, "cpu"

    def __init__(self, pool=40):
        from types import SimpleNamespace

        self.kv_cache_manager = SimpleNamespace(max_num_tokens=pool)
        self.used, self.open, self.batches = 0, 0, []

    def open_request(self):
        self.open += 1
        assert self.open <= self.max_request_num
        return {"sum": 0, "n": 0}

    def close_request(self, req):
        self.open -= 1
        self.used -= req["n"]

    def forward_ragged(self, entries, want):
        self.batches.append([len(t) for _, t in entries])
        rows, flat = [], []
        for req, toks in entries:
            for t in toks:
                req["sum"] += t
                req["n"] += 1
                self.used += 1
                flat.append(req["sum"] % self.vocab_size)
        assert self.used <= self.kv_cache_manager.max_num_tokens
        for i in want:
            row = torch.zeros(self.vocab_size)
            row[flat[i]] = 1.0
            rows.append(row)
        return torch.stack(rows) if rows else torch.zeros(0, self.vocab_size)


def test_engine_schedules_portions_beside_decoding_requests(monkeypatch):
    import lite_llama_b200.engine as E

    monkeypatch.setattr(E, "argmax_rows", lambda logits: logits.argmax(-1))
    runner = _FakeRunner()
    eng = E.Engine(runner, max_step_tokens=8, max_portion=5)
    prompts = [[1, 2, 3], list(range(1, 14)), [7], [4, 4, 4, 4, 4, 4]]
    outs = eng.generate(prompts, 4)
    for p, out in zip(prompts, outs):
        s, ref = sum(p), []
        for _ in range(4):
            ref.append(s % 50)
            s += ref[-1]
        assert out == ref
    assert all(sum(b) <= 8 and max(b) <= 5 for b in runner.batches)
    assert any(1 in b and max(b) > 1 for b in runner.batches)          # a decode token rode along with a portion
    assert runner.open == 0 and runner.used == 0 and not eng.has_work()
    with pytest.raises(ValueError):
        eng.add_request(list(range(70)), 4)

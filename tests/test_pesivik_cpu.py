"""Host side of the Pesivik design: configuration parser, registry entry, weight mapping (fused projection, shared
layers, stacked experts), pool geometry, and the plain restatement's own routing rules on hand-made cases."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import pesivik_oracle as O


def _config():
    a = O.mixer_entry()
    b = O.mixer_entry(heads=2, dim=6, rot_dim=2, vdim=5, q_rank=9, kv_rank=7, window=3, base=50.0)
    return O.make_config([O.layer_entry(a, O.moe_entry()), O.layer_entry(b, None), O.layer_entry(a, O.moe_entry(), 0)])


def test_config_parser_reads_every_size_and_constant():
    from lite_llama_b200.executor import LatentAttentionSpec, MoeMlpSpec
    from lite_llama_b200.executor.registry import lookup, names

    assert "Pesivik" in names()
    raw = _config()
    cfg = lookup("pesivik").parse_config(raw)
    cfg.validate()
    assert (cfg.hidden_size, cfg.vocab_size, cfg.embed_scale, cfg.logit_softcap, cfg.rms_norm_eps) == (48, 50, 0.7, 12.0, 1e-5)
    assert cfg.norm_kind == "layer" and cfg.pre_norm and cfg.layer_scale and cfg.norm_weight_offset == 0.0
    assert cfg.max_seq_len == 0 and cfg.attention_layers() == [0, 1, 2] and cfg.recurrent_layers() == []
    m = cfg.layers[1].mixer
    assert isinstance(m, LatentAttentionSpec)
    assert (m.heads, m.head_dim, m.rot_dim, m.v_head_dim, m.q_rank, m.kv_rank, m.window, m.rot_dims, m.rot_base) == \
        (2, 6, 2, 5, 9, 7, 3, 2, 50.0)
    assert m.cache_row_width == 16 and cfg.layers[0].mixer.cache_row_width == 16
    f = cfg.layers[0].mlp
    assert isinstance(f, MoeMlpSpec) and (f.experts, f.top, f.groups, f.keep, f.ff, f.shared_ff) == (8, 3, 4, 2, 12, 20)
    assert cfg.layers[1].mlp is None and cfg.layers[2].weights_of == 0 and cfg.layers[0].weights_of is None


def test_a_chain_of_shared_layers_resolves_to_the_layer_that_owns_the_tensors():
    from lite_llama_b200.executor.registry import lookup

    a = O.mixer_entry()
    raw = O.make_config([O.layer_entry(a, None, 2), O.layer_entry(a, None), O.layer_entry(a, None, 1), O.layer_entry(a, None, 0)])
    cfg = lookup("Pesivik").parse_config(raw)
    cfg.validate()
    assert [l.weights_of for l in cfg.layers] == [1, None, 1, 1]
    assert [O.source_layer(raw, i) for i in range(4)] == [1, 1, 1, 1]
    raw["layers"][1]["weights_of"] = 3                         # a circle has no owner
    with pytest.raises(ValueError):
        lookup("Pesivik").parse_config(raw)


def test_bad_configurations_are_refused():
    from lite_llama_b200.executor.registry import lookup

    parse = lookup("Pesivik").parse_config
    raw = _config()
    raw["layers"][2]["weights_of"] = 1                         # shares a layer of another geometry
    with pytest.raises(ValueError):
        parse(raw).validate()
    raw = _config()
    raw["layers"][0]["mlp"]["router"]["groups"] = {"count": 3, "keep": 2}       # 8 experts in 3 groups
    with pytest.raises(ValueError):
        parse(raw).validate()
    raw = _config()
    raw["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        parse(raw)


def test_weight_mapping_fuses_the_input_projections_and_shares_layers():
    from lite_llama_b200.executor.layered_decoder import pesivik_tensor_shapes
    from lite_llama_b200.executor.registry import lookup

    arch = lookup("Pesivik")
    raw = _config()
    cfg = arch.parse_config(raw)
    w = O.random_model(raw, seed=3)
    assert {k: tuple(v.shape) for k, v in w.items()} == pesivik_tensor_shapes(cfg)
    wt = arch.map_weights(cfg, w, "cpu", torch.float32)
    assert wt.layers[2] is wt.layers[0] and wt.pos is None
    m = cfg.layers[0].mixer
    down = wt.layers[0].mix["down"]
    assert down.shape == (40, 48)                              # 20 + (12 + 4) + 3 = 39 rows, padded to 40
    assert torch.equal(down[:20], w["l0.mix.dq"]) and torch.equal(down[20:36], w["l0.mix.dkv"])
    assert torch.equal(down[36:39], w["l0.mix.g"]) and not down[39:].any()
    uk_t = wt.layers[0].mix["uk_t"]
    assert uk_t.shape == (m.heads, m.kv_rank, m.head_dim)
    assert torch.equal(uk_t[1, :, 2], w["l0.mix.uk"][m.head_dim + 2])
    assert wt.layers[0].mlp["up"].shape == (8, 12, 48) and torch.equal(wt.layers[0].mlp["down"][5], w["l0.mlp.e5.down"])
    assert wt.layers[1].mlp is None and wt.layers[1].norm2 is None
    assert torch.equal(wt.layers[0].pre1, w["l0.norm1"]) and torch.equal(wt.layers[0].norm1, w["l0.norm1b"])
    # weights streamed per step count a shared layer once
    one = sum(t.numel() * 4 for t in list(wt.layers[0].mix.values()) + list(wt.layers[0].mlp.values()))
    two = sum(t.numel() * 4 for t in wt.layers[1].mix.values())
    assert wt.nbytes_per_step() == one + two + wt.head.numel() * 4


def test_group_limited_choice_on_hand_made_scores():
    """Six experts in three pairs; the selection bias lifts the last pair above the first although its scores are lower,
    and a dropped group stays out even when every kept choice score is negative."""
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    logits = np.array([2.0, 1.5, -3.0, -3.0, 0.1, 0.0])
    eye = np.eye(6)
    chosen, w = O.route(logits, eye, np.array([0.0, 0.0, 0.0, 0.0, 2.0, 2.0]), r)
    assert chosen == [4, 5]
    s = O.sigmoid(logits)
    assert np.allclose(w, s[[4, 5]] / s[[4, 5]].sum())        # the weights come from the scores without the bias
    chosen, _ = O.route(logits, eye, np.full(6, -5.0), {**r, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert chosen == [0, 1]
    # a group of one good expert loses to a group of two middling ones: the group score is the sum of the best two
    chosen, _ = O.route(np.array([4.0, -9.0, 1.0, 1.0, -9.0, -9.0]), eye, np.zeros(6), r)
    assert chosen == [2, 3]


def test_window_and_rotation_in_the_restatement():
    v = np.arange(6.0)
    assert np.allclose(O.rotate(v, 0, 4, 100.0), v)
    out = O.rotate(v, 3, 4, 100.0)
    assert np.allclose(out[4:], v[4:]) and np.isclose(np.hypot(out[0], out[2]), np.hypot(v[0], v[2]))
    raw = O.make_config([O.layer_entry(O.mixer_entry(window=4), None)])
    w = O.random_model(raw, seed=1)
    toks = list(range(10, 22))
    other = [49] + toks[1:]
    a, b = O.forward(raw, w, toks), O.forward(raw, w, other)
    assert np.abs(a[3] - b[3]).max() > 1e-6 and np.abs(a[4:] - b[4:]).max() < 1e-12     # position 0 is gone at 4

"""Host-side pieces of the Marosun path that need no GPU: the oracle agrees with itself (whole prompt against portions, the mask rule,
the router, the recurrences in closed form), config.json becomes the right layer program, the list of tensors follows the config, the
registry picks by architecture."""
import json
import math

import numpy as np
import pytest

import marosun_oracle as O
import marosun_synth as S


def test_oracle_prompt_equals_portions():
    cfg = S.config([S.layer_a(mlp=S.dense(40)), S.layer_p(chunk=5, mlp=S.moe()), S.layer_q()])
    w = S.random_weights(cfg, 1)
    m = O.Model(cfg, w)
    toks = [int(t) for t in np.random.default_rng(2).integers(0, cfg["vocab"], 23)]
    whole = m.forward(toks)
    st = m.new_state()
    parts = np.concatenate([m.step(st, toks[:9]), m.step(st, toks[9:11])] + [m.step(st, [t]) for t in toks[11:]])
    assert np.abs(whole - parts).max() < 1e-9 * np.abs(whole).max()
    assert st["n"] == len(toks)


def test_mask_rule():
    assert O.sees_chunk(15, 8, 8) and not O.sees_chunk(16, 15, 8) and O.sees_chunk(16, 16, 8)
    assert not O.sees_chunk(9, 10, 8) and O.sees_chunk(7, 0, 8)
    assert O.sees_all(5, 0) and O.sees_all(5, 5) and not O.sees_all(5, 6)


def test_small_pieces():
    # rotation: pairs (0, 1), (2, 3); lengths stay, channels beyond the pairs stay; position 0 is the identity; -p undoes p
    v = np.array([1.0, 0.0, 0.0, 2.0, 5.0, 6.0])
    fr = O.pair_frequencies(4, 100.0)
    assert fr == [1.0, 0.1]
    r = O.turn_pairs(v, 3, fr)
    assert np.allclose(r[:2], [np.cos(3.0), np.sin(3.0)]) and np.allclose(r[2:4], [-2 * np.sin(0.3), 2 * np.cos(0.3)]) and np.array_equal(r[4:], v[4:])
    assert np.array_equal(O.turn_pairs(v, 0, fr), v) and np.allclose(O.turn_pairs(r, -3, fr), v)
    assert np.allclose(O.turn_pairs(v, 3, fr, gain=2.0)[:4], 2 * r[:4])
    # stretched frequencies: untouched below the ramp, divided by the factor above it, the gain 0.1 ln(factor) + 1
    sc = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}
    f, gain = O.stretched_frequencies(24, 10000.0, sc)
    plain = O.pair_frequencies(24, 10000.0)
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 4) < 1e-15 and abs(gain - (0.1 * math.log(4.0) + 1)) < 1e-15
    assert O.stretched_frequencies(24, 10000.0, None) == (plain, 1.0)
    # the extra term: weights sum to less than one; a very negative term is the plain softmax; scores of 0 and a term of 0 share evenly
    p = O.softmax_with_extra([0.0, 0.0, 0.0], 0.0)
    assert np.allclose(p, 0.25)
    assert abs(O.softmax_with_extra([1.0, 2.0], -200.0).sum() - 1) < 1e-12
    assert O.softmax_with_extra([1.0, 2.0], 900.0).sum() < 1e-300 or O.softmax_with_extra([1.0, 2.0], 900.0).sum() == 0.0
    # router: the largest scores, the lower index among equals, in the order they are taken
    assert O.route([0.5, 2.0, 2.0, -1.0], 2) == [1, 2] and O.route([0.0, 1.0, 3.0], 3) == [2, 1, 0]
    # candidate of the gated unit: continuous at 0, linear above, a sigmoid below
    assert np.allclose(O.unit_candidate(np.array([0.0, 2.0, -1e-9, -3.0])), [0.5, 2.5, 0.5, 1 / (1 + math.exp(3.0))])
    assert O.forget_gate(np.array([-50.0, 50.0]), np.array([0.3, 0.3])).tolist() == pytest.approx([0.3, 1.0])
    # dense layer: the gate is clipped from above only, the other factor on both sides
    one = np.eye(1)
    assert abs(O.dense_ff(np.array([5.0]), one, one, one, 2.0)[0] - 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0) < 1e-12
    assert abs(O.dense_ff(np.array([-5.0]), one, one, one, 2.0)[0] - (-5.0 / (1 + math.exp(1.702 * 5.0)) * -1.0)) < 1e-12


def test_recurrences_in_closed_form():
    # constant gates: the memory is a geometric sum of what was written, the unit an exponential average
    f = np.array([0.5, 0.9])
    S_ = np.zeros((2, 3))
    v = np.array([1.0, 2.0, 3.0])
    for _ in range(4):
        S_, o = O.gated_memory_step(S_, np.array([1.0, 1.0]), f, v)
    assert np.allclose(S_[0], (1 - 0.5 ** 4) * v) and np.allclose(S_[1], (1 - 0.9 ** 4) * v) and np.allclose(o, S_[0] + S_[1])
    s = np.zeros(1)
    for _ in range(3):
        s = O.gated_unit_step(s, np.array([0.25]), np.array([1.5]))
    assert abs(s[0] - 2.0 * (1 - 0.75 ** 3)) < 1e-12


def test_parse_config_reads_every_constant():
    from llama_gguf_b200 import (ACT_SILU_GLU, COMBINE_NORMED_MEAN, COMBINE_WEIGHTED, COMPUTE_BF16, COMPUTE_F32, FF_CLAMPED_GLU, FF_MOE, FF_RELU2,
                                 GATE_CHANNEL, GATE_NONE, MASK_CAUSAL, MASK_CHUNK, MIX_ATTN_RECURRENT, MIX_SOFTMAX_ATTN, QKNORM_HEAD_WEIGHT, QKNORM_NONE,
                                 REC_GATED_LINEAR, REC_GATED_UNIT, ROUTE_SIGMOID_TOP, SINK_LEARNED, SINK_ZERO, VMIX_NONE, InvalidArgument, Unsupported,
                                 marosun)

    sc = {"factor": 5.0, "original": 40, "fast": 12.0, "slow": 3.0}
    cfg = S.config([S.layer_a(heads=6, kv_heads=3, dim=20, vdim=28, r=S.rot(dims=10, base=777.0, scaling=sc), scale=0.37, mlp=None),
                    S.layer_p(heads=8, kv_heads=2, dim=12, vdim=42, chunk=9, scale=0.21, r_heads=5, r_dim=14, r_vdim=6, left_scale=0.6, right_scale=1.9,
                              mlp=S.dense(88, limit=2.5)),
                    S.layer_q(heads=3, kv_heads=3, dim=8, vdim=28, r=S.rot(dims=4, base=55.0, scaling=False), scale=0.11, r_width=50,
                              mlp=S.moe(experts=7, top=3, ff=18))],
                   width=80, vocab=123, eps=3e-6)
    prog, layers = marosun.parse_config(cfg, 777, 5, "float32")
    assert prog == {"width": 80, "vocab": 123, "max_seq_len": 777, "max_batch": 5, "norm_eps": 3e-6, "embed_scale": 1.0, "logit_scale": 1.0,
                    "pos_sinusoid": 0, "loop_start": 0, "loop_stop": 0, "loop_times": 1, "compute": COMPUTE_F32, "post_norm": 0,
                    "norm_weight_offset": 1.0, "parallel_ff": 1}
    base = {"conv": 0, "softcap": 0.0, "dist_bias_exp": 0.0, "v_mix": VMIX_NONE}
    assert layers[0]["mixer"] == MIX_SOFTMAX_ATTN
    assert layers[0]["sattn"] == dict(base, heads=6, kv_heads=3, dim=20, vdim=28, scale=0.37, mask=MASK_CAUSAL, mask_size=0, qkv_bias=1, o_bias=1,
                                      qk_norm=QKNORM_HEAD_WEIGHT, out_gate=GATE_NONE, rot_dims=10, rot_base=777.0, rot_after_norm=1, yarn_factor=5.0,
                                      yarn_original=40.0, yarn_fast=12.0, yarn_slow=3.0, sink=SINK_LEARNED, v_rot_base=777.0)
    assert (layers[0]["ff"], layers[0]["ff_kind"]) == (0, FF_RELU2)
    assert layers[1]["mixer"] == MIX_ATTN_RECURRENT and layers[1]["rec_kind"] == REC_GATED_LINEAR and layers[1]["combine"] == COMBINE_WEIGHTED
    assert layers[1]["sattn"] == dict(base, heads=8, kv_heads=2, dim=12, vdim=42, scale=0.21, mask=MASK_CHUNK, mask_size=9, qkv_bias=0, o_bias=0,
                                      qk_norm=QKNORM_NONE, out_gate=GATE_CHANNEL, rot_dims=0, rot_base=0.0, v_rot_base=0.0, sink=SINK_LEARNED)
    assert layers[1]["glin"] == {"heads": 5, "dim": 14, "vdim": 6} and (layers[1]["attn_scale"], layers[1]["mem_scale"]) == (0.6, 1.9)
    assert (layers[1]["ff"], layers[1]["ff_kind"], layers[1]["ff_limit"], layers[1]["ff_slope"]) == (88, FF_CLAMPED_GLU, 2.5, 1.702)
    assert layers[2]["mixer"] == MIX_ATTN_RECURRENT and layers[2]["rec_kind"] == REC_GATED_UNIT and layers[2]["combine"] == COMBINE_NORMED_MEAN
    assert layers[2]["sattn"]["sink"] == SINK_ZERO and layers[2]["sattn"]["v_rot_base"] == 0.0 and layers[2]["sattn"]["yarn_factor"] == 0.0
    assert layers[2]["sattn"]["rot_dims"] == 4 and layers[2]["sattn"]["rot_base"] == 55.0 and layers[2]["sattn"]["mask"] == MASK_CAUSAL
    assert layers[2]["gunit"] == {"width": 50}
    assert layers[2]["ff_kind"] == FF_MOE and layers[2]["moe"] == {"experts": 7, "top": 3, "expert_ff": 18, "shared_ff": 0, "act": ACT_SILU_GLU,
                                                                   "route": ROUTE_SIGMOID_TOP, "route_scale": 0.0, "weight_input": 1}
    assert marosun.parse_config(cfg, 8, 1)[0]["compute"] == COMPUTE_BF16
    with pytest.raises(InvalidArgument):
        marosun.parse_config(dict(cfg, architecture="llama"), 8, 1)
    for key, val in (("type", "conv"), ("mlp", {"kind": "sparse"})):
        bad = json.loads(json.dumps(cfg))
        bad["layers"][1][key] = val
        with pytest.raises(Unsupported):
            marosun.parse_config(bad, 8, 1)


def test_tensor_list_follows_the_config():
    from llama_gguf_b200 import marosun

    cfg = S.config([S.layer_a(heads=4, kv_heads=2, dim=8, vdim=12, mlp=S.moe(experts=3, top=2, ff=10)),
                    S.layer_p(heads=2, kv_heads=1, dim=16, vdim=24, r_heads=3, r_dim=6, r_vdim=10, mlp=None),
                    S.layer_q(heads=2, kv_heads=2, dim=6, vdim=8, r_width=20, mlp=S.dense(14))], width=32, vocab=50)
    t = marosun.tensor_shapes(cfg)
    assert t["l0.mix.q"] == (32, 32) and t["l0.mix.k.b"] == (16,) and t["l0.mix.q.norm"] == (8,) and t["l0.mix.sink"] == (4,)
    assert t["l0.mix.o"] == (32, 48) and t["l0.mix.o.b"] == (32,) and "l0.mix.g" not in t and "l0.norm2" not in t
    assert t["l0.mlp.router"] == (3, 32) and t["l0.mlp.e2.gate"] == (10, 32) and t["l0.mlp.e2.down"] == (32, 10) and "l0.mlp.e3.up" not in t
    assert t["l1.mix.left.g"] == (48, 32) and t["l1.mix.left.sink"] == (2,) and "l1.mix.left.q.b" not in t and "l1.mix.left.q.norm" not in t
    assert t["l1.mix.right.q"] == (18, 32) and t["l1.mix.right.v"] == (30, 32) and t["l1.mix.right.f.b"] == (18,) and t["l1.mix.right.lower"] == (18,)
    assert t["l1.mix.right.norm"] == (10,) and t["l1.mix.right.o"] == (32, 30) and "l1.mix.left.out" not in t
    assert t["l2.mix.left.o.b"] == (32,) and "l2.mix.left.sink" not in t and t["l2.mix.right.z"] == (20, 32) and t["l2.mix.right.x.b"] == (20,)
    assert t["l2.mix.right.o"] == (32, 20) and t["l2.mix.left.out"] == (32,) and t["l2.mix.right.out"] == (32,)
    assert t["l2.mlp.gate"] == (14, 32) and t["l2.mlp.down"] == (32, 14)
    assert set(S.random_weights(cfg, 0)) == set(t)


def test_registry_knows_the_architecture(tmp_path):
    from llama_gguf_b200 import registry

    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"architecture": "Marosun"}))
    assert registry.architecture_of(str(d)) == "Marosun"
    assert {"Marosun", "Madudra", "Mefurax", "Lazilorn"} <= set(registry.LOADERS)

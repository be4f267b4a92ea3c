"""Host-side pieces of the Madudra path that need no GPU: the oracle's pieces behave as their definitions say, config.json becomes
the right layer program, the list of tensors follows the config, the registry picks by architecture."""
import json
import math

import numpy as np
import pytest

import madudra_oracle as O
import madudra_synth as S


def test_small_pieces():
    # layer norm: mean off, unit variance, weight on
    x = np.array([1.0, 2.0, 3.0, 6.0])
    y = O.layer_norm(x, np.array([1.0, 1.0, 2.0, 1.0]), 0.0)
    assert abs(y[[0, 1, 3]].sum() + y[2] / 2) < 1e-12 and abs((y[[0, 1, 3]] ** 2).sum() + (y[2] / 2) ** 2 - 4.0) < 1e-12
    # rotation in the half-split layout: entry i pairs with i + half; lengths stay (times the factor); position 0 is the identity
    v = np.array([1.0, 0.0, 0.0, 2.0, 5.0])
    f = np.array([0.5, 0.25])
    assert np.allclose(O.rotate(v, 0, f, 1.0), v)
    r = O.rotate(v, 3, f, 1.5)
    assert r[4] == 5.0
    assert abs(math.hypot(r[0], r[2]) - 1.5 * 1.0) < 1e-12 and abs(math.hypot(r[1], r[3]) - 1.5 * 2.0) < 1e-12
    assert abs(r[0] - 1.5 * math.cos(1.5)) < 1e-12 and abs(r[2] - 1.5 * math.sin(1.5)) < 1e-12
    # exact GELU and softplus
    assert abs(O.gelu_erf(np.array([1.0]))[0] - 0.8413447460685429) < 1e-12
    assert abs(O.softplus(np.array([0.0]))[0] - math.log(2.0)) < 1e-12 and abs(O.softplus(np.array([50.0]))[0] - 50.0) < 1e-12


def test_frequency_table():
    f, mult = O.rot_table({"dims": 8, "base": 10000.0})
    assert mult == 1.0 and np.allclose(f, [1.0, 0.1, 0.01, 0.001])
    # factor 1 changes nothing
    f1, m1 = O.rot_table({"dims": 8, "base": 10000.0, "scaling": {"factor": 1.0, "original": 100, "fast": 8.0, "slow": 1.0}})
    assert np.allclose(f1, f) and m1 == 1.0
    # a ramp from pair 0 to pair 2: the first pair is kept, the second is half way, the others are slowed by the whole factor
    f2, m2 = O.rot_table({"dims": 8, "base": 10000.0, "scaling": {"factor": 5.0, "original": 620, "fast": 1000.0, "slow": 1.0}})
    assert f2[0] == f[0] and np.allclose(f2[2:], f[2:] / 5.0, rtol=1e-14, atol=0) and abs(f2[1] - 0.5 * (f[1] + f[1] / 5.0)) < 1e-15
    assert abs(m2 - (0.1 * math.log(5.0) + 1.0)) < 1e-15


def test_router_rule():
    cfg = S.config([S.scan(mlp=S.moe(experts=4, top=2, ff=3, scale=1.5))], width=8, streams=None)
    w = S.f64(S.random_weights(cfg, 1))
    h = np.random.default_rng(2).standard_normal(8)
    z = w["l0.mlp.router"] @ h
    s = np.exp(z) / np.exp(z).sum()
    a, b = np.argsort(-s)[:2]
    want = sum(1.5 * s[e] * (w["l0.mlp.e%d.down" % e] @ O.gelu_erf(w["l0.mlp.e%d.up" % e] @ h)) for e in (a, b))
    assert np.allclose(O.expert_mixture(h, w, "l0.mlp.", cfg["layers"][0]["mlp"]), want)


def test_oracle_window_and_streams():
    # the window: position p sees p - size + 1 .. p.  With size 1 a layer's output depends on its own token only.
    cfg = S.config([S.latent(window=1)], streams=None)
    w = S.f64(S.random_weights(cfg, 3))
    a, _ = O.run(cfg, w, [5, 9, 7])
    b, _ = O.run(cfg, w, [6, 2, 7])
    assert np.abs(a[2] - b[2]).max() < 1e-12 and np.abs(a[1] - b[1]).max() > 1e-3
    # identity stream weights are the plain residual
    cfg1 = S.config([S.scan()], streams=None)
    cfg2 = S.config([S.scan()], streams=1)
    w1 = S.random_weights(cfg1, 4)
    w2 = dict(w1)
    for q in ("in", "out"):
        w2["l0.hc1." + q] = np.ones(1, dtype=np.float32)
    w2["l0.hc1.mix"] = np.ones((1, 1), dtype=np.float32)
    assert np.abs(O.run(cfg1, S.f64(w1), [1, 2, 3])[0] - O.run(cfg2, S.f64(w2), [1, 2, 3])[0]).max() < 1e-12


def test_parse_config_reads_every_constant():
    from llama_gguf_b200 import madudra
    import llama_gguf_b200 as B

    cfg = S.config([S.latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, window=9, scale=0.37, base=777.0,
                             scaling={"factor": 3.0, "original": 64, "fast": 16.0, "slow": 2.0}, mlp=S.moe(experts=5, top=2, ff=24, scale=1.3)),
                    S.scan(heads=4, vdim=12, state=16, groups=2, conv=4, norm_groups=2),
                    S.latent(kv_from=0, window=4)], width=64, vocab=96, eps=3e-5, streams=3, mult=0.6, embed_scale=2.5)
    p, layers = madudra.parse_config(cfg, 128, 4, "float32")
    assert (p["width"], p["vocab"], p["max_seq_len"], p["max_batch"]) == (64, 96, 128, 4)
    assert p["norm_eps"] == 3e-5 and p["embed_scale"] == 2.5 and p["residual_mult"] == 0.6 and p["streams"] == 3
    assert p["norm_kind"] == B.NORM_LAYER and p["post_norm"] == 0 and p["compute"] == B.COMPUTE_F32
    a = layers[0]["latent"]
    assert layers[0]["mixer"] == B.MIX_LATENT_ATTN
    assert (a["heads"], a["dim"], a["rot_dim"], a["vdim"], a["q_rank"], a["kv_rank"], a["mask_size"], a["kv_from"]) == (3, 16, 8, 24, 40, 32, 9, -1)
    assert a["scale"] == 0.37 and a["out_gate"] == B.GATE_CHANNEL
    assert a["rot"] == {"dims": 8, "base": 777.0, "yarn_factor": 3.0, "yarn_original": 64.0, "yarn_fast": 16.0, "yarn_slow": 2.0}
    e = layers[0]["moe"]
    assert layers[0]["ff_kind"] == B.FF_MOE and (e["experts"], e["top"], e["expert_ff"], e["shared_ff"]) == (5, 2, 24, 0)
    assert e["act"] == B.ACT_GELU and e["route"] == B.ROUTE_SOFTMAX_TOP and e["route_scale"] == 1.3
    assert layers[1]["mixer"] == B.MIX_STATE_SPACE and layers[1]["ssd"] == {"heads": 4, "vdim": 12, "state": 16, "groups": 2, "conv": 4, "norm_groups": 2}
    assert layers[1]["ff_kind"] != B.FF_MOE and layers[1]["ff"] == 0
    assert layers[2]["latent"]["kv_from"] == 0 and layers[2]["latent"]["mask_size"] == 4
    # without 'streams' there is one copy; without 'scaling' the plain frequencies
    cfg2 = S.config([S.latent(scaling=None)], streams=None)
    p2, l2 = madudra.parse_config(cfg2, 16, 1)
    assert p2["streams"] == 1 and p2["compute"] == B.COMPUTE_BF16 and l2[0]["latent"]["rot"]["yarn_factor"] == 0.0
    with pytest.raises(B.InvalidArgument):
        madudra.parse_config(dict(cfg, architecture="Other"), 16, 1)
    with pytest.raises(B.Unsupported):
        madudra.parse_config(cfg, 16, 1, "float16")


def test_tensor_list_follows_the_config():
    from llama_gguf_b200 import madudra

    cfg = S.config([S.latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, mlp=S.moe(experts=3, top=2, ff=10)),
                    S.scan(heads=4, vdim=12, state=16, groups=2, conv=4), S.latent(heads=2, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, kv_from=0)],
                   width=32, vocab=50, streams=2)
    t = madudra.tensor_shapes(cfg)
    assert t["l0.mix.dq"] == (40, 32) and t["l0.mix.dq.norm"] == (40,) and t["l0.mix.uq"] == (72, 40) and t["l0.mix.dkv"] == (40, 32)
    assert t["l0.mix.dkv.norm"] == (32,) and t["l0.mix.uk"] == (48, 32) and t["l0.mix.uv"] == (72, 32) and t["l0.mix.g"] == (72, 32)
    assert t["l0.mix.o"] == (32, 72) and t["l0.mlp.router"] == (3, 32) and t["l0.mlp.e2.down"] == (32, 10) and "l0.mlp.e3.up" not in t
    assert t["l0.hc1.mix"] == (2, 2) and t["l0.hc2.in"] == (2,) and "l1.hc2.in" not in t and "l1.norm2" not in t
    assert t["l1.mix.in"] == (2 * 48 + 2 * 32 + 4, 32) and t["l1.mix.conv"] == (48 + 64, 4) and t["l1.mix.conv.b"] == (112,)
    assert t["l1.mix.A_log"] == (4,) and t["l1.mix.norm"] == (48,) and t["l1.mix.o"] == (32, 48)
    assert "l2.mix.dkv" not in t and "l2.mix.dkv.norm" not in t and t["l2.mix.uk"] == (32, 32)
    assert "l0.hc1.in" not in madudra.tensor_shapes(S.config([S.scan()], streams=None))
    assert set(S.random_weights(cfg, 0)) == set(t)


def test_registry_knows_the_architecture(tmp_path):
    from llama_gguf_b200 import registry

    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"architecture": "Madudra"}))
    assert registry.architecture_of(str(d)) == "Madudra"
    assert {"Madudra", "Mefurax", "Lazilorn"} <= set(registry.LOADERS)

"""Marosun on the GPU against the plain oracle (tests/marosun_oracle.py): every mechanism alone, prompts against token-by-token
decoding, portions, unequal batches, slot reuse, chunk edges, far keys and far states, odd sizes, greedy generation through the scheduler.

The library runs in its f32 compute mode where the comparison has to be sharp (errors ~1e-6) and in bf16 mode with a bound that a
wrong mechanism exceeds by orders of magnitude."""
import copy

import numpy as np
import pytest

import marosun_oracle as O
import marosun_synth as S

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4
BF16_TOL = 6e-2


def tokens(n, vocab, seed=1):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def check_whole(cfg, n, seed=0, compute="float32", tol=F32_TOL, taps=True, w=None):
    w = w if w is not None else S.random_weights(cfg, seed)
    ref = O.Model(cfg, w)
    toks = tokens(n, cfg["vocab"], seed + 1)
    rt = []
    want = ref.forward(toks, rt)
    gpu = S.gpu_model(cfg, w, compute, max_seq_len=n + 8, taps=taps)
    try:
        got = gpu.step([(0, toks)], list(range(n)))
        if taps:
            gt = gpu.taps(n)
            assert gt.shape[0] == len(rt)
            for r in range(len(rt)):
                assert np.abs(gt[r] - rt[r]).max() <= tol * np.abs(rt[r]).max() * 4, f"residual stream after layer {r}"
        assert S.rel_err(got, want) < tol
    finally:
        gpu.close()
    return want


# ---------------------------------------------------------------------------------------------------- mechanisms alone
def test_attention_mixer_alone(b200):
    # biases, norm before the stretched rotation, turned values, learned term in the denominator, grouped heads; no feed-forward
    check_whole(S.config([S.layer_a()]), 40)


def test_attention_mixer_without_stretching_and_whole_head_rotated(b200):
    check_whole(S.config([S.layer_a(dim=16, vdim=16, r=S.rot(dims=16, base=50.0, scaling=False))]), 33, seed=1)


def test_stretch_ramp_inside_the_pair_range(b200):
    # lo and hi of the ramp fall strictly inside the pairs: some frequencies untouched, some divided, some in between
    r = S.rot(dims=24, base=10000.0, scaling={"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0})
    fr, gain = O.stretched_frequencies(24, 10000.0, r["scaling"])
    plain = O.pair_frequencies(24, 10000.0)
    ratios = [a / b for a, b in zip(fr, plain)]
    assert ratios[0] == 1.0 and abs(ratios[-1] - 0.25) < 1e-12 and any(0.26 < x < 0.99 for x in ratios) and gain > 1.1
    check_whole(S.config([S.layer_a(r=r)]), 70, seed=2)


def test_chunked_attention_beside_gated_memory(b200):
    check_whole(S.config([S.layer_p()]), 40, seed=3)


@pytest.mark.parametrize("left,right", [(1.0, 0.0), (0.0, 1.0)])
def test_branches_of_the_weighted_pair_alone(b200, left, right):
    check_whole(S.config([S.layer_p(left_scale=left, right_scale=right)]), 30, seed=4)


def test_attention_beside_gated_unit(b200):
    check_whole(S.config([S.layer_q()]), 40, seed=5)


def test_clamped_feed_forward_bites(b200):
    # a limit well inside the spread of the pre-activations: all three clamps act
    cfg = S.config([S.layer_a(mlp=S.dense(88, limit=0.4))])
    want = check_whole(cfg, 24, seed=6)
    loose = copy.deepcopy(cfg)
    loose["layers"][0]["mlp"]["limit"] = 50.0
    assert S.rel_err(O.Model(loose, S.random_weights(cfg, 6)).forward(tokens(24, cfg["vocab"], 7)), want) > 50 * F32_TOL


def test_mixture_of_experts(b200):
    check_whole(S.config([S.layer_p(mlp=S.moe(experts=6, top=3, ff=24))]), 30, seed=8)


def test_mixture_single_choice_and_every_expert(b200):
    check_whole(S.config([S.layer_q(mlp=S.moe(experts=3, top=1, ff=20)), S.layer_a(mlp=S.moe(experts=4, top=4, ff=12))]), 26, seed=9)


def test_expert_weight_goes_on_the_input(b200):
    # the score scales what the expert READS: with a blown-up expert the difference to a weight on the output is large
    cfg = S.config([S.layer_a(mlp=S.moe(experts=5, top=2, ff=16))], width=48)
    w = S.random_weights(cfg, 10)
    w["l0.mlp.e2.down"] = w["l0.mlp.e2.down"] * 8
    want = check_whole(cfg, 40, seed=10, w=w)
    ref = O.Model(cfg, w)

    def on_output(h, w_, pre, experts, top):      # what a weight on the expert's OUTPUT would give
        s = O.sigmoid(w_[pre + "router"] @ h)
        return sum(s[e] * O.expert(h, w_[pre + "e%d.gate" % e], w_[pre + "e%d.up" % e], w_[pre + "e%d.down" % e]) for e in O.route(list(s), top))

    keep = O.mixture_ff
    try:
        O.mixture_ff = on_output
        other = ref.forward(tokens(40, cfg["vocab"], 11))
    finally:
        O.mixture_ff = keep
    assert S.rel_err(other, want) > 50 * F32_TOL


def full_cfg():
    return S.config([S.layer_a(mlp=S.dense(72)), S.layer_q(mlp=S.moe()), S.layer_p(chunk=5, mlp=S.moe(experts=4, top=1, ff=16)),
                     S.layer_a(kv_heads=1, mlp=None), S.layer_p(kv_heads=4, chunk=11, mlp=S.dense(40, limit=0.8)), S.layer_q(kv_heads=1, mlp=S.dense(24))])


def test_whole_model(b200):
    check_whole(full_cfg(), 45, seed=12)


def test_bf16_mode_whole_model(b200):
    check_whole(full_cfg(), 48, seed=13, compute="bfloat16", tol=BF16_TOL, taps=False)


# ---------------------------------------------------------------------------------------------------- other sizes
@pytest.mark.parametrize("layers,width", [
    # one head, sizes that are not multiples of 4 / 8 / 32, a chunk of one position, one expert
    ([S.layer_a(heads=1, kv_heads=1, dim=10, vdim=14, r=S.rot(dims=6), mlp=S.dense(20)),
      S.layer_p(heads=1, kv_heads=1, dim=10, vdim=14, chunk=1, r_heads=1, r_dim=6, r_vdim=10, mlp=S.moe(experts=1, top=1, ff=6)),
      S.layer_q(heads=1, kv_heads=1, dim=10, vdim=14, r=S.rot(dims=10, scaling=False), r_width=9, mlp=None)], 36),
    # wide heads (keys above 128, values above 128), one K/V head for all query heads, memory keys above 128, a chunk longer than the prompt
    ([S.layer_a(heads=4, kv_heads=1, dim=136, vdim=144, r=S.rot(dims=64)),
      S.layer_p(heads=2, kv_heads=1, dim=160, vdim=136, chunk=500, r_heads=2, r_dim=136, r_vdim=40),
      S.layer_q(heads=2, kv_heads=2, dim=32, vdim=200, r=S.rot(dims=8, scaling=True), r_width=300)], 96),
    # as many K/V heads as query heads; branch sizes that differ from each other in every way
    ([S.layer_p(heads=6, kv_heads=6, dim=8, vdim=12, chunk=9, r_heads=5, r_dim=33, r_vdim=7, left_scale=2.0, right_scale=0.25, mlp=S.moe(experts=9, top=4, ff=8)),
      S.layer_q(heads=6, kv_heads=3, dim=12, vdim=8, r_width=130, mlp=S.dense(36, limit=2.0))], 72),
])
def test_other_sizes(b200, layers, width):
    check_whole(S.config(layers, width=width, vocab=70, eps=1e-6), 37, seed=14)


# ---------------------------------------------------------------------------------------------------- prompts, portions, batches, slots
def test_prompt_against_token_by_token(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 15)
    toks = tokens(40, cfg["vocab"], 16)
    gpu = S.gpu_model(cfg, w)
    try:
        whole = gpu.step([(0, toks)], list(range(len(toks))))
        one = np.stack([gpu.forward(t, seq=1) for t in toks])
        assert S.rel_err(one, whole) < F32_TOL
        assert S.rel_err(whole, O.Model(cfg, w).forward(toks)) < F32_TOL
    finally:
        gpu.close()


@pytest.mark.parametrize("portion", [2, 3, 7, 16])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_portions(b200, portion, compute):
    # the cache, both recurrent states and the chunk count have to carry over the cuts
    cfg = full_cfg()
    w = S.random_weights(cfg, 17)
    toks = tokens(37, cfg["vocab"], 18)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w, compute)
    try:
        got = []
        for a in range(0, len(toks), portion):
            part = toks[a:a + portion]
            got.append(gpu.step([(1, part)], list(range(len(part)))))
        assert S.rel_err(np.concatenate(got), want) < (F32_TOL if compute == "float32" else BF16_TOL)
    finally:
        gpu.close()


def test_unequal_batch_against_each_alone(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 19)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 20 + n) for n in (1, 13, 29, 6)]
    tails = [tokens(9, cfg["vocab"], 40 + i) for i in range(4)]
    gpu = S.gpu_model(cfg, w, max_batch=6)
    try:
        slots = [4, 0, 2, 5]
        got = gpu.step(list(zip(slots, prompts)), list(range(sum(len(p) for p in prompts))))
        at, states = 0, []
        for p in prompts:
            st = ref.new_state()
            assert S.rel_err(got[at:at + len(p)], ref.step(st, p)) < F32_TOL
            states.append(st)
            at += len(p)
        for k in range(9):                                          # the shortest request ends first, then the next one
            alive = [i for i in range(4) if k < 3 + 2 * i]
            lg = gpu.decode_batch([slots[i] for i in alive], [tails[i][k] for i in alive])
            for j, i in enumerate(alive):
                assert S.rel_err(lg[j], ref.step(states[i], [tails[i][k]])[0]) < F32_TOL, (k, i)
    finally:
        gpu.close()


def test_bf16_batch_rows_do_not_depend_on_the_batch(b200):
    cfg = S.config([S.layer_a(dim=32, mlp=S.dense(72)), S.layer_p(dim=32, chunk=20, mlp=S.moe()), S.layer_q(dim=32)])
    w = S.random_weights(cfg, 21)
    a, b = tokens(21, cfg["vocab"], 1), tokens(40, cfg["vocab"], 2)
    gpu = S.gpu_model(cfg, w, "bfloat16")
    try:
        alone = gpu.step([(0, a)], list(range(len(a))))
        both = gpu.step([(1, b), (2, a)], list(range(len(b), len(b) + len(a))))
        assert S.rel_err(both, alone) < 2e-2
        assert S.rel_err(alone, O.Model(cfg, w).forward(a)) < BF16_TOL
    finally:
        gpu.close()


def test_slots_freed_and_used_again(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 22)
    ref = O.Model(cfg, w)
    gpu = S.gpu_model(cfg, w, max_batch=3)
    try:
        assert gpu.pool_counts() == (0, 0)
        a, b, c = tokens(30, cfg["vocab"], 3), tokens(18, cfg["vocab"], 4), tokens(25, cfg["vocab"], 5)
        gpu.step([(0, a), (1, b)])
        assert gpu.pool_counts() == (2, 0)
        gpu.reset(0)
        assert gpu.pool_counts() == (1, 1) and gpu.position(0) == 0
        # slot 2 takes the block that slot 0 left (full of a's keys and states); slot 1 goes on undisturbed
        got = gpu.step([(2, c)], list(range(len(c))))
        assert gpu.pool_counts() == (2, 0)
        assert S.rel_err(got, ref.forward(c)) < F32_TOL
        st = ref.new_state()
        ref.step(st, b)
        for t in tokens(5, cfg["vocab"], 6):
            assert S.rel_err(gpu.forward(t, seq=1), ref.step(st, [t])[0]) < F32_TOL
        gpu.reset(2)
        gpu.reset(1)
        got = gpu.step([(1, a)], [len(a) - 1])
        assert S.rel_err(got, ref.forward(a)[-1]) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- chunk edges
def edge_cfg(size):
    # the chunked branch alone with scores of order one: every visible key carries a few percent of the weight, so one key more or
    # less in view moves the logits far beyond the tolerance
    return S.config([S.layer_p(heads=2, kv_heads=1, dim=16, vdim=24, chunk=size, scale=1.0, r_heads=1, r_dim=8, r_vdim=8, left_scale=1.0, right_scale=0.05)],
                    width=48, vocab=64)


@pytest.mark.parametrize("decode", [False, True])
def test_chunk_edges(b200, decode):
    size = 11
    cfg = edge_cfg(size)
    w = S.random_weights(cfg, 23)
    w["l0.mix.left.sink"] = w["l0.mix.left.sink"] * 0 - 2.0      # (a small extra term: the keys keep most of the weight)
    n = 64
    toks = tokens(n, cfg["vocab"], 24)
    want = O.Model(cfg, w).forward(toks)
    # the oracle itself must tell the neighbouring chunk sizes apart at most positions, or the test would prove nothing
    for other in (size - 1, size + 1):
        alt_cfg = copy.deepcopy(cfg)
        alt_cfg["layers"][0]["mixer"]["left"]["mask"]["size"] = other
        alt = O.Model(alt_cfg, w).forward(toks)
        far = [p for p in range(size + 2, n) if S.rel_err(alt[p], want[p]) > 20 * F32_TOL]
        assert len(far) > (n - size) // 2, other
    gpu = S.gpu_model(cfg, w)
    try:
        if decode:
            gpu.step([(0, toks[:3])])
            for p in range(3, n):
                assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
        else:
            got = gpu.step([(0, toks)], list(range(n)))
            for p in range(n):
                assert S.rel_err(got[p], want[p]) < F32_TOL, p
    finally:
        gpu.close()


def test_chunks_count_from_the_sequence_start_not_from_the_cut(b200):
    # a prompt cut in the middle of a chunk: the second portion's first tokens still see the first portion's last ones, and nothing else
    cfg = edge_cfg(8)
    w = S.random_weights(cfg, 25)
    toks = tokens(40, cfg["vocab"], 26)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        a = gpu.step([(0, toks[:13])], list(range(13)))
        b = gpu.step([(0, toks[13:])], list(range(27)))
        assert S.rel_err(np.concatenate([a, b]), want) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- the extra denominator term
def test_learned_denominator_term_matters_and_is_there(b200):
    # large positive terms take most of the weight away from the keys: a model that left them out would be far off
    cfg = S.config([S.layer_a(scale=0.3), S.layer_p(scale=0.3)])
    w = S.random_weights(cfg, 27)
    w["l0.mix.sink"] = S.round_bf16(np.array([3.0, -1.0, 2.0, 0.5]))
    w["l1.mix.left.sink"] = S.round_bf16(np.array([2.5, 1.0, -0.5, 3.5]))
    want = check_whole(cfg, 30, seed=27, w=w)
    off = dict(w)
    off["l0.mix.sink"] = w["l0.mix.sink"] * 0 - 60.0
    off["l1.mix.left.sink"] = w["l1.mix.left.sink"] * 0 - 60.0
    assert S.rel_err(O.Model(cfg, off).forward(tokens(30, cfg["vocab"], 28)), want) > 100 * F32_TOL


def test_one_added_to_the_denominator_matters_and_is_there(b200):
    cfg = S.config([S.layer_q(scale=0.1)])
    want = check_whole(cfg, 12, seed=29)
    keep = O.softmax_with_extra
    try:
        O.softmax_with_extra = lambda scores, extra: keep(scores, -80.0)
        other = O.Model(cfg, S.random_weights(cfg, 29)).forward(tokens(12, cfg["vocab"], 30))
    finally:
        O.softmax_with_extra = keep
    assert S.rel_err(other, want) > 100 * F32_TOL


# ---------------------------------------------------------------------------------------------------- far keys
def plant_probe(cfg, w, needle, probe, q_name, target):
    """the probe token's embedding row is solved for so that its projected query is `target` (up to a positive factor)"""
    e = np.linalg.pinv(w[q_name].astype(np.float64)) @ target
    w["embed"][probe] = S.round_bf16(e * (np.linalg.norm(w["embed"][needle]) / np.linalg.norm(e)))


def test_far_key_through_rotation_and_turned_values(b200):
    # position ~300 still sees position 8.  Plain norms (weights one, no biases) keep directions, so the probe token's query can be
    # aimed at the needle's key as it looks from 293 positions away; that one score stands out among hundreds of random ones, and
    # the output is the needle's value turned by the distance -- a wrong sign or position in either rotation would show.
    cfg = S.config([S.layer_a(heads=2, kv_heads=1, dim=16, vdim=24, r=S.rot(dims=4, base=200.0, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}),
                              scale=1.0)], width=48, vocab=64)
    m = cfg["layers"][0]["mixer"]
    w = S.random_weights(cfg, 31)
    for n_ in ("q", "k", "v", "o"):
        w["l0.mix.%s.b" % n_] = 0 * w["l0.mix.%s.b" % n_]
    w["l0.mix.q.norm"] = 0 * w["l0.mix.q.norm"] + 1
    w["l0.mix.k.norm"] = 0 * w["l0.mix.k.norm"] + 1
    w["l0.norm1"] = 0 * w["l0.norm1"]
    w["l0.mix.sink"] = 0 * w["l0.mix.sink"]
    n = 310
    toks = tokens(n, cfg["vocab"] - 2, 32)
    needle, probe = cfg["vocab"] - 2, cfg["vocab"] - 1
    k_needle = (w["l0.mix.k"].astype(np.float64) @ w["embed"][needle]).reshape(m["kv_heads"], m["dim"])
    fr, _ = O.stretched_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"]["scaling"])
    k_seen = np.stack([O.turn_pairs(r, 8 - 301, fr) for r in k_needle])     # q_p . R(8 - p) k: aimed from position 301
    plant_probe(cfg, w, needle, probe, "l0.mix.q", np.concatenate([k_seen[0]] * m["heads"]))
    toks[8] = needle
    for p in range(296, n):
        toks[p] = probe
    ref = O.Model(cfg, w)
    want = ref.forward(toks)
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        got = gpu.step([(0, toks[:300])], list(range(290, 300)))
        assert S.rel_err(got, want[290:300]) < F32_TOL
        for p in range(300, n):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()
    # with the needle replaced the answers at the far end change: the far key is really seen, in the prompt and in decoding
    toks2 = list(toks)
    toks2[8] = 0
    alt = ref.forward(toks2)
    for p in (299, 300, 301):
        assert S.rel_err(alt[p], want[p]) > 40 * F32_TOL, p


def test_far_key_inside_a_long_chunk(b200):
    # the chunk of 320 holds position 8 for position 300; position 320 starts a new chunk and has lost it
    cfg = edge_cfg(320)
    m = cfg["layers"][0]["mixer"]["left"]
    w = S.random_weights(cfg, 33)
    w["l0.norm1"] = 0 * w["l0.norm1"]
    w["l0.mix.left.sink"] = 0 * w["l0.mix.left.sink"]
    n = 326
    toks = tokens(n, cfg["vocab"] - 2, 34)
    needle, probe = cfg["vocab"] - 2, cfg["vocab"] - 1
    k_needle = (w["l0.mix.left.k"].astype(np.float64) @ w["embed"][needle]).reshape(m["kv_heads"], m["dim"])
    plant_probe(cfg, w, needle, probe, "l0.mix.left.q", np.concatenate([k_needle[0]] * m["heads"]))
    toks[8] = needle
    for p in range(296, n):
        toks[p] = probe
    ref = O.Model(cfg, w)
    want = ref.forward(toks)
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        got = gpu.step([(0, toks[:300])], list(range(290, 300)))
        assert S.rel_err(got, want[290:300]) < F32_TOL
        for p in range(300, n):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()
    toks2 = list(toks)
    toks2[8] = 0
    alt = ref.forward(toks2)
    for p in (299, 300, 319):
        assert S.rel_err(alt[p], want[p]) > 40 * F32_TOL, p
    # beyond the chunk's end only the memory branch (weight 0.05, short memory) could still know: the attention has lost the needle
    assert S.rel_err(alt[322:], want[322:]) < S.rel_err(alt[319], want[319]) / 20


# ---------------------------------------------------------------------------------------------------- far states
@pytest.mark.parametrize("kind", ["memory", "unit"])
def test_state_written_early_shapes_answers_hundreds_of_tokens_on(b200, kind):
    # The gates read one direction of the mixer's input, the needle token's: that token (position 5) overwrites most of the state,
    # every other token leaves it nearly as it is (forget gates ~0.997, update gates ~0.004).  What it wrote is still there at token
    # 300, through a prompt cut in two and decoding.
    W = 48
    if kind == "memory":
        cfg = S.config([S.layer_p(heads=2, kv_heads=1, dim=16, vdim=16, chunk=4, left_scale=0.1, right_scale=1.0)], width=W, vocab=64)
    else:
        cfg = S.config([S.layer_q(heads=2, kv_heads=1, dim=16, vdim=16, r_width=40)], width=W, vocab=64)
    w = S.random_weights(cfg, 35)
    w["l0.norm1"] = 0 * w["l0.norm1"]
    needle = cfg["vocab"] - 1
    hn = w["embed"][needle].astype(np.float64)
    hn = hn / np.sqrt(np.mean(hn * hn) + cfg["norm"]["eps"])
    if kind == "memory":
        rows = w["l0.mix.right.f"].shape[0]
        w["l0.mix.right.lower"] = 0 * w["l0.mix.right.lower"]
        w["l0.mix.right.f.b"] = 0 * w["l0.mix.right.f.b"] + 6.0
        w["l0.mix.right.f"] = S.round_bf16(np.outer(np.ones(rows), -12.0 / W * hn))
    else:
        rows = w["l0.mix.right.z"].shape[0]
        w["l0.mix.right.z.b"] = 0 * w["l0.mix.right.z.b"] - 6.0
        w["l0.mix.right.z"] = S.round_bf16(np.outer(np.ones(rows), 8.0 / W * hn))
        w["l0.mix.left.out"] = w["l0.mix.left.out"] * 0.05
    n = 306
    toks = tokens(n, cfg["vocab"] - 1, 36)
    toks[5] = needle
    ref = O.Model(cfg, w)
    want = ref.forward(toks)
    toks2 = list(toks)
    toks2[5] = 0
    alt = ref.forward(toks2)
    assert min(S.rel_err(alt[p], want[p]) for p in range(296, n)) > 20 * F32_TOL
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        gpu.step([(0, toks[:131])])
        got = gpu.step([(0, toks[131:300])], list(range(159, 169)))
        assert S.rel_err(got, want[290:300]) < F32_TOL
        for p in range(300, n):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()


def test_first_tokens_and_long_decoding(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 37)
    toks = tokens(120, cfg["vocab"], 38)      # more than ten chunks decoded one by one, from the very first token
    ref = O.Model(cfg, w)
    st = ref.new_state()
    gpu = S.gpu_model(cfg, w)
    try:
        for p, t in enumerate(toks):
            assert S.rel_err(gpu.forward(t), ref.step(st, [t])[0]) < F32_TOL, p
    finally:
        gpu.close()


def test_rotations_at_large_positions(b200):
    # angles in the thousands of radians, for keys and for values: an f32 angle would already be off in the fourth digit
    cfg = S.config([S.layer_a(heads=2, kv_heads=2, dim=16, vdim=16, r=S.rot(dims=16, base=4.0, scaling=False), scale=0.4)], width=32, vocab=40)
    w = S.random_weights(cfg, 39)
    n = 1500
    toks = tokens(n, cfg["vocab"], 40)
    ref = O.Model(cfg, w)
    # the oracle only has to answer at the last positions; it is quadratic, so its earlier tokens look at themselves only
    keep = O.sees_all
    try:
        O.sees_all = lambda t, s: s <= t and (t >= n - 2 or s == t)
        want = ref.forward(toks)[-2:]
    finally:
        O.sees_all = keep
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        got = gpu.step([(0, toks)], [n - 2, n - 1])
        assert S.rel_err(got, want) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- the scheduler
def test_greedy_generation_through_the_batched_engine(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 41)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 50 + n) for n in (5, 17, 9, 26, 3)]
    n_new = [6, 4, 8, 5, 7]
    want = []
    for p, k in zip(prompts, n_new):
        st = ref.new_state()
        lg = ref.step(st, p)[-1]
        out = []
        for _ in range(k):
            t = int(len(lg) - 1 - np.argmax(lg[::-1]))      # last maximum wins
            out.append(t)
            lg = ref.step(st, [t])[0]
        want.append(out)
    gpu = S.gpu_model(cfg, w, max_batch=3)
    eng = b200.BatchedEngine(gpu, max_batch_size=3, max_seq_len=200, eos_token_id=cfg["vocab"] + 7)   # (no token is EOS)
    try:
        ids = [eng.submit(p, k) for p, k in zip(prompts, n_new)]   # five requests on three slots: two wait, slots are reused
        got = {i: [] for i in ids}
        done = {}
        for ev in eng.run():
            if ev[0] == "token":
                got[ev[1]].append(ev[2])
            elif ev[0] == "done":
                done[ev[1]] = ev[2:]
            else:
                raise AssertionError(ev)
        for i, rid in enumerate(ids):
            assert got[rid] == want[i], i
            assert done[rid] == ("max_tokens", len(prompts[i]), n_new[i])
        assert gpu.pool_counts()[0] <= 3
    finally:
        eng.close()
        gpu.close()


def test_decode_greedy_entry_point(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 43)
    ref = O.Model(cfg, w)
    p = tokens(12, cfg["vocab"], 44)
    st = ref.new_state()
    ref.step(st, p[:-1])
    gpu = S.gpu_model(cfg, w)
    try:
        gpu.step([(0, p[:-1])])
        out, _ = gpu.decode_greedy(p[-1], 6)
        t, want = p[-1], []
        for _ in range(6):
            lg = ref.step(st, [t])[0]
            t = int(len(lg) - 1 - np.argmax(lg[::-1]))
            want.append(t)
        assert out.tolist() == want
    finally:
        gpu.close()


def test_bad_arguments(b200):
    cfg = S.config([S.layer_a()])
    w = S.random_weights(cfg, 45)
    gpu = S.gpu_model(cfg, w, max_seq_len=16)
    try:
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(0, [cfg["vocab"]])])
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(0, tokens(17, cfg["vocab"]))])
        assert gpu.path() == "layers"
    finally:
        gpu.close()
    del w["l0.mix.sink"]
    with pytest.raises(b200.InvalidArgument):
        S.gpu_model(cfg, w)
    bad = S.config([S.layer_a(vdim=41)])          # turned values come in pairs
    with pytest.raises(b200.InvalidArgument):
        S.gpu_model(bad, S.random_weights(bad, 46))


# ---------------------------------------------------------------------------------------------------- kernels against their plain forms
@pytest.mark.parametrize("kind,dims", [("a", (16, 24, 0)), ("a", (128, 128, 0)), ("p", (96, 56, 23)), ("p", (64, 40, 64)), ("q", (32, 40, 0))])
def test_tile_attention_against_warp_attention(b200, monkeypatch, kind, dims):
    # bf16 prompts take the tensor-pipe attention kernel when the head sizes allow it; the warp kernel computes the same thing in f32.
    # The extra denominator term, the turn-back of the summed values and the gate sit in both kernels' last lines.  Several unequal
    # runs in one step, one of them continued afterwards (its cache then holds rows of both steps).
    dim, vdim, size = dims
    if kind == "a":
        cfg = S.config([S.layer_a(heads=4, kv_heads=2, dim=dim, vdim=vdim)], width=64, vocab=80)
    elif kind == "p":
        cfg = S.config([S.layer_p(heads=4, kv_heads=2, dim=dim, vdim=vdim, chunk=size)], width=64, vocab=80)
    else:
        cfg = S.config([S.layer_q(heads=4, kv_heads=2, dim=dim, vdim=vdim)], width=64, vocab=80)
    w = S.random_weights(cfg, 47)
    a, b, c = tokens(150, cfg["vocab"], 1), tokens(64, cfg["vocab"], 2), tokens(17, cfg["vocab"], 3)
    more = tokens(70, cfg["vocab"], 4)
    outs = {}
    for tile in ("1", "0"):
        monkeypatch.setenv("B200_LP_ATTN_TILE", tile)
        gpu = S.gpu_model(cfg, w, "bfloat16", max_seq_len=256)
        try:
            first = gpu.step([(0, a), (1, b), (2, c)], list(range(len(a) + len(b) + len(c))))
            second = gpu.step([(1, more)], list(range(len(more))))
            outs[tile] = np.concatenate([first, second])
        finally:
            gpu.close()
    ref = O.Model(cfg, w)
    bm = ref.forward(b + more)
    want = np.concatenate([ref.forward(a), bm[:len(b)], ref.forward(c), bm[len(b):]])
    assert S.rel_err(outs["1"], outs["0"]) < 2e-2
    assert S.rel_err(outs["1"], want) < BF16_TOL
    assert S.rel_err(outs["0"], want) < BF16_TOL


def test_tensor_core_gemm_path(b200, monkeypatch):
    # bf16 mode with enough rows for the tcgen05 GEMM (the layer's one input projection with the feed-forward's part in it, biased
    # output projections, the experts' grouped products, K that is not a multiple of 64) against the CUDA-core kernel
    cfg = S.config([S.layer_a(heads=4, kv_heads=2, dim=32, vdim=40, mlp=S.dense(200)),
                    S.layer_q(heads=4, kv_heads=2, dim=32, vdim=40, r_width=104, mlp=S.moe(experts=6, top=2, ff=40)),
                    S.layer_p(heads=4, kv_heads=2, dim=32, vdim=40, chunk=50, r_heads=2, r_dim=32, r_vdim=24, mlp=S.moe(experts=4, top=1, ff=24))], width=168, vocab=300)
    w = S.random_weights(cfg, 48)
    toks = tokens(300, cfg["vocab"], 49)
    outs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("B200_LP_TC", tc)
        gpu = S.gpu_model(cfg, w, "bfloat16", max_seq_len=320)
        try:
            rows = [gpu.step([(0, toks[:n])], list(range(n))) for n in (40, 100)]
            gpu.reset(0)
            rows.append(gpu.step([(1, toks)], list(range(300))))
            outs[tc] = rows
        finally:
            gpu.close()
    # (a router logit that the two summation orders put on different sides of a neighbour flips an expert: rows are compared in bulk)
    for a, b in zip(outs["1"], outs["0"]):
        d = np.array([S.rel_err(a[i], b[i]) for i in range(len(a))])
        assert np.median(d) < 1.5e-2 and (d < 1.5e-2).mean() > 0.9
    ref = O.Model(cfg, w).forward(toks)
    d = np.array([S.rel_err(outs["1"][2][i], ref[i]) for i in range(300)])
    assert np.median(d) < BF16_TOL and (d < BF16_TOL).mean() > 0.9


def test_decode_kernels_for_few_rows_against_the_many_row_path(b200, monkeypatch):
    # decoding reads only the chosen experts' weights and takes the norm inside the layer's input projection; B200_LP_FUSE=0 sends
    # the same rows through separate kernels and the products over all experts.  Both against the oracle, in a batch whose members
    # sit at different positions, in f32; and against each other in bf16.
    cfg = S.config([S.layer_a(mlp=S.moe(experts=6, top=2, ff=24)), S.layer_p(mlp=S.moe(experts=3, top=3, ff=8)),
                    S.layer_q(mlp=S.moe(experts=4, top=1, ff=32)), S.layer_p(chunk=4, mlp=S.dense(40))])
    w = S.random_weights(cfg, 53)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 60 + n) for n in (3, 19, 1)]
    tails = [tokens(12, cfg["vocab"], 70 + i) for i in range(3)]
    states = [ref.new_state() for _ in prompts]
    for st, pr in zip(states, prompts):
        ref.step(st, pr)
    want = [[ref.step(states[i], [tails[i][k]])[0] for i in range(3)] for k in range(12)]
    bf = {}
    for fuse in ("1", "0"):
        monkeypatch.setenv("B200_LP_FUSE", fuse)
        for compute in ("float32", "bfloat16"):
            gpu = S.gpu_model(cfg, w, compute)
            try:
                gpu.step([(i, pr) for i, pr in enumerate(prompts)])
                rows = []
                for k in range(12):
                    lg = gpu.decode_batch([0, 1, 2], [tails[i][k] for i in range(3)])
                    rows.append(lg)
                    if compute == "float32":
                        for i in range(3):
                            assert S.rel_err(lg[i], want[k][i]) < F32_TOL, (fuse, k, i)
                if compute == "bfloat16":
                    bf[fuse] = np.concatenate(rows)
            finally:
                gpu.close()
    d = np.array([S.rel_err(bf["1"][i], bf["0"][i]) for i in range(len(bf["1"]))])
    assert np.median(d) < 2e-2 and (d < 2e-2).mean() > 0.9


@pytest.mark.parametrize("compute,rows", [("float32", 4), ("float32", 3), ("bfloat16", 8), ("bfloat16", 7), ("float32", 16)])
def test_few_rows_against_wide_matrices(b200, compute, rows):
    # a handful of rows whose staged copy for a wide output projection (64 heads x 48 = 3072 inputs) or down projection (3072) comes
    # to exactly, or just under, the shared memory that a launch gets without opting in; more rows than that go unstaged
    cfg = S.config([S.layer_p(heads=64, kv_heads=8, dim=8, vdim=48, chunk=5, r_heads=2, r_dim=16, r_vdim=24, mlp=S.dense(3072, limit=2.0)),
                    S.layer_a(heads=2, kv_heads=1, dim=16, vdim=16, r=S.rot(dims=8), mlp=S.moe(experts=4, top=2, ff=16))], width=96, vocab=60)
    w = S.random_weights(cfg, 81)
    toks = tokens(2 * rows + 1, cfg["vocab"], 82)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w, compute)
    try:
        got = [gpu.step([(0, toks[:rows])], list(range(rows))), gpu.step([(0, toks[rows:2 * rows])], list(range(rows))),
               gpu.step([(0, toks[2 * rows:])], [0])]
        d = np.array([S.rel_err(g, wnt) for g, wnt in zip(np.concatenate(got), want)])
        if compute == "float32":
            assert d.max() < F32_TOL
        else:
            assert np.median(d) < BF16_TOL and (d < BF16_TOL).mean() > 0.8
    finally:
        gpu.close()


@pytest.mark.parametrize("dims", [(2, 20, 12), (1, 136, 40), (3, 64, 64)])
def test_gated_memory_cut_into_segments(b200, monkeypatch, dims):
    # long runs on an empty GPU are folded segment by segment and chained through carries: a batch of a long run, a run shorter than
    # the segment count (empty segments) and a middling one, then a second long portion that starts from the state the first left;
    # against the oracle, and the whole-run kernel (B200_LP_GLIN_SEG=0) against the same
    heads, dim, vdim = dims
    cfg = S.config([S.layer_p(chunk=50, r_heads=heads, r_dim=dim, r_vdim=vdim, mlp=None),
                    S.layer_p(heads=2, kv_heads=1, dim=16, vdim=8, chunk=9, r_heads=heads, r_dim=dim, r_vdim=vdim, left_scale=0.1, right_scale=2.0,
                              mlp=S.dense(24))], width=48, vocab=64)
    w = S.random_weights(cfg, 91)
    # a lower bound near one on half of the channels keeps old tokens alive across many segments
    for i in range(2):
        lo = w["l%d.mix.right.lower" % i]
        lo[::2] = S.round_bf16(np.full_like(lo[::2], 0.99))
    ref = O.Model(cfg, w)
    a, b, c = tokens(300 + 280, 64, 92), tokens(3, 64, 93), tokens(131, 64, 94)
    wa, wb, wc = ref.forward(a), ref.forward(b), ref.forward(c)
    for seg in ("1", "0"):
        monkeypatch.setenv("B200_LP_GLIN_SEG", seg)
        gpu = S.gpu_model(cfg, w, max_seq_len=600)
        try:
            g = gpu.step([(0, a[:300]), (1, b), (2, c)], list(range(300 + 3 + 131)))
            assert S.rel_err(g[:300], wa[:300]) < F32_TOL and S.rel_err(g[300:303], wb) < F32_TOL and S.rel_err(g[303:], wc) < F32_TOL, seg
            g = gpu.step([(0, a[300:])], list(range(280)))
            assert S.rel_err(g, wa[300:]) < F32_TOL, seg
            assert S.rel_err(gpu.decode_batch([1, 2], [5, 6])[0], ref.forward(b + [5])[-1]) < F32_TOL
        finally:
            gpu.close()


def test_many_rows_of_experts_in_f32(b200):
    # enough rows for the sorted (token, choice) form: pre-activations, the pair's weight on the input, plain sum of the choices
    cfg = S.config([S.layer_q(mlp=S.moe(experts=5, top=2, ff=24)), S.layer_a(mlp=S.moe(experts=3, top=1, ff=16))])
    check_whole(cfg, 90, seed=55)


def test_gated_unit_segments(b200):
    # run lengths around the segment count of the unit's scan (1, fewer tokens than segments, not a multiple, long), started from a
    # state that earlier steps left
    cfg = S.config([S.layer_q(r_width=70)], width=40, vocab=50)
    w = S.random_weights(cfg, 57)
    toks = tokens(1 + 5 + 8 + 13 + 100, cfg["vocab"], 58)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        got, at = [], 0
        for n in (1, 5, 8, 13, 100):
            got.append(gpu.step([(0, toks[at:at + n])], list(range(n))))
            at += n
        assert S.rel_err(np.concatenate(got), want) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- the command line
def test_trace_runner_on_a_model_folder(b200, tmp_path):
    # config.json + model.safetensors (bf16) on disk -> registry -> bin/trace_run: two requests start together with unequal prompts, are
    # decoded together, the shorter one ends first; logits of the wanted rows come back in files
    import json
    import os
    import subprocess
    import sys

    from llama_gguf_b200.safetensors_io import bf16_bits, write_safetensors

    cfg = full_cfg()
    w = S.random_weights(cfg, 51)
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {n: bf16_bits(a).reshape(a.shape) for n, a in w.items()})
    a, b = tokens(19, cfg["vocab"], 52), tokens(7, cfg["vocab"], 53)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:15], "want": [0, 14]}, {"id": "y", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[15:16], "want": []}, {"id": "y", "tokens": b[5:6], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[16:17], "want": [0]}, {"id": "y", "tokens": b[6:7], "want": [0]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": a[17:19], "want": [1]}], "end": ["x"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == ["done %d" % i for i in range(4)]
    ref = O.Model(cfg, w)
    wa, wb = ref.forward(a), ref.forward(b)
    got = {i: np.fromfile(str(out / ("%d.f32" % i)), dtype="<f4").reshape(-1, cfg["vocab"]) for i in range(4)}
    assert S.rel_err(got[0], np.stack([wa[0], wa[14], wb[4]])) < F32_TOL
    assert S.rel_err(got[1], wb[5:6]) < F32_TOL
    assert S.rel_err(got[2], np.stack([wa[16], wb[6]])) < F32_TOL
    assert S.rel_err(got[3], wa[18:19]) < F32_TOL

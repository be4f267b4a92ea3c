"""Madudra on the GPU against the plain oracle (tests/madudra_oracle.py): every mechanism alone, prompts against token-by-token
decoding, portions, unequal batches, slot reuse, window edges, far keys and far state, odd sizes, greedy generation through the scheduler.

The library runs in its f32 compute mode where the comparison has to be sharp (errors ~1e-6) and in bf16 mode with a bound that a
wrong mechanism exceeds by orders of magnitude."""
import copy
import math

import numpy as np
import pytest

import madudra_oracle as O
import madudra_synth as S

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4
BF16_TOL = 8e-2


def tokens(n, vocab, seed=1):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def check_whole(cfg, n, seed=0, compute="float32", tol=F32_TOL, taps=True, w=None):
    w = w if w is not None else S.random_weights(cfg, seed)
    toks = tokens(n, cfg["vocab"], seed + 1)
    want, rt = O.run(cfg, S.f64(w), toks)
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


class Ref:
    """The oracle fed in pieces: one Sequence per request."""

    def __init__(self, cfg, w):
        self.cfg, self.w = cfg, S.f64(w)

    def new(self):
        return O.Sequence(self.cfg, self.w)

    def step(self, seq, toks):
        return np.array([seq.token(t)[0] for t in toks])

    def forward(self, toks):
        return self.step(self.new(), toks)


# ---------------------------------------------------------------------------------------------------- mechanisms alone
def test_latent_attention_alone(b200):
    check_whole(S.config([S.latent()], streams=None, mult=1.0), 40, 1)


def test_latent_attention_without_frequency_scaling_and_with_partial_rotation(b200):
    check_whole(S.config([S.latent(scaling=None)], streams=None), 30, 2)
    check_whole(S.config([S.latent(rot_dim=12, rot_dims=8)], streams=None), 30, 3)


def test_frequency_scaling_touches_only_slow_pairs(b200):
    # the ramp's ends lie inside the pair range for this choice: some pairs keep their frequency, some are slowed by the full factor
    rot = {"dims": 16, "base": 100.0, "scaling": {"factor": 4.0, "original": 40, "fast": 8.0, "slow": 2.0}}
    f, mult = O.rot_table(rot)
    plain = np.array([100.0 ** (-2.0 * i / 16) for i in range(8)])
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 4.0) < 1e-15 and any(plain[i] / 4 < f[i] < plain[i] for i in range(8))
    assert abs(mult - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    check_whole(S.config([S.latent(rot_dim=16, base=100.0, scaling=rot["scaling"], window=50)], streams=None), 60, 4)


def test_state_space_mixer_alone(b200):
    check_whole(S.config([S.scan()], streams=None, mult=1.0), 40, 5)


def test_mixture_of_experts(b200):
    check_whole(S.config([S.scan(mlp=S.moe())], streams=None), 30, 6)
    check_whole(S.config([S.latent(mlp=S.moe(experts=7, top=7, ff=8, scale=0.5))], streams=None), 30, 7)     # every expert chosen
    check_whole(S.config([S.latent(mlp=S.moe(experts=3, top=1, ff=40, scale=2.0))], streams=None), 30, 8)


def test_router_weights_are_not_renormalised(b200):
    # one expert blown up: a renormalised weight (or a softmax over the chosen only) would move the output by far more than the bound
    cfg = S.config([S.scan(mlp=S.moe(experts=6, top=2, ff=16, scale=1.0))], streams=None)
    w = S.random_weights(cfg, 9)
    w["l0.mlp.router"] = 0.05 * w["l0.mlp.router"]          # nearly flat: the chosen two hold about a third of the probability
    w["l0.mlp.e4.down"] = 6.0 * w["l0.mlp.e4.down"]
    check_whole(cfg, 30, 9, w=w)


def test_streams(b200):
    for streams in (1, 2, 4):
        check_whole(S.config([S.scan(mlp=S.moe()), S.latent()], streams=streams), 24, 10 + streams)


def test_borrowed_cache_rows(b200):
    # the borrowing layer has its own window, heads and sizes per head; a state-space layer sits between the two
    cfg = S.config([S.latent(window=7, mlp=S.moe()), S.scan(), S.latent(heads=2, dim=12, vdim=20, q_rank=24, window=13, kv_from=0, mlp=S.moe()),
                    S.latent(window=5, kv_from=0)], streams=3)
    check_whole(cfg, 40, 15)


def full_cfg():
    return S.config([S.latent(mlp=S.moe()), S.scan(mlp=S.moe(experts=4, top=3, ff=16)), S.scan(heads=2, vdim=20, state=24, groups=1, conv=2,
                                                                                              norm_groups=1),
                     S.latent(kv_from=0, window=14, mlp=S.moe())], streams=3)


def test_whole_model(b200):
    check_whole(full_cfg(), 48, 16)


def test_bf16_mode_whole_model(b200):
    check_whole(full_cfg(), 48, 16, compute="bfloat16", tol=BF16_TOL, taps=False)


@pytest.mark.parametrize("layers,width,streams", [
    ([S.latent(heads=1, dim=10, rot_dim=6, vdim=7, q_rank=9, kv_rank=18, window=1)], 40, None),           # one head, window of one
    ([S.latent(heads=5, dim=4, rot_dim=2, vdim=3, q_rank=5, kv_rank=17, window=300)], 36, 2),            # odd row size: the scalar paths
    ([S.latent(heads=2, dim=40, rot_dim=24, vdim=72, q_rank=100, kv_rank=136, window=6, mlp=S.moe(experts=2, top=1, ff=4))], 72, 3),
    ([S.latent(heads=2, dim=8, rot_dim=0, vdim=8, q_rank=8, kv_rank=16, window=8, rot_dims=0, scaling=None)], 32, 1),   # nothing rotated
    ([S.scan(heads=1, vdim=5, state=3, groups=1, conv=1, norm_groups=1)], 24, None),                      # one tap: no tail
    ([S.scan(heads=6, vdim=10, state=40, groups=6, conv=2, norm_groups=6)], 40, 2),                       # a group per head
    ([S.scan(heads=2, vdim=70, state=130, groups=1, conv=5, norm_groups=4)], 48, 3),                      # state beyond 128, many columns
    ([S.scan(heads=3, vdim=33, state=64, groups=3, conv=3, norm_groups=3, mlp=S.moe(experts=9, top=4, ff=12))], 56, 5),
])
def test_other_sizes(b200, layers, width, streams):
    check_whole(S.config(layers, width=width, vocab=50, streams=streams, mult=0.9, embed_scale=1.0), 26, 17)


def test_no_window_sees_everything(b200):
    cfg = S.config([S.latent()], streams=None)
    del cfg["layers"][0]["mixer"]["mask"]
    toks = tokens(40, cfg["vocab"], 3)
    w = S.random_weights(cfg, 18)
    wide = copy.deepcopy(cfg)
    wide["layers"][0]["mixer"]["mask"] = {"size": 1000}
    want = Ref(wide, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        assert S.rel_err(gpu.step([(0, toks)], list(range(40))), want) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- prompts, portions, batches
def test_prompt_against_token_by_token(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 19)
    toks = tokens(34, cfg["vocab"], 20)
    want = Ref(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        rows = [gpu.forward(t) for t in toks]                       # every token decoded alone, from the first one
        assert S.rel_err(np.stack(rows), want) < F32_TOL
        assert gpu.position() == len(toks)
        gpu.reset()
        last = gpu.forward_batch(toks[:20])                         # prompt, then decoding
        assert S.rel_err(last, want[19]) < F32_TOL
        for p in range(20, len(toks)):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()


@pytest.mark.parametrize("portion", [2, 3, 7, 16])
def test_portions(b200, portion):
    # the convolution's tail, the matrix state and the cached rows (also the borrowed ones) all have to carry over the cuts
    cfg = full_cfg()
    w = S.random_weights(cfg, 21)
    toks = tokens(37, cfg["vocab"], 22)
    want = Ref(cfg, w).forward(toks)
    for compute, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        gpu = S.gpu_model(cfg, w, compute)
        try:
            got = []
            for a in range(0, len(toks), portion):
                part = toks[a:a + portion]
                got.append(gpu.step([(1, part)], list(range(len(part)))))
            assert S.rel_err(np.concatenate(got), want) < tol
        finally:
            gpu.close()


def test_unequal_batch_against_each_alone(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 23)
    ref = Ref(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 20 + n) for n in (1, 13, 29, 6)]
    tails = [tokens(9, cfg["vocab"], 40 + i) for i in range(4)]
    gpu = S.gpu_model(cfg, w, max_batch=6)
    try:
        slots = [4, 0, 2, 5]
        got = gpu.step(list(zip(slots, prompts)), list(range(sum(len(p) for p in prompts))))
        at, states = 0, []
        for p in prompts:
            st = ref.new()
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
    cfg = full_cfg()
    w = S.random_weights(cfg, 24)
    a, b = tokens(21, cfg["vocab"], 1), tokens(40, cfg["vocab"], 2)
    gpu = S.gpu_model(cfg, w, "bfloat16")
    try:
        alone = gpu.step([(0, a)], list(range(len(a))))
        both = gpu.step([(1, b), (2, a)], list(range(len(b), len(b) + len(a))))
        assert S.rel_err(both, alone) < 3e-2
    finally:
        gpu.close()


def test_slots_freed_and_used_again(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 25)
    ref = Ref(cfg, w)
    gpu = S.gpu_model(cfg, w, max_batch=3)
    try:
        assert gpu.pool_counts() == (0, 0)
        a, b, c = tokens(30, cfg["vocab"], 3), tokens(18, cfg["vocab"], 4), tokens(25, cfg["vocab"], 5)
        gpu.step([(0, a), (1, b)])
        assert gpu.pool_counts() == (2, 0)
        gpu.reset(0)
        assert gpu.pool_counts() == (1, 1) and gpu.position(0) == 0
        # slot 2 takes the block that slot 0 left (full of a's rows, matrix states and convolution tails); slot 1 goes on undisturbed
        got = gpu.step([(2, c)], list(range(len(c))))
        assert gpu.pool_counts() == (2, 0)
        assert S.rel_err(got, ref.forward(c)) < F32_TOL
        st = ref.new()
        ref.step(st, b)
        for t in tokens(5, cfg["vocab"], 6):
            assert S.rel_err(gpu.forward(t, seq=1), ref.step(st, [t])[0]) < F32_TOL
        gpu.reset(2)
        gpu.reset(1)
        got = gpu.step([(1, a)], [len(a) - 1])
        assert S.rel_err(got, ref.forward(a)[-1]) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- window edges, far keys, far state
def edge_cfg(size, borrowed=False):
    # scores of order one and a small embedding: every visible key carries a few percent of the weight and the mixer's output
    # shapes the logits, so one key more or less in view moves them far beyond the tolerance
    layers = [S.latent(heads=2, dim=16, rot_dim=8, vdim=24, window=size, scale=0.12)]
    if borrowed:
        layers = [S.latent(heads=2, dim=16, rot_dim=8, vdim=24, window=3, scale=0.12), S.latent(heads=2, dim=16, rot_dim=8, vdim=24, window=size, scale=0.12, kv_from=0)]
    return S.config(layers, width=48, vocab=64, streams=None, mult=1.0, embed_scale=0.3)


@pytest.mark.parametrize("borrowed", [False, True])
@pytest.mark.parametrize("decode", [False, True])
def test_window_edges(b200, decode, borrowed):
    size = 11
    cfg = edge_cfg(size, borrowed)
    w = S.random_weights(cfg, 26)
    n = 64
    toks = tokens(n, cfg["vocab"], 27)
    want = Ref(cfg, w).forward(toks)
    # the oracle itself must tell the neighbouring windows apart at most positions, or the test would prove nothing
    for other in (size - 1, size + 1):
        alt_cfg = copy.deepcopy(cfg)
        alt_cfg["layers"][-1]["mixer"]["mask"]["size"] = other
        alt = Ref(alt_cfg, w).forward(toks)
        far = [p for p in range(size + 2, n) if S.rel_err(alt[p], want[p]) > 20 * F32_TOL]
        assert len(far) > (n - size) // 2, other
    for compute, tol in (("float32", F32_TOL), ("bfloat16", None)):
        gpu = S.gpu_model(cfg, w, compute)
        try:
            if decode:
                gpu.step([(0, toks[:3])])
                got = np.stack([gpu.forward(toks[p]) for p in range(3, n)])
                ref = want[3:]
            else:
                got = gpu.step([(0, toks)], list(range(n)))         # (64 rows: the tile kernel in bf16 mode)
                ref = want
            if tol is not None:
                for p in range(len(ref)):
                    assert S.rel_err(got[p], ref[p]) < tol, p
            else:       # bf16: closer to the right window than to either neighbour, on the whole
                errs = np.array([S.rel_err(got[p], ref[p]) for p in range(len(ref))])
                assert np.median(errs) < BF16_TOL / 2
        finally:
            gpu.close()


def planted_key_model(window, n_heads=2):
    """One latent-attention layer in which the probe token's queries point at the needle token's latent.  Fewer tokens than the width:
    a vector g with g . h = 1 for the needle's mixer input and 0 for every other token's exists, and W_dkv + (big u) g^T gives the
    needle alone the latent direction u, the mean direction of the probe's queries carried into the latent.  Its score stands out
    among hundreds of random ones in every head (the shared rotated key part is scaled down for that)."""
    cfg = S.config([S.latent(heads=n_heads, dim=16, rot_dim=8, vdim=24, q_rank=32, kv_rank=32, window=window, scale=1.0)], width=48, vocab=40,
                   streams=None, mult=1.0, embed_scale=0.3)
    w = S.random_weights(cfg, 28)
    w["l0.mix.dkv.norm"] = np.ones_like(w["l0.mix.dkv.norm"])
    needle, probe = cfg["vocab"] - 2, cfg["vocab"] - 1
    W = S.f64(w)
    m = cfg["layers"][0]["mixer"]
    Hin = np.stack([O.layer_norm(W["embed"][t] * cfg["embedding"]["scale"], W["l0.norm1"], cfg["norm"]["eps"]) for t in range(cfg["vocab"])])
    g = np.linalg.pinv(Hin)[:, needle]
    assert np.abs(Hin @ g - np.eye(cfg["vocab"])[needle]).max() < 1e-9
    cq = O.unit_rms(W["l0.mix.dq"] @ Hin[probe], cfg["norm"]["eps"]) * W["l0.mix.dq.norm"]
    q = (W["l0.mix.uq"] @ cq).reshape(m["heads"], m["dim"] + m["rot_dim"])
    uk = W["l0.mix.uk"].reshape(m["heads"], m["dim"], m["kv_rank"])
    qa = np.stack([uk[h].T @ q[h, :m["dim"]] for h in range(m["heads"])])
    u = (qa / np.linalg.norm(qa, axis=1, keepdims=True)).sum(axis=0)
    u /= np.linalg.norm(u)
    d = np.array(w["l0.mix.dkv"], dtype=np.float64)
    d[:m["kv_rank"]] += np.outer(60.0 * u, g)
    d[m["kv_rank"]:] *= 0.2                                     # (the rotated part stays in play but cannot outvote the planted score)
    w["l0.mix.dkv"] = d.astype(np.float32)
    return cfg, w, needle, probe


def test_far_key_among_hundreds(b200):
    # position 300 still sees position 8; the window (296) closes at position 304
    cfg, w, needle, probe = planted_key_model(296)
    n = 310
    toks = tokens(n, cfg["vocab"] - 2, 29)
    toks[8] = needle
    for p in range(296, n):
        toks[p] = probe
    ref = Ref(cfg, w)
    want = ref.forward(toks)
    toks2 = list(toks)
    toks2[8] = 0
    alt = ref.forward(toks2)
    for p in (299, 300, 303):        # the far key is really seen, in the prompt and in decoding
        assert S.rel_err(alt[p], want[p]) > 40 * F32_TOL, p
    assert S.rel_err(alt[304:], want[304:]) < 1e-9      # and has left the window of position 304
    for compute, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        gpu = S.gpu_model(cfg, w, compute, max_seq_len=n + 4)
        try:
            got = gpu.step([(0, toks[:300])], list(range(290, 300)))
            assert S.rel_err(got, want[290:300]) < tol
            for p in range(300, n):
                assert S.rel_err(gpu.forward(toks[p]), want[p]) < tol, p
        finally:
            gpu.close()


def test_far_state_of_the_recurrence(b200):
    # Slow decays and small steps: ordinary tokens write next to nothing into the matrix state, the needle token (its step size is
    # planted through a vector that picks its mixer input among all tokens') writes a lot.  What position 8 wrote shapes the answers
    # 300 tokens later, through a prompt cut in two and through decoding.
    cfg = S.config([S.scan(heads=2, vdim=16, state=16, groups=1, conv=3, norm_groups=1)], width=32, vocab=24, streams=None, mult=1.0,
                   embed_scale=0.1)
    w = S.random_weights(cfg, 30)
    w["l0.mix.A_log"] = np.full_like(w["l0.mix.A_log"], -6.0)
    w["l0.mix.dt_bias"] = np.full_like(w["l0.mix.dt_bias"], -6.0)
    needle = cfg["vocab"] - 1
    W = S.f64(w)
    Hin = np.stack([O.layer_norm(W["embed"][t] * cfg["embedding"]["scale"], W["l0.norm1"], cfg["norm"]["eps"]) for t in range(cfg["vocab"])])
    g = np.linalg.pinv(Hin)[:, needle]
    win = np.array(w["l0.mix.in"], dtype=np.float64)
    win[-2:] += np.outer(np.full(2, 10.0), g)                  # the last `heads` rows are the step sizes
    w["l0.mix.in"] = win.astype(np.float32)
    n = 310
    toks = tokens(n, cfg["vocab"] - 1, 31)
    toks[8] = needle
    ref = Ref(cfg, w)
    want = ref.forward(toks)
    toks2 = list(toks)
    toks2[8] = 0
    alt = ref.forward(toks2)
    assert min(S.rel_err(alt[p], want[p]) for p in range(290, n)) > 40 * F32_TOL
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        gpu.step([(0, toks[:150])])
        got = gpu.step([(0, toks[150:300])], list(range(140, 150)))
        assert S.rel_err(got, want[290:300]) < F32_TOL
        for p in range(300, n):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()


def test_first_tokens_and_long_decoding(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 32)
    toks = tokens(120, cfg["vocab"], 33)      # many windows decoded one by one, from the very first token
    want = Ref(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        got = np.stack([gpu.forward(t) for t in toks])
        for p in range(len(toks)):
            assert S.rel_err(got[p], want[p]) < F32_TOL, p
    finally:
        gpu.close()


def test_rotation_at_large_positions(b200):
    # a small base makes every pair turn many times; positions beyond 1500 in a prompt and decoded
    cfg = S.config([S.latent(heads=2, dim=8, rot_dim=16, vdim=16, window=40, base=4.0, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0})],
                   width=32, vocab=40, streams=None)
    w = S.random_weights(cfg, 34)
    n = 1560
    toks = tokens(n, cfg["vocab"], 35)
    want = Ref(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        got = gpu.step([(0, toks[:1550])], list(range(1500, 1550)))
        assert S.rel_err(got, want[1500:1550]) < F32_TOL
        for p in range(1550, n):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- generation through the scheduler
def test_greedy_generation_through_the_batched_engine(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 36)
    prompts = [tokens(n, cfg["vocab"], 50 + n) for n in (5, 17, 9, 26, 3)]
    n_new = [6, 4, 8, 5, 7]
    want = [O.greedy(cfg, S.f64(w), p, k) for p, k in zip(prompts, n_new)]
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
    w = S.random_weights(cfg, 37)
    p = tokens(12, cfg["vocab"], 38)
    want = O.greedy(cfg, S.f64(w), p, 6)
    gpu = S.gpu_model(cfg, w)
    try:
        first = gpu.step([(0, p)], [len(p) - 1])[0]
        t0 = int(len(first) - 1 - np.argmax(first[::-1]))
        assert t0 == want[0]
        out, _ = gpu.decode_greedy(t0, 5)
        assert out.tolist() == want[1:]
    finally:
        gpu.close()


def test_bad_arguments(b200):
    from llama_gguf_b200 import madudra

    cfg = full_cfg()
    bad = copy.deepcopy(cfg)
    bad["layers"][3]["mixer"]["kv_from"] = 1                    # a state-space layer has no rows to lend
    w = S.random_weights(cfg, 39)
    with pytest.raises(b200.InvalidArgument):
        S.gpu_model(bad, w)
    bad = copy.deepcopy(cfg)
    bad["layers"][1]["mixer"]["groups"] = 3                     # 4 heads do not split into 3 groups
    with pytest.raises(b200.InvalidArgument):
        b200.LayerProgramInference(*madudra.parse_config(bad, 64, 2, "float32"), {})
    short = dict(w)
    del short["l3.mix.uk"]
    with pytest.raises(b200.InvalidArgument):
        S.gpu_model(cfg, short)
    with pytest.raises(b200.Unsupported):
        madudra.parse_config(dict(cfg, layers=[{"type": "attention", "mixer": {}}]), 64, 2)


# ---------------------------------------------------------------------------------------------------- kernels against their plain forms
@pytest.mark.parametrize("sizes", [(16, 16, 32), (48, 16, 24), (96, 32, 64), (64, 8, 40)])
def test_tile_attention_against_warp_attention(b200, monkeypatch, sizes):
    # bf16 prompts of 16 rows and more take the tensor-pipe tile kernel when the cached row is a multiple of 16 wide (third case: it is
    # not, both runs take the warp kernel); B200_LP_ATTN_TILE=0 keeps the warp kernel
    kv_rank, rot_dim, window = sizes
    cfg = S.config([S.latent(heads=3, dim=16, rot_dim=rot_dim, vdim=24, q_rank=32, kv_rank=kv_rank, window=window)], width=64, vocab=64, streams=2)
    w = S.random_weights(cfg, 40)
    a, b = tokens(150, cfg["vocab"], 41), tokens(70, cfg["vocab"], 42)
    want = Ref(cfg, w).forward(a)
    out = {}
    for tile in ("1", "0"):
        monkeypatch.setenv("B200_LP_ATTN_TILE", tile)
        gpu = S.gpu_model(cfg, w, "bfloat16")
        try:
            gpu.step([(0, a[:37])])
            out[tile] = gpu.step([(1, b), (0, a[37:])], list(range(len(b), len(b) + len(a) - 37)))
        finally:
            gpu.close()
    assert S.rel_err(out["1"], want[37:]) < BF16_TOL
    assert S.rel_err(out["1"], out["0"]) < 2e-2


def test_tensor_core_gemm_path(b200, monkeypatch):
    # bf16 steps of 17 rows and more multiply on the tensor cores, the per-head products and the experts' grouped products included
    cfg = full_cfg()
    w = S.random_weights(cfg, 43)
    toks = tokens(200, cfg["vocab"], 44)
    want = Ref(cfg, w).forward(toks)
    out = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("B200_LP_TC", tc)
        gpu = S.gpu_model(cfg, w, "bfloat16")
        try:
            out[tc] = gpu.step([(0, toks)], list(range(len(toks))))
        finally:
            gpu.close()
    d = np.array([S.rel_err(out["1"][i], out["0"][i]) for i in range(len(toks))])
    assert np.median(d) < 2e-2 and (d < 4e-2).mean() > 0.9
    e = np.array([S.rel_err(out["1"][i], want[i]) for i in range(len(toks))])
    assert np.median(e) < BF16_TOL / 2


def test_decode_kernels_for_few_rows_against_the_many_row_path(b200, monkeypatch):
    # decoding reads only the chosen experts' weights; B200_LP_FUSE=0 sends the same rows through the products over all experts
    cfg = full_cfg()
    w = S.random_weights(cfg, 45)
    ref = Ref(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 60 + n) for n in (3, 19, 1)]
    tails = [tokens(12, cfg["vocab"], 70 + i) for i in range(3)]
    states = [ref.new() for _ in prompts]
    for st, pr in zip(states, prompts):
        ref.step(st, pr)
    want = [[ref.step(states[i], [tails[i][k]])[0] for i in range(3)] for k in range(12)]
    for fuse in ("1", "0"):
        monkeypatch.setenv("B200_LP_FUSE", fuse)
        gpu = S.gpu_model(cfg, w, "float32")
        try:
            gpu.step([(i, pr) for i, pr in enumerate(prompts)])
            for k in range(12):
                lg = gpu.decode_batch([0, 1, 2], [tails[i][k] for i in range(3)])
                for i in range(3):
                    assert S.rel_err(lg[i], want[k][i]) < F32_TOL, (fuse, k, i)
        finally:
            gpu.close()


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
    ref = Ref(cfg, w)
    wa, wb = ref.forward(a), ref.forward(b)
    got = {i: np.fromfile(str(out / ("%d.f32" % i)), dtype="<f4").reshape(-1, cfg["vocab"]) for i in range(4)}
    assert S.rel_err(got[0], np.stack([wa[0], wa[14], wb[4]])) < F32_TOL
    assert S.rel_err(got[1], wb[5:6]) < F32_TOL
    assert S.rel_err(got[2], np.stack([wa[16], wb[6]])) < F32_TOL
    assert S.rel_err(got[3], wa[18:19]) < F32_TOL

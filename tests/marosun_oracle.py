"""A plain, slow restatement of the Marosun design in float64: one function per mechanism, one token at a time, state kept in Python
lists and numpy arrays.  It shares no code with the library.

Notation.  x_t is the residual stream of token t (position t, counted from 0 in its sequence).  A layer has ONE norm and both of
its sublayers read it:
    h = N(x),   x <- x + mixer(h) + ff(h),   N(u) = u / sqrt(mean(u^2) + eps) * (1 + w).
Softmax branch (all three mixers have one): q, k, v = W h (+ b); optionally each head of q and k divided by its root mean square
and multiplied by a weight of the head's size; optionally the pairs (2i, 2i + 1) of the first `dims` channels of every head of q
and k turned by t * f_i; score(t, s) = scale q_t . k_s over the visible s; the softmax's denominator holds one more term exp(c)
that belongs to no key (c learned per head, or c = 0).  Query head n reads key / value head n // (H / G).
  "attention"   biases (also on the output), norm, rotation with stretched frequencies, every s <= t visible, learned c, and the
                VALUES carry positions too: v_s is turned by s (all of its pairs, plain frequencies of its own size) before it is
                stored, and the weighted sum of head n at t is turned back by -t.
  "parallel"    left: no biases, no norm, no rotation, s visible when s <= t and s // size == t // size, learned c, the heads' outputs
                times sigmoid(W_g h) per channel; right: a gated linear memory per head, S <- diag(f) S + (1 - f) v^T, o = S^T q with
                q = silu(W_q h), f = l + (1 - l) sigmoid(W_f h + b) (l a stored lower bound per channel), o divided by its root mean
                square per head times a weight; the mixer is a_left W_o,left(left) + a_right W_o,right(right).
  "parallel_2"  left: biases, norm, rotation (keys and queries only), every s <= t, c = 0; right: a gated unit per channel,
                s <- (1 - z) s + z c~ with z = sigmoid(W_z h + b), u = W_x h + b, c~ = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), output
                W_o (s * silu(W_g h)); the mixer is (N'(left) + N'(right)) / 2 with N'(u) = u / rms(u) * w (plain weights).
Feed-forward: dense  W_down (g sigmoid(1.702 g) (u + 1)), g = min(W_gate h, limit), u = clamp(W_up h, +-limit);
mixture: scores sigmoid(W_router h), the `top` largest chosen, output sum_e expert_e(score_e h), expert = W_down (silu(W_gate .) * W_up .)."""
import math

import numpy as np

GATE_SLOPE = 1.702      # the dense layer's gate is g * sigmoid(1.702 g)
YARN_GAIN = 0.1         # cos and sin of stretched frequencies are multiplied by 0.1 ln(factor) + 1


# ------------------------------------------------------------------------------------------------ small pieces
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(u, eps):
    return u / math.sqrt(float(np.mean(u * u)) + eps)


def offset_norm(u, w, eps):
    return unit_rms(u, eps) * (1.0 + w)


def plain_norm(u, w, eps):
    return unit_rms(u, eps) * w


def pair_frequencies(dims, base):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def stretched_frequencies(dims, base, scaling):
    """(frequencies of the dims / 2 pairs, factor on cos and sin).  scaling = None: the plain ones."""
    f = pair_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_to_dim(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, YARN_GAIN * math.log(factor) + 1.0


def turn_pairs(vec, pos, freqs, gain=1.0):
    """pairs (2i, 2i + 1), i < len(freqs), of vec turned by pos * freqs[i]; the rest passes."""
    out = vec.copy()
    for i, f in enumerate(freqs):
        c, s = math.cos(pos * f) * gain, math.sin(pos * f) * gain
        a, b = vec[2 * i], vec[2 * i + 1]
        out[2 * i] = a * c - b * s
        out[2 * i + 1] = b * c + a * s
    return out


def sees_all(t, s):
    return s <= t


def sees_chunk(t, s, size):
    return s <= t and t // size == s // size


def softmax_with_extra(scores, extra):
    """weights of the scores when the denominator also holds exp(extra)"""
    m = max(max(scores), extra)
    e = np.exp(np.asarray(scores) - m)
    return e / (e.sum() + math.exp(extra - m))


def softmax_branch(o, w, pre, h, t, cache, eps, kind):
    """One token of a softmax branch.  o: its sizes and constants (config), w: weights, pre: prefix of its tensors, cache: list of
    (k, v) of the earlier tokens, appended to.  kind: "attention" | "parallel" | "parallel_2"."""
    H, G, D, V = o["heads"], o["kv_heads"], o["dim"], o["vdim"]
    biased = kind != "parallel"
    q, k, v = w[pre + "q"] @ h, w[pre + "k"] @ h, w[pre + "v"] @ h
    if biased:
        q, k, v = q + w[pre + "q.b"], k + w[pre + "k.b"], v + w[pre + "v.b"]
    q, k, v = q.reshape(H, D).copy(), k.reshape(G, D).copy(), v.reshape(G, V).copy()
    if biased:
        for n in range(H):
            q[n] = plain_norm(q[n], w[pre + "q.norm"], eps)
        for g in range(G):
            k[g] = plain_norm(k[g], w[pre + "k.norm"], eps)
    rot = o.get("rot")
    if rot and kind != "parallel":
        fr, gain = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        for n in range(H):
            q[n] = turn_pairs(q[n], t, fr, gain)
        for g in range(G):
            k[g] = turn_pairs(k[g], t, fr, gain)
    turned_values = kind == "attention"
    if turned_values:
        fv = pair_frequencies(V, rot["base"])
        for g in range(G):
            v[g] = turn_pairs(v[g], t, fv)
    cache.append((k, v))
    size = o["mask"]["size"] if kind == "parallel" else None
    vis = [s for s in range(t + 1) if (sees_chunk(t, s, size) if size else sees_all(t, s))]
    out = np.zeros((H, V))
    for n in range(H):
        g = n // (H // G)
        scores = [o["scale"] * float(q[n] @ cache[s][0][g]) for s in vis]
        extra = 0.0 if kind == "parallel_2" else float(w[pre + "sink"][n])
        p = softmax_with_extra(scores, extra)
        for a, s in zip(p, vis):
            out[n] += a * cache[s][1][g]
        if turned_values:
            out[n] = turn_pairs(out[n], -t, fv)
    out = out.reshape(-1)
    if kind == "parallel":
        out = out * sigmoid(w[pre + "g"] @ h)
    y = w[pre + "o"] @ out
    if biased:
        y = y + w[pre + "o.b"]
    return y


def forget_gate(z, lower):
    return lower + (1.0 - lower) * sigmoid(z)


def gated_memory_step(S, q, f, v):
    """S [dim, vdim] <- diag(f) S + (1 - f) v^T; returns (S, S^T q)"""
    S = f[:, None] * S + (1.0 - f)[:, None] * v[None, :]
    return S, S.T @ q


def gated_memory_branch(o, w, pre, h, state, eps):
    H, D, V = o["heads"], o["dim"], o["vdim"]
    q = silu(w[pre + "q"] @ h).reshape(H, D)
    v = (w[pre + "v"] @ h).reshape(H, V)
    f = forget_gate(w[pre + "f"] @ h + w[pre + "f.b"], w[pre + "lower"]).reshape(H, D)
    if "S" not in state:
        state["S"] = np.zeros((H, D, V))
    out = np.zeros((H, V))
    for n in range(H):
        state["S"][n], r = gated_memory_step(state["S"][n], q[n], f[n], v[n])
        out[n] = plain_norm(r, w[pre + "norm"], eps)
    return w[pre + "o"] @ out.reshape(-1)


def unit_candidate(u):
    return np.where(u >= 0, u + 0.5, sigmoid(u))


def gated_unit_step(s, z, u):
    return (1.0 - z) * s + z * unit_candidate(u)


def gated_unit_branch(o, w, pre, h, state):
    z = sigmoid(w[pre + "z"] @ h + w[pre + "z.b"])
    u = w[pre + "x"] @ h + w[pre + "x.b"]
    if "s" not in state:
        state["s"] = np.zeros(o["width"])
    state["s"] = gated_unit_step(state["s"], z, u)
    return w[pre + "o"] @ (state["s"] * silu(w[pre + "g"] @ h))


def dense_ff(h, gate, up, down, limit):
    g = np.minimum(gate @ h, limit)
    u = np.clip(up @ h, -limit, limit)
    return down @ (g * sigmoid(GATE_SLOPE * g) * (u + 1.0))


def expert(h, gate, up, down):
    return down @ (silu(gate @ h) * (up @ h))


def route(scores, top):
    """indices of the `top` largest scores (the lower index first among equals), in the order they are taken"""
    order = sorted(range(len(scores)), key=lambda e: (-scores[e], e))
    return order[:top]


def mixture_ff(h, w, pre, experts, top):
    s = sigmoid(w[pre + "router"] @ h)
    y = 0.0
    for e in route(list(s), top):
        y = y + expert(s[e] * h, w[pre + "e%d.gate" % e], w[pre + "e%d.up" % e], w[pre + "e%d.down" % e])
    return y


# ------------------------------------------------------------------------------------------------ the model
class Model:
    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.eps = float(cfg["norm"]["eps"])

    def new_state(self):
        return {"n": 0, "layers": [{"cache": [], "right": {}} for _ in self.cfg["layers"]]}

    def mixer(self, i, L, h, t, st):
        pre, m, kind = "l%d.mix." % i, L["mixer"], L["type"]
        if kind == "attention":
            return softmax_branch(m, self.w, pre, h, t, st["cache"], self.eps, kind)
        left = softmax_branch(m["left"], self.w, pre + "left.", h, t, st["cache"], self.eps, kind)
        if kind == "parallel":
            right = gated_memory_branch(m["right"], self.w, pre + "right.", h, st["right"], self.eps)
            return m["left_scale"] * left + m["right_scale"] * right
        if kind == "parallel_2":
            right = gated_unit_branch(m["right"], self.w, pre + "right.", h, st["right"])
            return 0.5 * (plain_norm(left, self.w[pre + "left.out"], self.eps) + plain_norm(right, self.w[pre + "right.out"], self.eps))
        raise ValueError(kind)

    def ff(self, i, L, h):
        mlp, pre = L.get("mlp"), "l%d.mlp." % i
        if mlp is None:
            return 0.0
        if mlp["kind"] == "dense":
            return dense_ff(h, self.w[pre + "gate"], self.w[pre + "up"], self.w[pre + "down"], float(mlp["limit"]))
        return mixture_ff(h, self.w, pre, mlp["router"]["experts"], mlp["router"]["top"])

    def token(self, tok, state, taps=None):
        t = state["n"]
        x = self.w["embed"][tok].copy()
        for i, L in enumerate(self.cfg["layers"]):
            h = offset_norm(x, self.w["l%d.norm1" % i], self.eps)
            x = x + (self.mixer(i, L, h, t, state["layers"][i]) + self.ff(i, L, h))
            if taps is not None:
                taps[i].append(x.copy())
        state["n"] = t + 1
        return self.w["head"] @ offset_norm(x, self.w["final.norm"], self.eps)

    def step(self, state, tokens, taps_out=None):
        """the next tokens of the sequence that `state` holds -> logits [len(tokens), vocab]; taps_out (a list) receives the residual
        stream after every layer, [layers][tokens, width]"""
        taps = [[] for _ in self.cfg["layers"]] if taps_out is not None else None
        out = [self.token(tok, state, taps) for tok in tokens]
        if taps_out is not None:
            taps_out.extend(np.stack(a) for a in taps)
        return np.stack(out)

    def forward(self, tokens, taps_out=None):
        return self.step(self.new_state(), tokens, taps_out)

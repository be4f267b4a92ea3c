"""A plain float64 restatement of the Madudra design, one function per mechanism, one token at a time.  It shares nothing with the
library: the tests compare the library's logits and residual streams with what these functions give.

Notation.  h: a sublayer's input vector; W[name]: a tensor of the model, linear maps stored [out, in] and applied as W @ h;
p: the token's position in its sequence, counted from 0."""
import math

import numpy as np


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w, the variance being the mean squared deviation; no bias."""
    d = x - x.mean()
    return d / math.sqrt((d * d).mean() + eps) * w


def unit_rms(x, eps):
    return x / math.sqrt((x * x).mean() + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_erf(z):
    return np.array([0.5 * v * (1.0 + math.erf(v / math.sqrt(2.0))) for v in np.atleast_1d(z)])


def rot_table(rot):
    """Frequencies of the pairs and the factor on cos / sin.  Without 'scaling': base^(-2i/dims) and 1.  With it, pairs whose
    wavelength is long against the original context are slowed down by `factor`, short ones are kept, with a linear ramp between."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v, p, freqs, mult):
    """Pairs (i, i + half) of the first 2 * len(freqs) entries of v turn by the angle p * freqs[i]; cos and sin carry `mult`."""
    half = len(freqs)
    out = np.array(v, dtype=np.float64)
    a = p * freqs
    c, s = np.cos(a) * mult, np.sin(a) * mult
    u, w = v[:half], v[half:2 * half]
    out[:half] = u * c - w * s
    out[half:2 * half] = w * c + u * s
    return out


class LatentCache:
    """What a latent-attention layer keeps per position: the normed latent and the rotated shared key part."""

    def __init__(self):
        self.c, self.kr = [], []


def latent_attention(h, p, W, pre, mx, eps, cache, own_kv):
    """One token.  `cache` is this layer's (own_kv) or the layer's it borrows from; a borrowing layer appends nothing."""
    H, dim, rd, vd, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    freqs, mult = rot_table(mx["rot"])
    cq = unit_rms(W[pre + "dq"] @ h, eps) * W[pre + "dq.norm"]
    q = (W[pre + "uq"] @ cq).reshape(H, dim + rd)
    if own_kv:
        d = W[pre + "dkv"] @ h
        cache.c.append(unit_rms(d[:rank], eps) * W[pre + "dkv.norm"])
        cache.kr.append(rotate(d[rank:], p, freqs, mult))
    assert len(cache.c) == p + 1
    first = max(0, p - mx["mask"]["size"] + 1)
    uk = W[pre + "uk"].reshape(H, dim, rank)
    uv = W[pre + "uv"].reshape(H, vd, rank)
    out = np.zeros((H, vd))
    for hd in range(H):
        qr = rotate(q[hd, dim:], p, freqs, mult)
        s = np.array([(q[hd, :dim] @ (uk[hd] @ cache.c[j]) + qr @ cache.kr[j]) * mx["scale"] for j in range(first, p + 1)])
        a = np.exp(s - s.max())
        a /= a.sum()
        for n, j in enumerate(range(first, p + 1)):
            out[hd] += a[n] * (uv[hd] @ cache.c[j])
    gated = out.reshape(-1) * sigmoid(W[pre + "g"] @ h)
    return W[pre + "o"] @ gated


class ScanState:
    """What a state-space layer keeps per sequence: the matrix state per head and the last inputs of the convolution."""

    def __init__(self, mx):
        inner = mx["heads"] * mx["vdim"]
        self.S = np.zeros((mx["heads"], mx["state"], mx["vdim"]))
        self.tail = np.zeros((mx["conv"] - 1, inner + 2 * mx["groups"] * mx["state"]))


def state_space(h, W, pre, mx, eps, st):
    """One token of the gated linear recurrence with input-dependent step size."""
    H, vd, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = H * vd
    y = W[pre + "in"] @ h
    z, xbc, dt = y[:inner], y[inner:2 * inner + 2 * G * N], y[2 * inner + 2 * G * N:]
    window = np.vstack([st.tail, xbc[None, :]])                      # [taps, channels], oldest first
    conv = (window * W[pre + "conv"].T).sum(axis=0) + W[pre + "conv.b"]
    st.tail = window[1:]
    conv = silu(conv)
    x = conv[:inner].reshape(H, vd)
    Bm = conv[inner:inner + G * N].reshape(G, N)
    Cm = conv[inner + G * N:].reshape(G, N)
    dt = softplus(dt + W[pre + "dt_bias"])
    out = np.zeros((H, vd))
    for hd in range(H):
        g = hd // (H // G)
        st.S[hd] = math.exp(-math.exp(W[pre + "A_log"][hd]) * dt[hd]) * st.S[hd] + dt[hd] * np.outer(Bm[g], x[hd])
        out[hd] = st.S[hd].T @ Cm[g] + W[pre + "D"][hd] * x[hd]
    gated = out.reshape(-1) * silu(z)
    parts = gated.reshape(mx["norm_groups"], -1)
    normed = np.concatenate([unit_rms(part, eps) for part in parts]) * W[pre + "norm"]
    return W[pre + "o"] @ normed


def expert_mixture(h, W, pre, mlp):
    """Softmax over all experts, the `top` largest taken, their probabilities times router.scale (no renormalisation)."""
    r = mlp["router"]
    z = W[pre + "router"] @ h
    s = np.exp(z - z.max())
    s /= s.sum()
    order = sorted(range(r["experts"]), key=lambda e: (-s[e], e))[:r["top"]]
    out = np.zeros(W[pre + "e0.down"].shape[0])
    for e in order:
        out += s[e] * r["scale"] * (W[pre + "e%d.down" % e] @ gelu_erf(W[pre + "e%d.up" % e] @ h))
    return out


def streams_in(X, W, pre):
    """The sublayer's input: the streams weighted by '.in' (one stream without such a tensor: itself)."""
    return X[0] if pre + "in" not in W else np.tensordot(W[pre + "in"], X, axes=1)


def streams_out(X, y, W, pre, mult):
    """All streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + mult * out[t] * y."""
    if pre + "in" not in W:
        return X + mult * y
    return W[pre + "mix"].T @ X + mult * np.outer(W[pre + "out"], y)


class Sequence:
    """One sequence fed token by token."""

    def __init__(self, cfg, W):
        self.cfg, self.W, self.p = cfg, W, 0
        self.state = []
        for L in cfg["layers"]:
            if L["type"] == "latent_attention":
                self.state.append(LatentCache())
            elif L["type"] == "mamba2":
                self.state.append(ScanState(L["mixer"]))
            else:
                raise ValueError(L["type"])

    def token(self, tok):
        """-> (logits [vocab], the sum of the streams after every layer [layers, width])"""
        cfg, W = self.cfg, self.W
        eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
        n_streams = int(cfg.get("streams", 1))
        x0 = W["embed"][tok] * cfg["embedding"]["scale"]
        X = np.tile(x0, (n_streams, 1))
        taps = []
        for i, L in enumerate(cfg["layers"]):
            pre = "l%d." % i
            h = layer_norm(streams_in(X, W, pre + "hc1."), W[pre + "norm1"], eps)
            if L["type"] == "latent_attention":
                src = L["mixer"].get("kv_from")
                own = src is None
                y = latent_attention(h, self.p, W, pre + "mix.", L["mixer"], eps, self.state[i if own else src], own)
            else:
                y = state_space(h, W, pre + "mix.", L["mixer"], eps, self.state[i])
            X = streams_out(X, y, W, pre + "hc1.", mult)
            if L.get("mlp") is not None:
                h = layer_norm(streams_in(X, W, pre + "hc2."), W[pre + "norm2"], eps)
                X = streams_out(X, expert_mixture(h, W, pre + "mlp.", L["mlp"]), W, pre + "hc2.", mult)
            taps.append(X.sum(axis=0))
        self.p += 1
        return W["head"] @ layer_norm(X.sum(axis=0), W["final.norm"], eps), np.array(taps)


def run(cfg, W, tokens):
    """-> logits [n, vocab], taps [layers, n, width]"""
    s = Sequence(cfg, W)
    out = [s.token(t) for t in tokens]
    return np.array([o[0] for o in out]), np.stack([o[1] for o in out], axis=1)


def greedy(cfg, W, prompt, n):
    """The prompt, then n tokens each the last largest logit (the library's tie rule)."""
    s = Sequence(cfg, W)
    for t in prompt:
        logits, _ = s.token(t)
    out = []
    for _ in range(n):
        v = logits.max()
        t = int(np.nonzero(logits == v)[0][-1])
        out.append(t)
        logits, _ = s.token(t)
    return out

"""Nalizen, written out plainly: float64 numpy, one token at a time, one function per mechanism.

Shares no code with the package.  A model is a dict `cfg` (the nested form of its config.json) and a dict of
float64 arrays by tensor name; `Plain(cfg, tensors)` keeps one sequence's state and `step(token)` returns the
logits of the next position.

Notation: d width, H heads, G key/value heads, dk key size, dv value size, eps the norm's epsilon.
  layer            x <- x + LN1(mixer(shift(x)));  x <- x + LN2(ff(x));  x <- x + side(x, token)
  LN(y)            (y - mean) / sqrt(var + eps) * w + b
  shift(x)_t       x_t + (x_(t-1) - x_t) * s      (x_(-1) = 0; the unshifted x_t is what the next token sees)
  attention        q, k rotated on their first r elements (i with i + r/2), then each head over its root mean square;
                   keys j with 0 <= t - j < window; softmax((q . k) scale); heads side by side times sigmoid(W_g h); W_o
  hgrn2            q = silu(W_q h); f = l + (1 - l) sigmoid(W_f h + b); S <- diag(f) S + (1 - f) v^T; o = S^T q;
                   o over its root mean square per head, times a weight; W_o
  dense ff         W_down (gelu_tanh(W_gate x) * (W_up x))
  routed ff        z = W_r x + b; the `top` largest z; softmax over those; sum of weight * W_down relu(W_up x)^2
  side             e = table[token, slice]; y = W_proj (gelu_tanh(W_gate x) * e); y / rms(y) * w
"""
import math

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def layer_norm(y, w, b, eps):
    m = y.mean(-1, keepdims=True)
    v = ((y - m) ** 2).mean(-1, keepdims=True)
    return (y - m) / np.sqrt(v + eps) * w + b


def unit_rms(y, eps):
    return y / np.sqrt((y ** 2).mean(-1, keepdims=True) + eps)


def token_shift(x, prev, s):
    return x + (prev - x) * s


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with scaling {factor, low, high, original}: long wavelengths (above
    original/low) are divided by factor, short ones (below original/high) kept, the ones between blended."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    if not scaling:
        return f
    fac, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        wl = 2.0 * math.pi / fi
        if wl < orig / high:
            out[i] = fi
        elif wl > orig / low:
            out[i] = fi / fac
        else:
            s = (orig / wl - low) / (high - low)
            out[i] = (1.0 - s) * fi / fac + s * fi
    return out


def rotate(x, pos, freqs):
    """x [heads, size]: the first 2 len(freqs) elements of each head are rotated, element i with i + len(freqs).  Positions,
    frequencies and their product are float32 numbers (the design computes angles in 32-bit); the rest is float64."""
    n = len(freqs)
    if n == 0:
        return x
    a = (np.float32(pos) * np.asarray(freqs, dtype=np.float32)).astype(np.float64)      # the angle is a float32 product
    c, s = np.cos(a), np.sin(a)
    out = x.copy()
    u, v = x[:, :n], x[:, n:2 * n]
    out[:, :n] = u * c - v * s
    out[:, n:2 * n] = v * c + u * s
    return out


def attend(q, keys, values, pos, window, scale, group):
    """q [H, dk]; keys [t+1][G, dk]; values [t+1][G, dv]: position pos sees j with 0 <= pos - j < window."""
    first = 0 if window is None else max(0, pos - window + 1)
    K = np.stack(keys[first:pos + 1], 0)          # [n, G, dk]
    V = np.stack(values[first:pos + 1], 0)
    out = []
    for h in range(q.shape[0]):
        g = h // group
        s = (K[:, g, :] @ q[h]) * scale
        w = np.exp(s - s.max())
        w /= w.sum()
        out.append(w @ V[:, g, :])
    return np.stack(out, 0)


def hgrn2_step(S, q, f, v):
    """S [H, dk, dv]; q, f [H, dk]; v [H, dv] -> (new S, o [H, dv])."""
    S = f[:, :, None] * S + (1.0 - f)[:, :, None] * v[:, None, :]
    return S, np.einsum("hkv,hk->hv", S, q)


def dense_ff(x, gate, up, down):
    return down @ (gelu_tanh(gate @ x) * (up @ x))


def routed_ff(x, router, router_b, ups, downs, top):
    z = router @ x + router_b
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    w = np.exp(z[order] - z[order].max())
    w /= w.sum()
    out = np.zeros_like(x)
    for e, we in zip(order, w):
        out += we * (downs[e] @ np.maximum(ups[e] @ x, 0.0) ** 2)
    return out


def side_input(x, e, gate, proj, w, eps):
    y = proj @ (gelu_tanh(gate @ x) * e)
    return unit_rms(y, eps) * w


class Plain:
    """One sequence through a model; every call of step() is the next position."""

    def __init__(self, cfg, tensors):
        self.cfg = cfg
        self.t = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = float(cfg["norm"]["eps"])
        self.layers = cfg["layers"]
        self.pos = 0
        d = int(cfg["width"])
        self.prev = [np.zeros(d) for _ in self.layers]
        self.keys = [[] for _ in self.layers]
        self.values = [[] for _ in self.layers]
        self.S = [None] * len(self.layers)
        self.freqs = []
        for L in self.layers:
            m = L["mixer"]
            rot = m.get("rot") if L["type"] == "attention" else None
            self.freqs.append(np.zeros(0) if not rot else
                              rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling")))
            if L["type"] == "hgrn2":
                self.S[len(self.freqs) - 1] = np.zeros((int(m["heads"]), int(m["dim"]), int(m["vdim"])))

    def _attention(self, i, h):
        t, m, p = self.t, self.layers[i]["mixer"], f"l{i}.mix."
        H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        G = int(m.get("kv_heads", H))
        src = m.get("kv_from")
        q = unit_rms(rotate((t[p + "q"] @ h).reshape(H, dk), self.pos, self.freqs[i]), self.eps)
        if src is None:
            k = unit_rms(rotate((t[p + "k"] @ h).reshape(G, dk), self.pos, self.freqs[i]), self.eps)
            self.keys[i].append(k)
            self.values[i].append((t[p + "v"] @ h).reshape(G, dv))
            src = i
        window = m["mask"]["size"] if m.get("mask") else None
        a = attend(q, self.keys[src], self.values[src], self.pos, window, float(m["scale"]), H // G)
        return t[p + "o"] @ (a.reshape(-1) * sigmoid(t[p + "g"] @ h))

    def _hgrn2(self, i, h):
        t, m, p = self.t, self.layers[i]["mixer"], f"l{i}.mix."
        H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        q = silu(t[p + "q"] @ h).reshape(H, dk)
        low = t[p + "lower"]
        f = (low + (1.0 - low) * sigmoid(t[p + "f"] @ h + t[p + "f.b"])).reshape(H, dk)
        v = (t[p + "v"] @ h).reshape(H, dv)
        self.S[i], o = hgrn2_step(self.S[i], q, f, v)
        o = unit_rms(o, self.eps) * t[p + "norm"]
        return t[p + "o"] @ o.reshape(-1)

    def _ff(self, i, x):
        t, f, p = self.t, self.layers[i]["mlp"], f"l{i}.mlp."
        if f["kind"] == "dense":
            return dense_ff(x, t[p + "gate"], t[p + "up"], t[p + "down"])
        E, top = int(f["router"]["experts"]), int(f["router"]["top"])
        return routed_ff(x, t[p + "router"], t[p + "router.b"], [t[f"{p}e{e}.up"] for e in range(E)],
                         [t[f"{p}e{e}.down"] for e in range(E)], top)

    def step(self, token, streams=None):
        t, cfg = self.t, self.cfg
        x = t["embed"][token] * float(cfg.get("embedding", {}).get("scale", 1.0))
        side = int((cfg.get("token_side") or {}).get("dim", 0))
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            h = token_shift(x, self.prev[i], t[p + "shift"])
            self.prev[i] = x.copy()
            y = self._attention(i, h) if L["type"] == "attention" else self._hgrn2(i, h)
            x = x + layer_norm(y, t[p + "norm1"], t[p + "norm1.b"], self.eps)
            if L.get("mlp") is not None:
                x = x + layer_norm(self._ff(i, x), t[p + "norm2"], t[p + "norm2.b"], self.eps)
            if side:
                e = t["side.embed"][token, i * side:(i + 1) * side]
                x = x + side_input(x, e, t[p + "side.gate"], t[p + "side.proj"], t[p + "side.norm"], self.eps)
            if streams is not None:
                streams.append(x.copy())
        self.pos += 1
        xf = layer_norm(x, t["final.norm"], t["final.norm.b"], self.eps)
        return t["embed"] @ xf


def run(cfg, tensors, tokens):
    """Logits [len(tokens), vocab] of a whole sequence."""
    m = Plain(cfg, tensors)
    return np.stack([m.step(int(tok)) for tok in tokens], 0)

"""A plain, slow implementation of the Meresun design in PyTorch on the CPU: one function per
mechanism, no cache, no batching, no kernels.  It shares no code with fellm_b200: the tests compare
the engine with it.

Notation: d model width, H heads, dn / dr the unrotated / rotated sizes of a head's query and key, dv the value
size, rq / rk the ranks of the query and key-value latents, T tokens, E experts.  Weights are a dict
{tensor name: tensor}; everything is computed in the dtype of the weights handed in (float64 for the oracle).
`cfg` is the parsed config.json of the model.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def grouped_rms_norm(x, w, eps, groups):
    """The last axis in `groups` equal consecutive parts, each over its own root mean square; then the weight."""
    T, d = x.shape
    return rms_unit(x.view(T, groups, d // groups), eps).reshape(T, d) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def scaled_frequencies(dims, base, scaling):
    """(frequency of every pair [dims/2], factor of cos and sin).  Without scaling: base^(-2i/dims) and 1.  With
    {factor, original, fast, slow}: pairs that turn more than `fast` times over `original` positions keep their
    frequency, pairs that turn fewer than `slow` times have it divided by `factor`, a linear ramp over the pair
    index between; cos and sin times 0.1 ln(factor) + 1."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, orig = scaling["factor"], scaling["original"]

    def pair_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(scaling["fast"])), 0)
    hi = min(math.ceil(pair_of(scaling["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, freqs, mag, first=0):
    """x [T, ..., dims]: element 2i paired with 2i+1, angle = position * freqs[i]; cos and sin times mag.
    Positions are first, first + 1, ..."""
    T = x.shape[0]
    a = (torch.arange(T, dtype=x.dtype) + first)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [len(freqs)]
    c, s = (torch.cos(a) * mag).view(shape), (torch.sin(a) * mag).view(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def sink_softmax_attention(q, k, v, scale, window, sink):
    """q [T, H, dq]; k [T, H, dq]; v [T, H, dv]; sink [H].  Position i reads j with 0 <= i - j < window (all j <= i
    without a window); the softmax's denominator also holds exp(sink_h), which has no value."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[i, h] = (e @ v[lo:i + 1, h]) / (e.sum() + torch.exp(sink[h] - m))
    return out


def latent_attention_mixer(h, W, p, m, eps):
    """Queries through a normed latent; one normed key-value latent and one rotated key part shared by the heads;
    per head the unrotated keys and the values are projections of the latent."""
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    cq = rms_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, dn + dr)
    kv = h @ W[p + "dkv"].T
    c = rms_norm(kv[:, :rk], W[p + "dkv.norm"], eps)
    rot = m.get("rot")
    kr = kv[:, rk:].view(T, 1, dr)
    qn, qr = q[..., :dn], q[..., dn:]
    if rot:
        freqs, mag = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        n = rot["dims"]
        qr = torch.cat([rotate_pairs(qr[..., :n], freqs, mag), qr[..., n:]], -1)
        kr = torch.cat([rotate_pairs(kr[..., :n], freqs, mag), kr[..., n:]], -1)
    kn = (c @ W[p + "uk"].T).view(T, H, dn)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    qq = torch.cat([qn, qr], -1)
    kk = torch.cat([kn, kr.expand(T, H, dr)], -1)
    window = m["mask"]["size"] if m.get("mask") else None
    o = sink_softmax_attention(qq, kk, v, m["scale"], window, W[p + "sink"])
    return o.reshape(T, H * dv) @ W[p + "o"].T


def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, N = over the root mean square of the row."""
    a, b, c, e = coef
    return a * rms_unit(z, eps) + b * rms_unit(z ** 2, eps) + c * rms_unit(z ** 3, eps) + e


def dense_ff(h, W, p, eps):
    return poly_norm(h @ W[p + "up"].T, W[p + "act"], eps) @ W[p + "down"].T


def clamped_glu_expert(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def route(z, correction, router):
    """z [T, E] router logits -> (experts [T, top], weights [T, top]).  Scores are sigmoids; the choice looks at
    score + correction, only inside the `keep` groups whose two best choice scores sum highest; the weights are the
    plain scores of the chosen over their sum."""
    s = torch.sigmoid(z)
    choice = s + correction
    T, E = z.shape
    groups = router.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = choice.view(T, n, E // n)
        gs = torch.topk(per, min(2, E // n), dim=-1).values.sum(-1)
        kept = torch.topk(gs, keep, dim=-1).indices
        allowed = torch.zeros(T, n, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        choice = torch.where(allowed[:, :, None].expand(T, n, E // n).reshape(T, E), choice,
                             torch.full_like(choice, -math.inf))
    chosen = torch.topk(choice, router["top"], dim=-1).indices
    w = torch.gather(s, 1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20)


def routed_experts(h, W, p, mlp):
    chosen, w = route(h @ W[p + "router"].T, W[p + "correction"], mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], w[t]):
            q = f"{p}e{int(e)}."
            out[t] = out[t] + wt * clamped_glu_expert(h[t:t + 1], W[q + "gate"], W[q + "up"], W[q + "down"],
                                                      mlp["expert"]["limit"])[0]
    return out


def feed_forward(h, W, p, mlp, eps):
    if mlp["kind"] == "dense":
        return dense_ff(h, W, p, eps)
    return routed_experts(h, W, p, mlp)


def token_side_input(x, tokens, W, p, i, dim, eps):
    """What the token itself adds after layer i: its part of the side table, gated by the stream, projected, normed."""
    e = W["side.embed"][torch.tensor(tokens)][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ W[p + "gate"].T) * e
    return rms_norm(g @ W[p + "proj"].T, W[p + "norm"], eps)


def layer_order(cfg):
    """[(layer, True where the entry opens a pass of the loop other than the first)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for t in range(times):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(tokens, W, cfg, layers_out=None):
    """tokens: list of ids of one sequence -> logits [T, vocab].  layers_out: a list that receives the residual
    stream after every layer run."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x = W["embed"][torch.tensor(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    x0 = x.clone()
    side = cfg.get("token_side")
    for i, reopens in layer_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if reopens:
            x = x + x0
        h = grouped_rms_norm(x, W[p + "norm1"], eps, groups)
        y = latent_attention_mixer(h, W, p + "mix.", L["mixer"], eps) * torch.sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        if L.get("mlp") is not None:
            y = y + feed_forward(h, W, p + "mlp.", L["mlp"], eps) * torch.sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
        x = x + y
        if side:
            x = x + token_side_input(x, tokens, W, p + "side.", i, side["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return grouped_rms_norm(x, W["final.norm"], eps, groups) @ W["head"].T

"""A plain restatement of the Vufasun design, one function per mechanism, whole sequences at a time (float64 unless a
dtype is given).  It shares no code with the package: the tests compare the framework's step function, cache / state
manager and kernels with it.

Checkpoint names: ``embed``, ``final.norm`` and per layer ``l<i>.norm1 / norm2``, ``l<i>.hc1.* / hc2.*`` (stream
weights), ``l<i>.mix.<name>``, ``l<i>.mlp.<name>``.  Linear weights are ``[out, in]``.
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot, dtype=F64):
    """``f_i = base ** (-2 i / dims)``, with the optional wavelength-dependent slowdown of long waves."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=dtype)
    f = torch.as_tensor(float(rot["base"]), dtype=dtype) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        wave = 2.0 * math.pi / f
        s = (orig / wave - low) / (high - low)
        mid = (1.0 - s) * f / factor + s * f
        f = torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, mid))
    return f


def rotate(x, pos, rot):
    """``x [T, heads, D]`` at positions ``pos [T]``: dimension ``i`` and ``i + dims/2`` of the first ``dims`` turn."""
    if not rot:
        return x
    dims = rot["dims"]
    half = dims // 2
    ang = pos.to(x.dtype).reshape(-1, 1) * frequencies(rot, x.dtype).reshape(1, -1)          # [T, half]
    c, s = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def causal_softmax_attention(q, k, v, scale, sink=None):
    """``q [T, H, D]``, ``k [T, G, D]``, ``v [T, G, Dv]`` -> ``[T, H, Dv]``.  ``sink [H]``: one more term
    ``exp(sink_h)`` in every denominator, with no key and no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[: t + 1, g] @ q[t, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[t, h] = (e / den) @ v[: t + 1, g]
    return out


def retention(q, k, v, decay):
    """``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head; ``q, k [T, H, D]``, ``v [T, H, Dv]``."""
    T, H, D = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(D, v.shape[-1], dtype=q.dtype)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def attention_mixer(h, w, m, eps, whole_norm=False):
    """Softmax attention of grouped heads with partial rotation; ``whole_norm``: q and k are RMS-normed over their whole
    projection (all heads at once) with a weight of that size, ahead of the rotation.  A ``sink`` tensor adds its term."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if whole_norm:
        q, k = rms(q, eps) * w["q.norm"], rms(k, eps) * w["k.norm"]
    pos = torch.arange(T)
    q, k = rotate(q.reshape(T, H, D), pos, m.get("rot")), rotate(k.reshape(T, G, D), pos, m.get("rot"))
    o = causal_softmax_attention(q, k, v.reshape(T, G, Dv), m["scale"], w.get("sink"))
    return o.reshape(T, H * Dv) @ w["o"].T


def retention_mixer(h, w, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((h @ w["q"].T).reshape(T, H, D), pos, m.get("rot"))
    k = rotate((h @ w["k"].T).reshape(T, H, D), pos, m.get("rot")) * D ** -0.5
    v = (h @ w["v"].T).reshape(T, H, Dv)
    o = retention(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = rms(o, eps).reshape(T, H * Dv) * silu(h @ w["g"].T)
    return o @ w["o"].T


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def parallel_mixer(h, w, m, eps):
    left = attention_mixer(h, sub(w, "left."), m["left"], eps, whole_norm=True)
    right = retention_mixer(h, sub(w, "right."), m["right"], eps)
    return 0.5 * (rms(left, eps) * w["left.out"] + rms(right, eps) * w["right.out"])


def glu(h, w, act):
    return (act(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def moe(h, w, m, margins=None):
    """Sigmoid scores, the ``top`` largest chosen, the score scales the chosen expert's INPUT; a shared expert on top.
    ``margins``: a list that receives, per token, the gap between the last chosen score and the first one left out."""
    E, top = m["router"]["experts"], m["router"]["top"]
    s = torch.sigmoid(h @ w["router"].T)                                    # [T, E]
    if margins is not None and top < E:
        ranked = s.sort(dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            out[t] += glu((s[t, e] * h[t]).unsqueeze(0), sub(w, f"e{e}."), silu)[0]
    if m.get("shared"):
        out = out + glu(h, sub(w, "shared."), silu)
    return out


def feed_forward(h, w, m, margins=None):
    return glu(h, w, gelu_tanh) if m["kind"] == "dense" else moe(h, w, m, margins)


def layer_runs(config):
    """The order in which layers run: the looped range ``times`` times in a row, then the rest."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(config, sd, tokens, dtype=F64, layer_outputs=None, margins=None):
    """Logits ``[T, vocab]`` of one sequence.  ``layer_outputs``: a list that receives the sum of the streams after
    every layer run; ``margins``: a list that receives the routers' per-token score gaps (see ``moe``)."""
    sd = {k: v.to(dtype) for k, v in sd.items() if v.is_floating_point()}
    eps = config["norm"]["eps"]
    S = int(config.get("streams") or 1)
    x0 = sd["embed"][torch.as_tensor(tokens)]
    xs = [x0.clone() for _ in range(S)]
    for i in layer_runs(config):
        L = config["layers"][i]
        w = sub(sd, f"l{i}.")
        for q in (1, 2):
            if q == 2 and not L.get("mlp"):
                continue
            hc = sub(w, f"hc{q}.")
            if not hc:                                     # no stream weights: the plain residual sum
                hc = {"in": torch.ones(1, dtype=dtype), "out": torch.ones(1, dtype=dtype), "mix": torch.ones(1, 1, dtype=dtype)}
            u = sum(hc["in"][s] * xs[s] for s in range(S))
            hn = rms(u, eps) * w[f"norm{q}"]
            if q == 1:
                mw = sub(w, "mix.")
                y = parallel_mixer(hn, mw, L["mixer"], eps) if L["type"] == "parallel" else attention_mixer(hn, mw, L["mixer"], eps)
            else:
                y = feed_forward(hn, sub(w, "mlp."), L["mlp"], margins)
            xs = [sum(hc["mix"][s, t] * xs[s] for s in range(S)) + hc["out"][t] * y for t in range(S)]
        if layer_outputs is not None:
            layer_outputs.append(sum(xs))
    x = rms(sum(xs), eps) * sd["final.norm"]
    return x @ sd["embed"].T


def random_weights(cfg, seed=0, dtype=torch.float32):
    """A checkpoint of the design with weights that keep activations of order one through the layers (values that are
    exact in bfloat16, so that a bfloat16 model holds the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    W, V, S = cfg["width"], cfg["vocab"], int(cfg.get("streams") or 1)

    def bf(t):
        return t.to(torch.bfloat16).to(dtype)

    def mat(o, i, s=None):
        return bf(torch.randn(o, i, generator=g) * (s if s is not None else i ** -0.5))

    def vec(n, mean=0.0, s=0.1):
        return bf(mean + torch.randn(n, generator=g) * s)

    def attention(p, m, sink, whole):
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        sd[p + "q"], sd[p + "k"], sd[p + "v"], sd[p + "o"] = mat(H * D, W, 1.5 * W ** -0.5), mat(G * D, W, 1.5 * W ** -0.5), mat(G * Dv, W), mat(W, H * Dv)
        if sink:
            sd[p + "sink"] = vec(H, 0.5, 1.0)
        if whole:
            sd[p + "q.norm"], sd[p + "k.norm"] = vec(H * D, 1.0, 0.3), vec(G * D, 1.0, 0.3)

    sd = {"embed": mat(V, W, 1.0), "final.norm": vec(W, 1.0)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for q in (1, 2) if L.get("mlp") else (1,):
            sd[p + f"norm{q}"] = vec(W, 1.0)
            if "streams" in cfg:
                sd[p + f"hc{q}.in"] = vec(S, 1.0 / S, 0.2)
                sd[p + f"hc{q}.out"] = vec(S, 0.8, 0.3)
                sd[p + f"hc{q}.mix"] = bf(torch.eye(S) * 0.9 + torch.randn(S, S, generator=g) * 0.15)
        if L["type"] == "attention":
            attention(p + "mix.", m, True, False)
        else:
            attention(p + "mix.left.", m["left"], False, True)
            r = m["right"]
            H, D, Dv = r["heads"], r["dim"], r["vdim"]
            sd[p + "mix.right.q"], sd[p + "mix.right.k"] = mat(H * D, W), mat(H * D, W)
            sd[p + "mix.right.v"], sd[p + "mix.right.g"] = mat(H * Dv, W), mat(H * Dv, W)
            sd[p + "mix.right.o"] = mat(W, H * Dv)
            sd[p + "mix.left.out"], sd[p + "mix.right.out"] = vec(W, 1.0, 0.2), vec(W, 1.0, 0.2)
        mlp = L.get("mlp")
        if not mlp:
            continue
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            sd[p + "mlp.gate"], sd[p + "mlp.up"], sd[p + "mlp.down"] = mat(F, W), mat(F, W), mat(W, F)
        else:
            F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            sd[p + "mlp.router"] = mat(E, W, 2.0 * W ** -0.5)
            names = [f"e{e}." for e in range(E)] + (["shared."] if mlp.get("shared") else [])
            for n in names:
                Fn = mlp["shared"]["ff"] if n == "shared." else F
                sd[p + "mlp." + n + "gate"], sd[p + "mlp." + n + "up"] = mat(Fn, W), mat(Fn, W)
                sd[p + "mlp." + n + "down"] = mat(W, Fn)
    return sd


def greedy(cfg, sd, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, sd, toks)[-1].argmax()))
    return toks[len(prompt):]


def close_calls(config, sd, tokens, gap=0.01):
    """Positions at which some router's last chosen score and the first one left out lie within ``gap``: rounding the
    router's input to 16 bits may legitimately choose the other expert there."""
    margins = []
    forward(config, sd, tokens, margins=margins)
    if not margins:
        return set()
    return set(torch.nonzero(torch.stack(margins).min(dim=0).values < gap).reshape(-1).tolist())

"""A plain float64 restatement of the Gogalix design, one function per mechanism, whole sequences at a time.  It shares
no code with the package: the tests compare the framework's step function, cache / state manager and kernels with it.

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1`` (one number), ``l<i>.ls1 / ls2``
(layer scale), ``l<i>.rg1 / rg2`` with ``.b`` (residual gates), ``l<i>.mix.<name>``, ``l<i>.mlp.<name>``.  Linear weights
are ``[out, in]``.
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is ONE number for all coordinates."""
    return rms(x, eps) * g.reshape(())


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def short_conv(x, w):
    """``x [T, C]``, ``w [C, taps]`` (last column = the current token), zeros before the start -> ``[T, C]``."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1 - j)
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y


def unit(x):
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_mixer(h, w, m, eps, per_channel):
    """Gated delta rule, ``h [T, W]``.  ``per_channel``: one decay per head and key channel (through a low-rank pair
    ``a1, a2``) and a sigmoid low-rank output gate; otherwise one decay per head and a silu output gate."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, Dv)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w["b"].T)                                             # [T, H]
    if per_channel:
        pre = (h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]                              # [T, H * D]
        g = torch.exp(-torch.exp(w["A_log"]).reshape(1, H, 1) * softplus(pre).reshape(T, H, D))
        gate = torch.sigmoid((h @ w["g1"].T) @ w["g2"].T)
    else:
        pre = h @ w["a"].T + w["dt_bias"]                                           # [T, H]
        g = torch.exp(-torch.exp(w["A_log"]) * softplus(pre)).reshape(T, H, 1).expand(T, H, D)
        gate = silu(h @ w["g"].T)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(D, Dv, dtype=F64)
        for t in range(T):
            S = g[t, hd].reshape(D, 1) * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, hd] = S.T @ q[t, kv]
    out = rms(out, eps) * w["norm"].reshape(1, 1, Dv)
    return (out.reshape(T, H * Dv) * gate) @ w["o"].T


def attention_keys_values(h, w, m):
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    return (h @ w["k"].T).reshape(T, G, 2, D), (h @ w["v"].T).reshape(T, G, Dv)


def diff_attention(h, w, m, eps, k, v):
    """Differential attention with a sliding window; ``k [T, G, 2, D]``, ``v [T, G, Dv]`` are this layer's or, with
    ``kv_from``, another layer's."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window = (m.get("mask") or {}).get("size")
    q = (h @ w["q"].T).reshape(T, H, 2, D)
    lam = (torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + m["diff"])
    i = torch.arange(T).reshape(T, 1)
    j = torch.arange(T).reshape(1, T)
    vis = (j <= i)
    if window:
        vis = vis & (i - j < window)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        kv = hd // (H // G)
        maps = []
        for mp in range(2):
            s = (q[:, hd, mp] @ k[:, kv, mp].T) * m["scale"]
            s = s.masked_fill(~vis, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, kv])
        o = maps[0] - lam * maps[1]
        out[:, hd] = rms(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * Dv) @ w["o"].T


def dense_ff(h, w):
    return (silu(h @ w["gate"].T + w["gate.b"]) * (h @ w["up"].T + w["up.b"])) @ w["down"].T + w["down.b"]


def moe_ff(h, w, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w["router"].T + w["router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    p = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            a = silu(h[t] @ w[f"e{e}.gate"].T) * (h[t] @ w[f"e{e}.up"].T)
            out[t] += p[t, c] * (a @ w[f"e{e}.down"].T)
    return out


def sub(sd, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in sd.items() if k.startswith(prefix)}


def forward(cfg, sd, tokens, return_layers=False):
    """Logits ``[T, vocab]`` (float64) of one sequence; with ``return_layers`` also the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = sd["embed"].to(F64)[torch.tensor(tokens)] * cfg["embedding"]["scale"]
    kv = {}
    streams = []
    for i, L in enumerate(cfg["layers"]):
        h = scalar_norm(x, sd[f"l{i}.norm1"].to(F64), eps)
        w, m = sub(sd, f"l{i}.mix."), L["mixer"]
        if L["type"] == "attention":
            j = m.get("kv_from")
            if j is None:
                kv[i] = attention_keys_values(h, w, m)
                j = i
            y = diff_attention(h, w, m, eps, *kv[j])
        else:
            y = delta_mixer(h, w, m, eps, per_channel=L["type"] == "channel_delta")
        gate = torch.sigmoid(h @ sd[f"l{i}.rg1"].to(F64).T + sd[f"l{i}.rg1.b"].to(F64))
        upd = y * sd[f"l{i}.ls1"].to(F64) * gate
        if L.get("mlp"):
            wm = sub(sd, f"l{i}.mlp.")
            f = dense_ff(h, wm) if L["mlp"]["kind"] == "dense" else moe_ff(h, wm, L["mlp"])
            gate2 = torch.sigmoid(h @ sd[f"l{i}.rg2"].to(F64).T + sd[f"l{i}.rg2.b"].to(F64))
            upd = upd + f * sd[f"l{i}.ls2"].to(F64) * gate2
        x = x + upd
        streams.append(x.clone())
    logits = scalar_norm(x, sd["final.norm"].to(F64), eps) @ sd["head"].to(F64).T
    return (logits, torch.stack(streams)) if return_layers else logits


def random_weights(cfg, seed=0, dtype=torch.float32, std=None):
    """A checkpoint of the design with weights that keep activations of order one through the layers."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=None):
        return (torch.randn(o, i, generator=g) * (s if s is not None else (std or i ** -0.5))).to(dtype)

    def vec(n, mean=0.0, s=0.1):
        return (mean + torch.randn(n, generator=g) * s).to(dtype)

    sd = {"embed": mat(V, W, 1.0 / cfg["embedding"]["scale"]), "head": mat(V, W), "final.norm": vec(1, 1.0).reshape(())}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        sd[p + "norm1"] = vec(1, 1.0).reshape(())
        sd[p + "ls1"], sd[p + "rg1"], sd[p + "rg1.b"] = vec(W, 0.5, 0.2), mat(W, W), vec(W, 0.0, 0.5)
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            sd[p + "mix.q"] = mat(H * 2 * D, W)
            if m.get("kv_from") is None:
                sd[p + "mix.k"], sd[p + "mix.v"] = mat(G * 2 * D, W), mat(G * Dv, W)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                sd[p + "mix." + n] = vec(D, 0.0, 0.3)
            sd[p + "mix.o"] = mat(W, H * Dv)
        else:
            taps = m["conv"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                sd[p + f"mix.{n}"] = mat(rows, W)
                sd[p + f"mix.{n}.conv"] = mat(rows, taps, 0.6)
            sd[p + "mix.b"] = mat(H, W)
            sd[p + "mix.A_log"] = vec(H, -0.5, 0.8)
            sd[p + "mix.norm"] = vec(Dv, 1.0, 0.2)
            if L["type"] == "channel_delta":
                r = m.get("rank", max(2, D // 4))
                sd[p + "mix.a1"], sd[p + "mix.a2"] = mat(r, W), mat(H * D, r)
                sd[p + "mix.g1"], sd[p + "mix.g2"] = mat(r, W), mat(H * Dv, r)
                sd[p + "mix.dt_bias"] = vec(H * D, -1.0, 1.0)
            else:
                sd[p + "mix.a"], sd[p + "mix.g"] = mat(H, W), mat(H * Dv, W)
                sd[p + "mix.dt_bias"] = vec(H, -1.0, 1.0)
            sd[p + "mix.o"] = mat(W, H * Dv)
        mlp = L.get("mlp")
        if mlp:
            sd[p + "ls2"], sd[p + "rg2"], sd[p + "rg2.b"] = vec(W, 0.5, 0.2), mat(W, W), vec(W, 0.0, 0.5)
            if mlp["kind"] == "dense":
                F = mlp["ff"]
                sd[p + "mlp.gate"], sd[p + "mlp.gate.b"] = mat(F, W), vec(F)
                sd[p + "mlp.up"], sd[p + "mlp.up.b"] = mat(F, W), vec(F)
                sd[p + "mlp.down"], sd[p + "mlp.down.b"] = mat(W, F), vec(W)
            else:
                F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
                sd[p + "mlp.router"], sd[p + "mlp.router.b"] = mat(E, W, 2.0 * W ** -0.5), vec(E, 0.0, 0.5)
                for e in range(E):
                    sd[p + f"mlp.e{e}.gate"], sd[p + f"mlp.e{e}.up"] = mat(F, W), mat(F, W)
                    sd[p + f"mlp.e{e}.down"] = mat(W, F)
    return sd


def greedy(cfg, sd, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, sd, toks)[-1].argmax()))
    return toks[len(prompt):]


assert math.isclose(float(softplus(torch.tensor(0.0, dtype=F64))), math.log(2.0))

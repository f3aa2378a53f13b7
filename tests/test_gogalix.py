"""Gogalix family against the float64 oracle of ``tests/gogalix_oracle.py``: every mechanism alone, then the model through
the framework's step function, cache / state manager and schedulers.  Every test runs on the CPU (the ops' PyTorch
path) and, marked ``gpu``, on CUDA (the kernels) in fp32 and bf16."""
import json
import os
import subprocess
import sys

import pytest
import torch

import gogalix_oracle as O
from neuronx_distributed_llama3_2_b200.inference import GogalixInferenceModel, InferenceConfig
from neuronx_distributed_llama3_2_b200.inference.kv_cache import KVCache
from neuronx_distributed_llama3_2_b200.inference.trace_replay import TraceReplayer
from neuronx_distributed_llama3_2_b200.models.gogalix import (GogalixConfig, convert_gogalix_state_dict,
                                                              export_gogalix_state_dict, in_proj_columns, tiny_gogalix)
from neuronx_distributed_llama3_2_b200.modules.moe.sparse import SparseMoE
from neuronx_distributed_llama3_2_b200.ops import delta_rule as dr
from neuronx_distributed_llama3_2_b200.ops import mlstm as ml
from neuronx_distributed_llama3_2_b200.ops import moe_sparse as ms
from neuronx_distributed_llama3_2_b200.ops import norm as norm_ops
from neuronx_distributed_llama3_2_b200.ops import window_attention as wa

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64
CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu),
         pytest.param("cuda", torch.bfloat16, marks=pytest.mark.gpu)]
case = pytest.mark.parametrize("dev,dt", CASES)
DEVS = pytest.mark.parametrize("dev", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])


def tol(dt):
    return 2e-4 if dt == torch.float32 else 6e-2


def close(a, b, dt, scale=1.0):
    err = (a.detach().to("cpu", F64) - b.to(F64)).abs().max().item()
    assert err <= tol(dt) * scale, f"max error {err:.3e} above {tol(dt) * scale:.1e}"


ATT = dict(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.3, diff=0.4, mask={"size": 9})
DELTA = dict(heads=4, kv_heads=2, dim=8, vdim=12, conv=3)
CHANNEL = dict(heads=2, kv_heads=2, dim=12, vdim=8, conv=4, rank=6)
FF = {"kind": "dense", "ff": 56}
MOE = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}


def layer(kind, mlp=FF, **kw):
    m = dict({"attention": ATT, "delta": DELTA, "channel_delta": CHANNEL}[kind])
    m.update(kw)
    return {"type": kind, "mixer": m, "mlp": mlp}


def config(layers=None, vocab=96, width=40, scale=3.0, eps=1e-5):
    layers = layers or [layer("delta"), layer("attention", mlp=MOE), layer("channel_delta", mlp=None),
                        layer("attention", kv_from=1, mask={"size": 5}), layer("delta", mlp=MOE, conv=2)]
    return {"architecture": "Gogalix", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": layers}


# what the usual configurations make equal or 1: a single head, as many key heads as heads and one key head for all,
# one tap (no convolution), top-1 and all experts chosen, a window of one and none, a low-rank pair of rank one, equal and
# odd key / value sizes, no feed-forward at all, an attention first layer, key size wider than a warp
ODD = config(layers=[
    layer("attention", mlp=None, heads=3, kv_heads=3, dim=6, vdim=6, mask={"size": 1}, diff=0.8, scale=1.0),
    layer("channel_delta", heads=1, kv_heads=1, dim=5, vdim=7, conv=1, rank=1,
          mlp={"kind": "moe", "expert": {"ff": 9}, "router": {"experts": 3, "top": 1}}),
    layer("attention", heads=6, kv_heads=1, dim=10, vdim=3, mask=None, diff=0.1, scale=0.05,
          mlp={"kind": "moe", "expert": {"ff": 7}, "router": {"experts": 2, "top": 2}}),
    layer("delta", mlp=None, heads=3, kv_heads=1, dim=33, vdim=35, conv=5),
    layer("attention", mlp=None, heads=6, kv_heads=1, dim=10, vdim=3, mask={"size": 20}, diff=0.1, scale=0.05, kv_from=2),
    layer("channel_delta", mlp={"kind": "dense", "ff": 11}, heads=4, kv_heads=2, dim=70, vdim=4, conv=2, rank=3),
], vocab=50, width=30, scale=0.7, eps=1e-3)


def build(cfg, dev, dt, lines=4, seq_len=96, seed=0, paged=False, pages=None, page_size=8, sd=None):
    sd = sd if sd is not None else O.random_weights(cfg, seed)
    gc = GogalixConfig.from_dict(cfg, torch_dtype=dt).with_checkpoint_shapes(sd)
    ic = InferenceConfig(batch_size=lines, max_batch_size=lines, max_context_length=seq_len, seq_len=seq_len,
                         is_continuous_batching=True, use_cuda_graphs=False, paged_kv=paged, page_size=page_size,
                         num_kv_pages=pages)
    model = GogalixInferenceModel(gc, ic, device=torch.device(dev))
    missing, unexpected = model.load_state_dict(convert_gogalix_state_dict(sd, gc), strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    model.init_kv_cache(device=torch.device(dev))
    return model, sd


def tokens_of(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def replay(model, steps):
    rp = TraceReplayer(model)
    got = {}
    for entries, end in steps:
        out = rp.step(entries, end)
        r = 0
        for e in entries:
            for _ in e["want"]:
                got.setdefault(e["id"], []).append(out[r].cpu())
                r += 1
    return got


def check_rows(rows, ref, places, dt, strict=2e-4):
    """Every position against the oracle: centred difference over the vocabulary, relative to the spread of the logits.
    fp32 is strict; bf16 rounding through the tiny layers reaches a few percent at single positions, so bf16 bounds every
    position at 0.2 and the mean over positions at 0.05 -- a wrong key, edge or state moves positions by far more."""
    assert len(rows) == len(places)
    rels = []
    for row, p in zip(rows, places):
        d = row.to(F64) - ref[p]
        d = d - d.mean()
        rel = float(d.pow(2).mean().sqrt() / ref[p].std())
        assert rel <= (strict if dt == torch.float32 else 0.2), f"position {p}: relative error {rel:.2e}"
        rels.append(rel)
    assert dt == torch.float32 or sum(rels) / len(rels) <= 0.05, f"mean relative error {sum(rels) / len(rels):.2e}"


# ---- mechanisms alone ------------------------------------------------------------------------------------------------------
@case
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_convolution_unit_norm_and_its_state(dev, dt, taps):
    """q | k | v channels at odd columns of a wider row, fed in portions of 1 .. 5 tokens next to a padded row, on a line
    that holds a stale state: equal to the convolution over the whole sequence."""
    torch.manual_seed(0)
    H, G, D, Dv, T = 3, 1, 5, 7, 19
    C = 2 * G * D + H * Dv
    ld, oq, ok, ov = C + 11, 3, 3 + G * D + 2, 3 + 2 * G * D + 4
    raw = torch.randn(2, T, ld).to(dt)
    w = torch.randn(C, taps) * 0.5
    state = torch.randn(3, taps - 1, C).to(dev)                 # lines 2 and 0 are used; what they hold is stale
    lines = torch.tensor([2, 0], dtype=torch.int32, device=dev)
    got = [[], []]
    lens = [T, 11]
    at = [0, 0]
    for size in (1, 2, 5, 3, 4, 4):
        n_new = [min(size, lens[b] - at[b]) for b in range(2)]
        chunk = torch.zeros(2, size, ld, dtype=dt)
        for b in range(2):
            chunk[b, : n_new[b]] = raw[b, at[b]: at[b] + n_new[b]]
        q, k, v = dr.delta_prep(chunk.to(dev), (oq, ok, ov), w.to(dev), state, torch.tensor(at, dtype=torch.int32, device=dev),
                                H, G, D, Dv, 0.5, 1e-6, n_new=torch.tensor(n_new, dtype=torch.int32, device=dev), seq_ids=lines)
        for b in range(2):
            got[b].append(torch.cat([q[b, : n_new[b]].flatten(1), k[b, : n_new[b]].flatten(1),
                                     v[b, : n_new[b]].flatten(1)], dim=-1).cpu())
            at[b] += n_new[b]
    for b in range(2):
        x = raw[b, : lens[b]].to(F64)
        x = torch.cat([x[:, oq: oq + G * D], x[:, ok: ok + G * D], x[:, ov: ov + H * Dv]], dim=-1)
        y = O.silu(O.short_conv(x, w.to(F64)))
        q = O.unit(y[:, : G * D].reshape(-1, G, D)).reshape(-1, G * D) * 0.5
        k = O.unit(y[:, G * D: 2 * G * D].reshape(-1, G, D)).reshape(-1, G * D)
        close(torch.cat(got[b]), torch.cat([q, k, y[:, 2 * G * D:]], dim=-1), dt, scale=0.5)


def scan_oracle(q, k, v, g, beta):
    """float64: q, k [T, G, D], v [T, H, Dv], g [T, H, D] decay factors, beta [T, H] -> o [T, H, Dv]."""
    T, G, D = q.shape
    H, Dv = v.shape[1], v.shape[2]
    out = torch.zeros(T, H, Dv, dtype=F64)
    for h in range(H):
        S = torch.zeros(D, Dv, dtype=F64)
        for t in range(T):
            S = g[t, h].reshape(D, 1) * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h // (H // G)])
            S = S + torch.outer(k[t, h // (H // G)], u)
            out[t, h] = S.T @ q[t, h // (H // G)]
    return out


@DEVS
@pytest.mark.parametrize("per_channel", [False, True], ids=["head_decay", "channel_decay"])
@pytest.mark.parametrize("H,G,D,Dv", [(1, 1, 5, 7), (4, 2, 16, 12), (2, 1, 40, 33), (2, 2, 70, 20), (1, 1, 130, 9)])
def test_delta_recurrence_in_portions_with_padding_on_a_stale_line(dev, per_channel, H, G, D, Dv):
    torch.manual_seed(1)
    T, lens = 37, [37, 20]
    q = O.unit(torch.randn(2, T, G, D, dtype=F64)) * D ** -0.5
    k = O.unit(torch.randn(2, T, G, D, dtype=F64))
    v = torch.randn(2, T, H, Dv, dtype=F64)
    na = H * D if per_channel else H
    a_pre = torch.randn(2, T, 3 + na, dtype=F64)
    b_pre = torch.randn(2, T, H + 2, dtype=F64)
    a_log, dt_bias = torch.randn(H, dtype=F64) * 0.5 - 1.0, torch.randn(na, dtype=F64)
    g = torch.exp(-torch.exp(a_log).reshape(H, 1) * O.softplus(a_pre[..., 3:] + dt_bias).reshape(2, T, H, -1)).expand(2, T, H, D)
    beta = torch.sigmoid(b_pre[..., 2:])
    S = torch.randn(3, H, D, Dv).to(dev)                          # stale content: both rows start at position 0
    lines = torch.tensor([1, 2], dtype=torch.int32, device=dev)
    f32 = lambda x: x.float().contiguous().to(dev)                # noqa: E731
    got, at = [[], []], [0, 0]
    for size in (1, 16, 3, 17):
        n_new = [min(size, lens[b] - at[b]) for b in range(2)]

        def part(x):
            out = torch.zeros((2, size) + x.shape[2:], dtype=F64)
            for b in range(2):
                out[b, : n_new[b]] = x[b, at[b]: at[b] + n_new[b]]
            return out

        o = dr.delta_scan(f32(part(q)), f32(part(k)), f32(part(v)), f32(part(a_pre)).reshape(2 * size, -1), 3,
                          f32(part(b_pre)).reshape(2 * size, -1), 2, f32(a_log), f32(dt_bias), S,
                          torch.tensor(at, dtype=torch.int32, device=dev), per_channel,
                          n_new=torch.tensor(n_new, dtype=torch.int32, device=dev), seq_ids=lines)
        for b in range(2):
            assert float(o[b, n_new[b]:].abs().max() if n_new[b] < size else 0.0) == 0.0      # padding comes out as zeros
            got[b].append(o[b, : n_new[b]].cpu())
            at[b] += n_new[b]
    for b in range(2):
        ref = scan_oracle(q[b, : lens[b]], k[b, : lens[b]], v[b, : lens[b]], g[b, : lens[b]], beta[b, : lens[b]])
        close(torch.cat(got[b]), ref, torch.float32, scale=max(1.0, float(ref.abs().max())))


def maps_oracle(q, k, v, pos_q, scale, window):
    """float64 softmax attention of ``q [Tq, H, D]`` at positions ``pos_q`` over ``k [Tk, G, D]``, ``v [Tk, Gv, Dv]``."""
    H, G = q.shape[1], k.shape[1]
    j = torch.arange(k.shape[0]).reshape(1, -1)
    i = torch.tensor(pos_q).reshape(-1, 1)
    vis = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T * scale).masked_fill(~vis, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g % v.shape[1]])
    return torch.stack(out, dim=1)


@case
@pytest.mark.parametrize("paged", [False, True], ids=["contiguous", "paged"])
@pytest.mark.parametrize("D,Dv,window", [(8, 12, 9), (32, 32, 33), (64, 64, 16), (10, 3, None), (48, 96, 20), (32, 64, 7)])
def test_two_maps_over_shared_values_and_the_window_edge(dev, dt, paged, D, Dv, window):
    """Map-major query / key heads (2H over 2G) read G value heads; a key that dominates map 1 is planted so that it is
    just inside the window of one query and just outside the next one's, in a prompt portion and in decoding."""
    torch.manual_seed(2)
    H, G, T0, T1 = 4, 2, 7, 40
    T = T0 + T1 + 2
    page = 8
    q = torch.randn(T, 2 * H, D) * 0.5
    k = torch.randn(T, 2 * G, D) * 0.5
    v = torch.randn(T, G, Dv)
    w = window or 0
    plant = 12
    k[plant, :G] = 0.0
    k[plant, :G, 0] = 8.0
    q[:, :H, 0] = 6.0                                          # every query of map 1 looks for the planted key
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    lines = 3
    if paged:
        n_pages = lines * ((T + page - 1) // page)
        ck = torch.zeros(n_pages, 2 * G, page, D, dtype=dt, device=dev)
        cv = torch.zeros(n_pages, G, page, Dv, dtype=dt, device=dev)
        table = torch.randperm(n_pages).reshape(lines, -1).to(torch.int32).to(dev)
        kw = dict(block_table=table, page_size=page)
    else:
        ck = torch.randn(lines, 2 * G, T, D, device=dev).to(dt)       # stale rows behind the written ones
        cv = torch.randn(lines, G, T, Dv, device=dev).to(dt)
        kw = {}
    line = torch.tensor([1], dtype=torch.int32, device=dev)
    got = []
    for lo, hi in ((0, T0), (T0, T0 + T1)):
        n = hi - lo
        row = torch.cat([q[lo:hi].reshape(n, -1), k[lo:hi].reshape(n, -1), v[lo:hi].reshape(n, -1)], dim=-1)
        wide = torch.zeros(1, n + 3, row.shape[1] + 5, dtype=dt)        # three rows of padding, five foreign columns
        wide[0, :n, : row.shape[1]] = row
        wide = wide.to(dev)
        start = torch.tensor([lo], dtype=torch.int32, device=dev)
        nn_ = torch.tensor([n], dtype=torch.int32, device=dev)
        qq = wa.qk_norm_cache_write(wide[..., : row.shape[1]], ck, cv, start, 2 * H, 2 * G, D, Dv, 1e-6, n_new=nn_,
                                    seq_ids=line, normalize=False, value_heads=G, **kw)
        o = wa.window_attention_prefill(qq, ck, cv, start, 0.4, w, n_new=nn_, seq_ids=line, value_heads=G, **kw)
        got.append(o[0, :n].cpu())
    for t in range(T0 + T1, T):
        row = torch.cat([q[t].reshape(1, -1), k[t].reshape(1, -1), v[t].reshape(1, -1)], dim=-1).reshape(1, 1, -1).to(dev)
        start = torch.tensor([t], dtype=torch.int32, device=dev)
        qq = wa.qk_norm_cache_write(row, ck, cv, start, 2 * H, 2 * G, D, Dv, 1e-6, seq_ids=line, normalize=False,
                                    value_heads=G, **kw)
        got.append(wa.window_attention_decode(qq[:, 0], ck, cv, start, 0.4, w, seq_ids=line, value_heads=G, **kw).cpu())
    got = torch.cat(got)
    ref = maps_oracle(q.to(F64), k.to(F64), v.to(F64), list(range(T)), 0.4, w)
    close(got, ref, dt, scale=2.0)
    if window:                              # the planted key decides map 1 while it is visible, and only then
        inside, outside = plant + window - 1, plant + window
        vp = v[plant].to(F64)
        assert float((ref[inside, 0] - vp[0]).abs().max()) < 1e-3 and float((ref[outside, 0] - vp[0]).abs().max()) > 0.1
    # the combination of the two maps
    lq1, lk1, lq2, lk2 = (torch.randn(D) * 0.3 for _ in range(4))
    lam = torch.exp((lq1 * lk1).sum().to(F64)) - torch.exp((lq2 * lk2).sum().to(F64)) + 0.3
    comb = O.rms(ref[:, :H] - lam * ref[:, H:], 1e-5) * 0.7
    out = wa.diff_attention_combine(ref.to(dt).to(dev), lq1.to(dev), lk1.to(dev), lq2.to(dev), lk2.to(dev), 0.3, 1e-5)
    close(out, comb.reshape(T, -1), dt, scale=3.0)


@case
def test_gated_residual_with_layer_scale_and_the_one_weight_norm(dev, dt):
    torch.manual_seed(3)
    N, W = 9, 37
    x = torch.randn(N, W) * 3 + 1.0
    y1, y2 = torch.randn(N, W).to(dt), torch.randn(N, W)            # the second sublayer's result may be fp32
    gate = torch.randn(N, 2 * W + 13).to(dt)
    b2, gb1, gb2, s1, s2 = (torch.randn(W) for _ in range(5))
    wn = torch.tensor([1.7])
    f = lambda t: t.to(F64)                                         # noqa: E731
    for two in (True, False):
        ref = f(x) + f(s1) * torch.sigmoid(f(gate)[:, 5: 5 + W] + f(gb1)) * f(y1)
        if two:
            ref = ref + f(s2) * torch.sigmoid(f(gate)[:, W + 9: 2 * W + 9] + f(gb2)) * (f(y2) + f(b2))
        xs = x.clone().to(dev)
        d = lambda t: t.to(dev)                                     # noqa: E731
        xo, h = norm_ops.gated_residual_norm_(xs, d(y1), d(y2) if two else None, d(b2) if two else None, d(gate),
                                              (5, W + 9), d(gb1), d(gb2) if two else None, d(s1), d(s2) if two else None,
                                              d(wn), 1e-4, dt)
        assert xo.data_ptr() == xs.data_ptr()
        close(xs, ref, torch.float32, scale=10.0)
        close(h, O.scalar_norm(ref, f(wn), 1e-4), dt, scale=2.0)
    xs = x.clone().to(dev)
    _, h = norm_ops.gated_residual_norm_(xs, None, w_next=wn.to(dev), eps=1e-4, out_dtype=dt)        # the plain norm
    assert torch.equal(xs.cpu(), x)
    close(h, O.scalar_norm(f(x), f(wn), 1e-4), dt, scale=2.0)


@case
@pytest.mark.parametrize("E,top", [(5, 2), (3, 1), (2, 2), (40, 3)])
def test_router_with_bias_chosen_logits_softmax_and_plain_gated_experts(dev, dt, E, top):
    torch.manual_seed(4)
    N, W, F = 33, 24, 10
    h = torch.randn(N, W).to(dt)
    wr, br = torch.randn(E, W), torch.randn(E) * 2
    z = h.to(F64) @ wr.to(F64).T + br.to(F64)
    val, idx = torch.topk(z, top, dim=-1)
    gi, gw, _ = ms.route(h.to(dev), wr.to(dev), None, top, 1.0, logit_bias=br.to(dev), renormalize=True)
    assert torch.equal(gi.cpu().long().sort(dim=-1).values, idx.sort(dim=-1).values)       # no near ties with this seed
    order = gi.cpu().long()
    close(gw, torch.softmax(z.gather(1, order), dim=-1), torch.float32)
    moe = SparseMoE(W, E, top, F, None, dtype=dt, device=torch.device(dev), router_bias=True, renormalize=True)
    wg, wu, wd = torch.randn(E, F, W) * 0.3, torch.randn(E, F, W) * 0.3, torch.randn(E, W, F) * 0.3
    with torch.no_grad():
        moe.router.linear_router.weight.copy_(wr)
        moe.router.logit_bias.copy_(br)
        moe.experts.gate_up_proj.weight.copy_(torch.cat([wg.transpose(1, 2), wu.transpose(1, 2)], dim=2).to(dt))
        moe.experts.down_proj.weight.copy_(wd.transpose(1, 2).to(dt))
    sd = {"router": wr, "router.b": br}
    for e in range(E):
        sd[f"e{e}.gate"], sd[f"e{e}.up"], sd[f"e{e}.down"] = wg[e].to(dt), wu[e].to(dt), wd[e].to(dt)
    ref = O.moe_ff(h.to(F64), {k: v.to(F64) for k, v in sd.items()}, {"router": {"experts": E, "top": top}})
    for path in ("pairs", "sorted"):
        close(moe(h.to(dev), path=path), ref, dt, scale=3.0)
    # gate and up as column ranges of a wider row, with biases
    src = torch.randn(N, 2 * F + 9).to(dt)
    gb, ub = torch.randn(F), torch.randn(F)
    act = ms.glu_bias(src.to(dev), 2, F + 7, F, gb.to(dev), ub.to(dev))
    s64 = src.to(F64)
    close(act, O.silu(s64[:, 2: 2 + F] + gb.to(F64)) * (s64[:, F + 7: 2 * F + 7] + ub.to(F64)), dt, scale=4.0)


@case
def test_head_norm_with_a_silu_gate_from_a_wider_row(dev, dt):
    torch.manual_seed(5)
    N, H, Dv = 7, 3, 10
    o = torch.randn(N, H, Dv)
    src = torch.randn(N, H * Dv + 6).to(dt)
    w = torch.randn(Dv).abs() + 0.5
    for act, fn in (("silu", O.silu), ("sigmoid", torch.sigmoid)):
        got = ml.head_norm_gate(o.to(dev), src.to(dev), 4, H, Dv, w.repeat(H).to(dev), 1e-5, True, dt, gate_act=act)
        ref = (O.rms(o.to(F64), 1e-5) * w.to(F64)).reshape(N, -1) * fn(src.to(F64)[:, 4: 4 + H * Dv])
        close(got, ref, dt, scale=3.0)


def test_cache_holds_two_key_heads_per_value_head_and_the_recurrent_state_per_line():
    cfg = tiny_gogalix()
    model = GogalixInferenceModel(cfg, InferenceConfig(batch_size=2, max_batch_size=2, seq_len=16, max_context_length=16))
    kc = model.init_kv_cache()
    k, v = kc.layer(1)
    m = cfg.layers[1].mixer
    assert k.shape == (2, 2 * m.kv_heads, 16, m.dim) and v.shape == (2, m.kv_heads, 16, m.vdim)
    assert kc.layer(3)[0].data_ptr() == k.data_ptr() and not kc.owns(3)
    d = cfg.layers[2].mixer
    assert kc.state(2)["S"].shape == (2, d.heads, d.dim, d.vdim) and kc.state(2)["conv"].shape == (2, d.conv - 1, d.channels)
    assert kc.layer(0) == (None, None)
    gen = KVCache(1, 2, 0, 8, 0, dtype=torch.float32, layer_specs=[(6, 4, 5, "heads", 3)])
    assert gen.layer(0)[0].shape == (2, 6, 8, 4) and gen.layer(0)[1].shape == (2, 3, 8, 5)


def test_checkpoint_names_round_trip_and_the_fused_projection_layout():
    cfg = tiny_gogalix()
    model = GogalixInferenceModel(cfg, InferenceConfig(batch_size=1, max_batch_size=1, seq_len=8, max_context_length=8))
    with torch.no_grad():
        for name, p in model.named_parameters():
            if not name.endswith(("in_proj.weight", "gate_proj", "mixer.a2", "mixer.g2", "out_norm", "correction")):
                p.copy_(torch.randn_like(p))
    sd = export_gogalix_state_dict(model)
    back = convert_gogalix_state_dict(sd, cfg)
    again = export_gogalix_state_dict_from(back, cfg)
    assert set(again) == set(sd)
    for k in sd:
        assert torch.equal(again[k], sd[k]), k
    assert GogalixConfig.from_dict(cfg.to_dict(), torch.float32).to_dict() == cfg.to_dict()
    for L in cfg.layers:                                            # every part of the fused projection starts aligned
        cols, n_out = in_proj_columns(cfg, L)
        assert n_out % 8 == 0 and all(at % 8 == 0 for at, _ in cols.values())
    bad = config(layers=[layer("attention"), layer("attention", kv_from=0, dim=4)])
    with pytest.raises(ValueError):
        GogalixConfig.from_dict(bad)
    with pytest.raises(ValueError):
        GogalixConfig.from_dict(config(layers=[layer("delta"), layer("attention", kv_from=0)]))


def export_gogalix_state_dict_from(state, cfg):
    model = GogalixInferenceModel(cfg, InferenceConfig(batch_size=1, max_batch_size=1, seq_len=8, max_context_length=8))
    missing, unexpected = model.load_state_dict(state, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    return export_gogalix_state_dict(model)


# ---- the model through the framework -----------------------------------------------------------------------------------
@case
@pytest.mark.parametrize("cfg", [config(), ODD], ids=["mixed", "odd"])
def test_prefill_matches_oracle_and_token_by_token_decoding(dev, dt, cfg):
    toks = tokens_of(cfg, 45, 1)
    model, sd = build(cfg, dev, dt)
    ref, streams = O.forward(cfg, sd, toks, return_layers=True)
    want = list(range(45))
    seen = []
    model.layer_probe = lambda i, x: seen.append(x.detach().to("cpu", F64))
    whole = replay(model, [([{"id": "a", "tokens": toks, "want": want}], ["a"])])["a"]
    model.layer_probe = None
    check_rows(whole, ref, want, dt)
    assert len(seen) == len(streams)
    for got, exp in zip(seen, streams):                       # the residual stream after every layer
        assert float((got[0] - exp).abs().max()) <= (2e-3 if dt == torch.float32 else 0.5)
    steps = [([{"id": "b", "tokens": toks[:1], "want": [0]}], [])]
    steps += [([{"id": "b", "tokens": [t], "want": [0]}], []) for t in toks[1:]]
    check_rows(replay(model, steps)["b"], ref, want, dt)


@case
@pytest.mark.parametrize("portion", [2, 5, 16])
def test_portions_of_a_prompt(dev, dt, portion):
    cfg = config()
    toks = tokens_of(cfg, 41, 6)
    model, sd = build(cfg, dev, dt)
    ref = O.forward(cfg, sd, toks)
    steps, places = [], []
    for lo in range(0, 41, portion):
        part = toks[lo:lo + portion]
        steps.append(([{"id": "p", "tokens": part, "want": list(range(len(part)))}], []))
        places += list(range(lo, lo + len(part)))
    check_rows(replay(model, steps)["p"], ref, places, dt)


@case
def test_unequal_batch_equals_each_alone_and_lines_are_reused(dev, dt):
    cfg = config()
    model, sd = build(cfg, dev, dt, lines=3)
    lens = {"a": 1, "b": 30, "c": 13, "d": 22, "e": 2}
    toks = {k: tokens_of(cfg, n + 6, 10 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: O.forward(cfg, sd, v) for k, v in toks.items()}
    first = [{"id": k, "tokens": toks[k][:lens[k]], "want": [lens[k] - 1]} for k in "abc"]
    steps = [(first, ["a"])]                                     # a one-token request ends at once: its line is free
    for s in range(3):
        steps.append(([{"id": k, "tokens": [toks[k][lens[k] + s]], "want": [0]} for k in "bc"], ["c"] if s == 2 else []))
    # two new requests take the lines that a and c gave back: stale keys, a stale matrix state and a stale convolution
    # state lie in them (e is shorter than the convolution)
    steps.append(([{"id": k, "tokens": toks[k][:lens[k]], "want": [0, lens[k] - 1]} for k in "de"], []))
    for s in range(6):
        steps.append(([{"id": k, "tokens": [toks[k][lens[k] + s]], "want": [0]} for k in "de"], []))
    got = replay(model, steps)
    check_rows(got["a"], ref["a"], [0], dt)
    for k in "bc":
        check_rows(got[k], ref[k], [lens[k] - 1, lens[k], lens[k] + 1, lens[k] + 2], dt)
    for k in "de":
        check_rows(got[k], ref[k], [0, lens[k] - 1] + [lens[k] + s for s in range(6)], dt)


@case
def test_long_decoding_past_every_window_over_a_small_page_pool(dev, dt):
    cfg = config()
    toks = tokens_of(cfg, 90, 4)
    model, sd = build(cfg, dev, dt, lines=2, paged=True, pages=14, page_size=8)
    ref = O.forward(cfg, sd, toks)
    steps = [([{"id": "x", "tokens": toks[:5], "want": [4]}], [])]
    steps += [([{"id": "x", "tokens": [t], "want": [0]}], []) for t in toks[5:]]
    check_rows(replay(model, steps)["x"], ref, list(range(4, 90)), dt)


@case
@pytest.mark.parametrize("kind", ["delta", "channel_delta"])
def test_a_token_far_back_lives_on_in_the_state(dev, dt, kind):
    """One recurrent layer with a slow decay whose write strength (beta) is next to zero for every token but one: token id
    5, at position 1 only, is the only one with a non-zero embedding column 1, which the beta rows read with a large
    positive weight, while they read column 0 -- shared by all tokens -- with a negative one.  The state then holds what
    position 1 wrote, and the logits 280 positions later still depend on it (the oracle says by how much): in a long
    prompt step, in a portion at an offset and while decoding."""
    cfg = config(layers=[layer(kind, mlp=None)], scale=2.0)
    sd = O.random_weights(cfg, seed=3)
    sd["l0.mix.A_log"] = torch.full_like(sd["l0.mix.A_log"], -7.0)          # decay factors of 0.999 and more
    sd["embed"][:, 0], sd["embed"][:, 1] = 1.0, 0.0                          # times the embedding scale of 2
    sd["embed"][5, 1] = 3.0
    sd["l0.mix.b"][:] = 0.0
    sd["l0.mix.b"][:, 0], sd["l0.mix.b"][:, 1] = -6.0, 8.0
    sd["l0.ls1"][:] = 2.0                                                    # the mixer's share of the stream
    sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    toks = [t if t != 5 else 6 for t in tokens_of(cfg, 300, 9)]
    toks[1] = 5
    ref = O.forward(cfg, sd, toks)
    moved = list(toks)
    moved[1] = 6
    far = O.forward(cfg, sd, moved)
    d = (far[290] - ref[290])
    assert float((d - d.mean()).pow(2).mean().sqrt() / ref[290].std()) > 0.2
    model, _ = build(cfg, dev, dt, sd=sd, seq_len=320, lines=2)
    steps = [([{"id": "f", "tokens": toks[:200], "want": [0, 1, 2, 199]}], []),
             ([{"id": "f", "tokens": toks[200:280], "want": [0, 79]}], [])]
    steps += [([{"id": "f", "tokens": [t], "want": [0]}], []) for t in toks[280:]]
    check_rows(replay(model, steps)["f"], ref, [0, 1, 2, 199, 200, 279] + list(range(280, 300)), dt, strict=1e-3)


@case
def test_window_edges_in_prompts_and_in_decoding(dev, dt):
    """One attention layer with a window of 9: only token id 5, at position 11, has a non-zero embedding column 1; the first
    key dimension of map 1 reads that column and the first query dimension of map 1 reads column 0, which all tokens
    share, so that key takes map 1 of every query that sees it.  Position 19 is the last that does."""
    cfg = config(layers=[layer("attention", mlp=None, scale=1.0)], scale=1.0)
    m = cfg["layers"][0]["mixer"]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    sd = O.random_weights(cfg, seed=11)
    sd["embed"][:, 0], sd["embed"][:, 1] = 1.0, 0.0
    sd["embed"][5, 1] = 6.0
    for g in range(G):
        sd["l0.mix.k"][g * 2 * D] = 0.0
        sd["l0.mix.k"][g * 2 * D, 1] = 3.0
    for h in range(H):
        sd["l0.mix.q"][h * 2 * D] = 0.0
        sd["l0.mix.q"][h * 2 * D, 0] = 8.0
    sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    toks = [t if t != 5 else 6 for t in tokens_of(cfg, 44, 2)]
    toks[11] = 5
    ref = O.forward(cfg, sd, toks)
    wider = config(layers=[layer("attention", mlp=None, scale=1.0, mask={"size": 10})], scale=1.0)
    for p, differs in ((19, False), (20, True), (21, False)):            # a window one longer shows at position 20 only
        d = O.forward(wider, sd, toks)[p] - ref[p]
        assert (float((d - d.mean()).pow(2).mean().sqrt() / ref[p].std()) > 0.1) == differs
    model, _ = build(cfg, dev, dt, sd=sd)
    for cut in (13, 20, 21):                  # the edge inside a portion, at a portion's first token, in decoding
        steps = [([{"id": "c", "tokens": toks[:cut], "want": list(range(cut))}], []),
                 ([{"id": "c", "tokens": toks[cut:30], "want": list(range(30 - cut))}], [])]
        steps += [([{"id": "c", "tokens": [t], "want": [0]}], ["c"] if i == 13 else []) for i, t in enumerate(toks[30:])]
        check_rows(replay(model, steps)["c"], ref, list(range(44)), dt)
    steps = [([{"id": "d", "tokens": toks[:15], "want": [14]}], [])]
    steps += [([{"id": "d", "tokens": [t], "want": [0]}], []) for t in toks[15:25]]
    check_rows(replay(model, steps)["d"], ref, list(range(14, 25)), dt)


@case
def test_sizes_of_the_tensor_core_and_wide_register_kernels_through_the_model(dev, dt):
    """Key sizes 64 / 128 (the attention's tensor-core kernels in bf16, the widest register slices of the recurrence),
    grouped heads, prompts of 70 and 150 tokens in one batch, a portion at an offset, decoding."""
    cfg = config(layers=[layer("delta", heads=2, kv_heads=1, dim=128, vdim=64, mlp=None),
                         layer("attention", heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, mask={"size": 48}, mlp=MOE),
                         layer("channel_delta", heads=2, kv_heads=2, dim=64, vdim=128, rank=16, mlp=None),
                         layer("attention", heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, mask={"size": 80}, kv_from=1)],
                 width=64, vocab=80)
    model, sd = build(cfg, dev, dt, lines=2, seq_len=200)
    a, b = tokens_of(cfg, 170, 51), tokens_of(cfg, 80, 52)
    ra, rb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    steps = [([{"id": "a", "tokens": a[:100], "want": [0, 47, 48, 99]}, {"id": "b", "tokens": b[:70], "want": [69]}], []),
             ([{"id": "a", "tokens": a[100:160], "want": [0, 59]}], [])]
    steps += [([{"id": "a", "tokens": [a[160 + s]], "want": [0]}, {"id": "b", "tokens": [b[70 + s]], "want": [0]}], [])
              for s in range(6)]
    got = replay(model, steps)
    check_rows(got["a"], ra, [0, 47, 48, 99, 100, 159] + list(range(160, 166)), dt, strict=1e-3)
    check_rows(got["b"], rb, [69] + list(range(70, 76)), dt, strict=1e-3)


@case
def test_greedy_generation_through_generate_and_the_continuous_batcher(dev, dt):
    cfg = config()
    sd = O.random_weights(cfg, seed=5)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (7, 12, 3)]
    want = [O.greedy(cfg, sd, p, 6) for p in prompts]
    model, _ = build(cfg, dev, dt, lines=3, sd=sd)
    T = max(len(p) for p in prompts)
    ids = torch.zeros(3, T, dtype=torch.long)
    mask = torch.zeros(3, T, dtype=torch.long)
    for b, p in enumerate(prompts):
        ids[b, :len(p)], mask[b, :len(p)] = torch.tensor(p), 1
    out = model.generate(ids.to(dev), mask.to(dev), max_new_tokens=6)
    strict = dt == torch.float32
    for b, p in enumerate(prompts):
        got = out[b, len(p):len(p) + 6].tolist()
        assert got == want[b] or not strict, (got, want[b])
        assert got[0] == want[b][0]
    from neuronx_distributed_llama3_2_b200.inference.continuous_batching import ContinuousBatcher

    model2, _ = build(cfg, dev, dt, lines=2, sd=sd, paged=True, pages=9, page_size=4, seq_len=32)
    cb = ContinuousBatcher(model2)
    rids = [cb.submit(torch.tensor(p), 6) for p in prompts]
    res = cb.run()
    for rid, w in zip(rids, want):
        assert res[rid][:6] == w or not strict, (res[rid], w)
        assert res[rid][0] == w[0]


@case
def test_runner_buckets_match_oracle_greedy(dev, dt):
    from neuronx_distributed_llama3_2_b200.inference import GogalixRunner

    cfg = config()
    sd = O.random_weights(cfg, seed=12)
    gc = GogalixConfig.from_dict(cfg, torch_dtype=dt).with_checkpoint_shapes(sd)
    ic = InferenceConfig(batch_size=3, max_context_length=32, seq_len=64, buckets=[16, 32], max_new_tokens=5,
                         use_cuda_graphs=dev == "cuda")
    runner = GogalixRunner(gc, ic, checkpoint_loader=lambda: convert_gogalix_state_dict(sd, gc), device=torch.device(dev))
    runner.trace()
    prompts = [tokens_of(cfg, n, 40 + n) for n in (11, 5)]
    ids = torch.zeros(2, 11, dtype=torch.long)
    mask = torch.zeros(2, 11, dtype=torch.long)
    for b, p in enumerate(prompts):
        ids[b, :len(p)], mask[b, :len(p)] = torch.tensor(p), 1
    out = runner.generate(ids.to(dev), mask.to(dev), max_new_tokens=5)
    runner.close()
    for b, p in enumerate(prompts):
        w = O.greedy(cfg, sd, p, 5)
        got = out[b, len(p):len(p) + 5].tolist()
        assert got[0] == w[0]
        assert got == w or dt != torch.float32, (got, w)


def test_registry_and_command_line_replay(tmp_path):
    """``bin/trace_run`` on a model directory: family chosen from config.json (the low-rank size from the tensors' shapes),
    steps on stdin, logits in files."""
    from safetensors.torch import save_file

    from neuronx_distributed_llama3_2_b200.inference.registry import families

    assert "gogalix" in families()
    cfg = json.loads(json.dumps(ODD))
    sd = O.random_weights(cfg, seed=8)
    for L in cfg["layers"]:
        L["mixer"].pop("rank", None)
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in sd.items()}, str(mdir / "model.safetensors"))
    sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    toks = tokens_of(cfg, 20, 3)
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:15], "want": [0, 14]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[15:16], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": toks[16:17], "want": [0]}], "end": ["r"]}]
    out = tmp_path / "out"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, env=env, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.split("\n") if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    ref = O.forward(cfg, sd, toks)
    import numpy as np

    a = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    b = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, cfg["vocab"]))
    check_rows([a[0], a[1], b[0]], ref, [0, 14, 16], torch.float32)

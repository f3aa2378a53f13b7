"""Vufasun family against the plain oracle of ``tests/vufasun_oracle.py``: every mechanism alone, then the model through
the framework's step function, cache / state manager and schedulers.  Every test runs on the CPU (the ops' PyTorch
path) and, marked ``gpu``, on CUDA (the kernels) in fp32 and bf16."""
import json
import os
import subprocess
import sys

import pytest
import torch

import vufasun_oracle as O
from neuronx_distributed_llama3_2_b200.inference import InferenceConfig, VufasunInferenceModel
from neuronx_distributed_llama3_2_b200.inference.trace_replay import TraceReplayer
from neuronx_distributed_llama3_2_b200.models.vufasun import (VufasunConfig, convert_vufasun_state_dict,
                                                              export_vufasun_state_dict, in_proj_columns, tiny_vufasun)
from neuronx_distributed_llama3_2_b200.modules.moe.sparse import SparseMoE
from neuronx_distributed_llama3_2_b200.ops import hyper_connection as hc
from neuronx_distributed_llama3_2_b200.ops import mlstm as ml
from neuronx_distributed_llama3_2_b200.ops import moe_sparse as ms
from neuronx_distributed_llama3_2_b200.ops import retention as rt
from neuronx_distributed_llama3_2_b200.ops import rope as rp
from neuronx_distributed_llama3_2_b200.ops import window_attention as wa

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64
CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu),
         pytest.param("cuda", torch.bfloat16, marks=pytest.mark.gpu)]
case = pytest.mark.parametrize("dev,dt", CASES)


def tol(dt):
    return 2e-4 if dt == torch.float32 else 6e-2


def close(a, b, dt, scale=1.0):
    err = (a.detach().to("cpu", F64) - b.to(F64)).abs().max().item()
    assert err <= tol(dt) * scale, f"max error {err:.3e} above {tol(dt) * scale:.1e}"


ROT = {"base": 10000.0, "dims": 8}
ATT = dict(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.3, rot=ROT)
LEFT = dict(heads=2, kv_heads=1, dim=16, vdim=24, scale=0.2,
            rot={"base": 5000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}})
RIGHT = dict(heads=3, dim=8, vdim=16, decay=[0.9, 0.97, 0.995], rot={"base": 100.0, "dims": 4})
FF = {"kind": "dense", "ff": 52}
MOE = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 16}}


def layer(kind, mlp=FF, **kw):
    if kind == "attention":
        m = dict(ATT)
        m.update(kw)
    else:
        m = {"left": dict(LEFT, **kw.get("left", {})), "right": dict(RIGHT, **kw.get("right", {}))}
    return {"type": kind, "mixer": m, "mlp": mlp}


def config(layers=None, vocab=96, width=40, streams=3, eps=1e-5, loop=(0, 2, 2)):
    layers = layers or [layer("attention", mlp=None), layer("parallel", mlp=MOE), layer("attention"),
                        layer("parallel", mlp=FF)]
    d = {"architecture": "Vufasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        d["streams"] = streams
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# what the usual configurations make equal or 1: a single stream, a single head, as many key heads as heads and one for
# all, rotation over the whole head and none at all, no frequency scaling, equal and odd key / value sizes, top-1 and all
# experts chosen, no shared expert, no feed-forward, a loop of one layer three times at the end, key size wider than a warp
ODD = config(layers=[
    layer("parallel", mlp={"kind": "moe", "expert": {"ff": 9}, "router": {"experts": 3, "top": 1}},
          left=dict(heads=1, kv_heads=1, dim=6, vdim=6, scale=1.0, rot={"base": 50.0, "dims": 6}),
          right=dict(heads=1, dim=5, vdim=7, decay=[0.5], rot=None)),
    layer("attention", mlp=None, heads=3, kv_heads=3, dim=6, vdim=6, scale=1.0, rot=None),
    layer("attention", heads=6, kv_heads=1, dim=10, vdim=3, scale=0.05, rot={"base": 3.0, "dims": 10},
          mlp={"kind": "moe", "expert": {"ff": 7}, "router": {"experts": 2, "top": 2}}),
    layer("parallel", mlp={"kind": "dense", "ff": 11},
          left=dict(heads=4, kv_heads=2, dim=34, vdim=5, scale=0.1, rot={"base": 7.0, "dims": 2}),
          right=dict(heads=2, dim=33, vdim=35, decay=[1.0, 0.25], rot={"base": 1e6, "dims": 32})),
], vocab=50, width=30, streams=1, eps=1e-3, loop=(3, 4, 3))

PLAIN = config(layers=[layer("attention"), layer("parallel", mlp=None)], streams=None, loop=None)   # no stream weights at all

# five streams (more than the vectorised stream kernel takes), a middle range run four times, a fast and a nearly lossless
# decay side by side, rotation over half of a head that is no power of two, a strongly slowed frequency band
FIVE = config(layers=[
    layer("attention", heads=3, kv_heads=1, dim=24, vdim=40, scale=0.3, rot={"base": 1e4, "dims": 8},
          mlp={"kind": "moe", "expert": {"ff": 48}, "router": {"experts": 3, "top": 3}, "shared": {"ff": 40}}),
    layer("attention", heads=2, kv_heads=2, dim=80, vdim=16, scale=0.11, rot={"base": 1e5, "dims": 80}, mlp={"kind": "dense", "ff": 120}),
    layer("parallel", mlp={"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 4}, "shared": {"ff": 8}},
          left=dict(heads=6, kv_heads=2, dim=16, vdim=16, scale=0.25,
                    rot={"base": 1e4, "dims": 16, "scaling": {"factor": 16.0, "low": 2.0, "high": 3.0, "original": 64}}),
          right=dict(heads=3, dim=24, vdim=40, decay=[0.5, 0.9, 0.99999], rot={"base": 5e4, "dims": 12})),
], vocab=130, width=72, streams=5, loop=(1, 3, 4))


def build(cfg, dev, dt, lines=4, seq_len=96, seed=1, paged=False, pages=None, page_size=8, sd=None):
    sd = sd if sd is not None else O.random_weights(cfg, seed)
    vc = VufasunConfig.from_dict(cfg, torch_dtype=dt).with_checkpoint_shapes(sd)
    ic = InferenceConfig(batch_size=lines, max_batch_size=lines, max_context_length=seq_len, seq_len=seq_len,
                         is_continuous_batching=True, use_cuda_graphs=False, paged_kv=paged, page_size=page_size,
                         num_kv_pages=pages)
    model = VufasunInferenceModel(vc, ic, device=torch.device(dev))
    missing, unexpected = model.load_state_dict(convert_vufasun_state_dict(sd, vc), strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    model.init_kv_cache(device=torch.device(dev))
    return model, sd


def tokens_of(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def replay(model, steps):
    rp_ = TraceReplayer(model)
    got = {}
    for entries, end in steps:
        out = rp_.step(entries, end)
        r = 0
        for e in entries:
            for _ in e["want"]:
                got.setdefault(e["id"], []).append(out[r].cpu())
                r += 1
    return got


def rel_err(row, ref):
    d = row.to(F64) - ref
    d = d - d.mean()
    return float(d.pow(2).mean().sqrt() / ref.std())


def check_rows(rows, ref, places, dt, strict=2e-4, risky=()):
    """Every position against the oracle: centred difference over the vocabulary, relative to the spread of the logits.
    fp32 is strict; bf16 rounding through the tiny layers reaches a few percent at single positions, so bf16 bounds every
    position at 0.2 and the mean over positions (without the worst tenth: an expert swapped at a nearly tied score moves a
    position by up to that bound) at 0.05 -- a wrong key, edge or state moves positions by far more.
    ``risky``: positions at which the oracle's router scores are nearly tied (``O.close_calls``); 16-bit rounding may
    choose the other expert there, so bf16 leaves them out (fp32 checks them like all others)."""
    assert len(rows) == len(places)
    rels = []
    for row, p in zip(rows, places):
        if dt != torch.float32 and p in risky:
            continue
        rel = rel_err(row, ref[p])
        assert rel <= (strict if dt == torch.float32 else 0.2), f"position {p}: relative error {rel:.2e}"
        rels.append(rel)
    assert len(rels) >= 0.5 * len(places), "too many positions with nearly tied router scores: take another seed"
    kept = sorted(rels)[: max(1, len(rels) - max(1, len(rels) // 10))]        # bf16: the mean without the worst tenth
    assert dt == torch.float32 or sum(kept) / len(kept) <= 0.05, f"mean relative error {sum(kept) / len(kept):.2e}"


# ---- mechanisms alone ------------------------------------------------------------------------------------------------------
@case
@pytest.mark.parametrize("S,W", [(1, 40), (2, 64), (3, 50), (8, 33)])
def test_stream_write_and_read(dev, dt, S, W):
    """Write of a sublayer's output into every stream next to the mixing of the streams (all from the old ones), then the
    normed weighted read; also the mean of two normed branches as the written value, the read alone, the write alone."""
    torch.manual_seed(S)
    N, eps = 6, 1e-4
    X = torch.randn(N, S, W)
    y, y2 = torch.randn(N, W).to(dt), (torch.randn(N, W) * 3).to(dt)
    mix, ow, iw, nw = torch.randn(S, S), torch.randn(S), torch.randn(S), torch.randn(W)
    wa_, wb = torch.randn(W), torch.randn(W)
    x64 = X.to(F64)
    for two in (False, True):
        yv = y.to(F64)
        if two:
            yv = 0.5 * (O.rms(yv, eps) * wa_.to(F64) + O.rms(y2.to(F64), eps) * wb.to(F64))
        new = torch.stack([sum(mix[s, t].to(F64) * x64[:, s] for s in range(S)) + ow[t].to(F64) * yv for t in range(S)], dim=1)
        h_ref = O.rms(sum(iw[s].to(F64) * new[:, s] for s in range(S)), eps) * nw.to(F64)
        Xd = X.clone().to(dev)
        h = hc.hc_step(Xd, y.to(dev), mix.to(dev), ow.to(dev), iw.to(dev), nw.to(dev), eps, dt,
                       y2=y2.to(dev) if two else None, branch_w=(wa_.to(dev), wb.to(dev)) if two else None)
        close(Xd, new, torch.float32, scale=10.0)
        close(h, h_ref, dt, scale=4.0)
        Xw = X.clone().to(dev)                                                       # the write alone
        assert hc.hc_step(Xw, y.to(dev), mix.to(dev), ow.to(dev), eps=eps, out_dtype=dt,
                          y2=y2.to(dev) if two else None, branch_w=(wa_.to(dev), wb.to(dev)) if two else None) is None
        close(Xw, new, torch.float32, scale=10.0)
    Xr = X.clone().to(dev)                                                           # the read alone leaves the streams
    h = hc.hc_step(Xr, in_w=iw.to(dev), norm_w=nw.to(dev), eps=eps, out_dtype=dt)
    assert torch.equal(Xr.cpu(), X)
    close(h, O.rms(sum(iw[s].to(F64) * x64[:, s] for s in range(S)), eps) * nw.to(F64), dt, scale=4.0)


def test_scaled_frequencies_keep_short_waves_slow_long_ones_and_blend_between():
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = O.frequencies({"base": 10000.0, "dims": 32})
    ref = O.frequencies(rot)
    wave = 2 * torch.pi / plain
    assert bool((ref[wave < 16] == plain[wave < 16]).all()) and bool((wave < 16).any())
    assert torch.allclose(ref[wave > 64], plain[wave > 64] / 8.0) and bool((wave > 64).any())
    mid = (wave >= 16) & (wave <= 64)
    assert bool(mid.any()) and bool(((ref[mid] < plain[mid]) & (ref[mid] > plain[mid] / 8.0)).all())
    cos, sin = rp.build_interleaved_rope_cache(50, 32, 10000.0, scaling=(8.0, 1.0, 4.0, 64))
    ang = torch.arange(50, dtype=F64).reshape(-1, 1) * ref.reshape(1, -1)
    assert torch.allclose(cos.to(F64), ang.cos(), atol=1e-6) and torch.allclose(sin.to(F64), ang.sin(), atol=1e-6)


@case
@pytest.mark.parametrize("whole", [False, True])
@pytest.mark.parametrize("H,G,D,Dv,dims", [(4, 2, 16, 8, 8), (3, 3, 6, 6, 6), (2, 1, 34, 5, 2), (8, 2, 64, 64, 32)])
def test_projection_norm_rotation_and_cache_write(dev, dt, whole, H, G, D, Dv, dims):
    """q | k | v columns of a wider row: (whole-projection norm,) rotation of the halves of the first ``dims``
    dimensions at each row's own positions, keys and values into the lines of a paged cache; padding rows write nothing."""
    torch.manual_seed(D)
    B, T, eps, page = 2, 7, 1e-3, 4
    n = H * D + G * (D + Dv)
    big = torch.randn(B, T, n + 13).to(dt)
    rot = {"base": 77.0, "dims": dims, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}}
    cos, sin = rp.build_interleaved_rope_cache(32, dims, 77.0, scaling=(4.0, 1.0, 4.0, 16))
    qw, kw = torch.randn(H * D), torch.randn(G * D)
    starts, cnt, lines = [0, 9], [7, 4], [2, 0]
    table = torch.tensor([[5, 1, 7, 0], [2, 9, 4, 8], [3, 6, 10, 11]], dtype=torch.int32)
    ck = torch.full((12, G, page, D), 9.0, dtype=dt)
    cv = torch.full((12, G, page, Dv), 9.0, dtype=dt)
    ckd, cvd = ck.clone().to(dev), cv.clone().to(dev)
    q = wa.qk_norm_cache_write(big.to(dev)[..., 5: 5 + n], ckd, cvd, torch.tensor(starts, device=dev), H, G, D, Dv, eps,
                               n_new=torch.tensor(cnt, device=dev), seq_ids=torch.tensor(lines, device=dev),
                               normalize=whole, q_weight=qw.to(dev) if whole else None,
                               k_weight=kw.to(dev) if whole else None, rope=(cos.to(dev), sin.to(dev)),
                               rope_layout="halves", whole_norm=whole, block_table=table.to(dev), page_size=page)
    written = torch.zeros(12, page, dtype=torch.bool)
    for b in range(B):
        x = big[b, :, 5: 5 + n].to(F64)
        qq, kk, vv = x[:, : H * D], x[:, H * D: (H + G) * D], x[:, (H + G) * D:]
        if whole:
            qq, kk = O.rms(qq, eps) * qw.to(F64), O.rms(kk, eps) * kw.to(F64)
        pos = torch.arange(starts[b], starts[b] + T)
        qq, kk = O.rotate(qq.reshape(T, H, D), pos, rot), O.rotate(kk.reshape(T, G, D), pos, rot)
        close(q[b, :cnt[b]], qq[:cnt[b]], dt, scale=6.0)
        for t in range(cnt[b]):
            pg, off = int(table[lines[b], (starts[b] + t) // page]), (starts[b] + t) % page
            close(ckd[pg, :, off], kk[t], dt, scale=6.0)
            close(cvd[pg, :, off], vv[t].reshape(G, Dv), dt, scale=6.0)
            written[pg, off] = True
    keep = ~written
    assert torch.equal(ckd.cpu().transpose(1, 2)[keep], ck.transpose(1, 2)[keep])
    assert torch.equal(cvd.cpu().transpose(1, 2)[keep], cv.transpose(1, 2)[keep])


@case
@pytest.mark.parametrize("H,G,D,Dv", [(4, 2, 16, 8), (1, 1, 6, 6), (6, 1, 10, 3), (4, 2, 64, 64), (2, 1, 128, 128)])
def test_softmax_with_a_sink_term(dev, dt, H, G, D, Dv):
    """Attention over the cache whose denominator holds exp(sink_h) once: prompt rows at an offset, a single decoded row,
    a sink far below and far above the scores (no effect / nearly all the mass), and no sink at all."""
    torch.manual_seed(H * D)
    T, scale = 40, D ** -0.5
    q = torch.randn(T, H, D).to(dt)
    k, v = torch.randn(T, G, D).to(dt), torch.randn(T, G, Dv).to(dt)
    ck = torch.zeros(2, G, 48, D, dtype=dt)
    cv = torch.zeros(2, G, 48, Dv, dtype=dt)
    ck[1, :, :T], cv[1, :, :T] = k.transpose(0, 1), v.transpose(0, 1)
    line = torch.tensor([1], device=dev)
    for sink in (torch.randn(H), torch.full((H,), -40.0), torch.full((H,), 9.0), None):
        ref = O.causal_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, sink.to(F64) if sink is not None else None)
        sk = sink.to(dev) if sink is not None else None
        got = wa.window_attention_prefill(q[None, 11:].to(dev), ck.to(dev), cv.to(dev), torch.tensor([11], device=dev), scale,
                                          seq_ids=line, sinks=sk)
        close(got[0], ref[11:], dt, scale=2.0)
        one = wa.window_attention_decode(q[None, T - 1].to(dev), ck.to(dev), cv.to(dev), torch.tensor([T - 1], device=dev),
                                         scale, seq_ids=line, sinks=sk)
        close(one[0], ref[T - 1], dt, scale=2.0)
    none = O.causal_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, None)
    heavy = O.causal_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, torch.full((H,), 9.0, dtype=F64))
    assert float(heavy.abs().max()) < 0.2 * float(none.abs().max())                    # the sink took the mass


@case
@pytest.mark.parametrize("H,D,Dv,dims", [(3, 8, 16, 4), (1, 5, 7, 0), (2, 33, 35, 32), (2, 64, 64, 64), (2, 128, 128, 32)])
def test_retention_in_portions_on_stale_lines(dev, dt, H, D, Dv, dims):
    """q | k | v at odd columns of a wider row, fed in portions (1 token up to more than two chunks) next to a shorter,
    padded row, on lines that hold a stale state: equal to the recurrence over the whole sequence, with both kernels, and
    the state after the step equal to the oracle's."""
    torch.manual_seed(D)
    T = 217
    ld = 2 * H * D + H * Dv + 9
    offs = (2, 2 + H * D + 3, 2 + 2 * H * D + 5)
    raw = (torch.randn(2, T, ld) * 0.7).to(dt)
    decay = [1.0, 0.93, 0.999][:H]
    rot = {"base": 40.0, "dims": dims} if dims else None
    rope = tuple(t.to(dev) for t in rp.build_interleaved_rope_cache(256, dims, 40.0)) if dims else None
    lens = [T, 150]
    refs = []
    for b in range(2):
        x = raw[b, :lens[b]].to(F64)
        pos = torch.arange(lens[b])
        qq = O.rotate(x[:, offs[0]: offs[0] + H * D].reshape(-1, H, D), pos, rot)
        kk = O.rotate(x[:, offs[1]: offs[1] + H * D].reshape(-1, H, D), pos, rot) * D ** -0.5
        refs.append(O.retention(qq, kk, x[:, offs[2]: offs[2] + H * Dv].reshape(-1, H, Dv), torch.tensor(decay, dtype=F64)))
    lines = torch.tensor([2, 0], dtype=torch.int32, device=dev)
    dec = torch.tensor(decay, dtype=torch.float32, device=dev)
    for fn in (rt.retention_scan, rt.retention_chunkwise):
        state = torch.randn(3, H, D, Dv).to(dev)                     # what the lines hold is stale
        got, at = [[], []], [0, 0]
        for size in (1, 2, 63, 64, 65, 22):
            step = torch.zeros(2, size, ld, dtype=dt)
            n_new = []
            for b in range(2):
                n = max(0, min(size, lens[b] - at[b]))
                step[b, :n] = raw[b, at[b]: at[b] + n]
                n_new.append(n)
            out = fn(step.to(dev), offs, dec, state, torch.tensor(at, device=dev), H, D, Dv, D ** -0.5, rope=rope,
                     rope_layout="halves", n_new=torch.tensor(n_new, device=dev), seq_ids=lines)
            for b in range(2):
                got[b].append(out[b, :n_new[b]].cpu())
                assert float(out[b, n_new[b]:].abs().max()) == 0.0 if n_new[b] < size else True
                at[b] += n_new[b]
        for b in range(2):
            close(torch.cat(got[b]), refs[b], torch.float32, scale=30.0 if dt == torch.float32 else 3000.0)


@case
def test_retention_keeps_a_key_from_far_back_and_loses_it_with_a_fast_decay(dev, dt):
    """One key / value pair at position 2 among 300 zeros: with decay 0.999 the query at position 290 still reads 3/4 of
    it, with decay 0.9 nothing; through the chunk-wise kernel in one step and through the token scan after a portion."""
    H, D, Dv, T = 2, 8, 8, 300
    x = torch.zeros(1, T, 2 * H * D + H * Dv, dtype=dt)
    x[0, 2, H * D: 2 * H * D] = 1.0                                 # k at position 2
    x[0, 2, 2 * H * D:] = 2.0                                       # v at position 2
    x[0, 290, : H * D] = 1.0                                        # q at position 290
    dec = torch.tensor([0.999, 0.9], device=dev)
    want = torch.tensor([0.999 ** 288, 0.9 ** 288], dtype=F64) * 2.0 * D * D ** -0.5
    for cut in (T, 100):
        state = torch.randn(1, H, D, Dv).to(dev)
        outs, at = [], 0
        for n in ([T] if cut == T else [100] + [1] * 200):
            fn = rt.retention_chunkwise if n >= 64 else rt.retention_scan
            outs.append(fn(x[:, at: at + n].to(dev), (0, H * D, 2 * H * D), dec, state, torch.tensor([at], device=dev), H, D,
                           Dv, D ** -0.5).cpu())
            at += n
        o = torch.cat(outs, dim=1)[0]
        close(o[290, :, 0], want, torch.float32, scale=5.0)
        assert abs(float(o[290, 0, 0]) - 0.75 * 2.0 * D ** 0.5) < 0.1 and abs(float(o[290, 1, 0])) < 1e-6
        assert float(o[:290].abs().max()) == 0.0


@case
@pytest.mark.parametrize("top,E,shared", [(2, 5, 16), (1, 3, 0), (4, 4, 8)])
def test_sigmoid_router_weights_the_experts_input(dev, dt, top, E, shared):
    """Scores are sigmoids of the logits, the chosen ones are not renormalised and scale the INPUT of their expert (which is
    not the same as scaling its output: the check against the output-weighted sum must fail); a shared expert is added as it
    is.  Both execution paths."""
    torch.manual_seed(E)
    N, W, F = 40, 24, 12
    h = torch.randn(N, W).to(dt)
    m = {"router": {"experts": E, "top": top}, "expert": {"ff": F}}
    if shared:
        m["shared"] = {"ff": shared}
    w = {"router": torch.randn(E, W) * 0.7}
    for n, f in [(f"e{e}.", F) for e in range(E)] + ([("shared.", shared)] if shared else []):
        w[n + "gate"], w[n + "up"], w[n + "down"] = (torch.randn(f, W) * 0.4).to(dt), (torch.randn(f, W) * 0.4).to(dt), (torch.randn(W, f) * 0.4).to(dt)
    w64 = {k: v.to(F64) for k, v in w.items()}
    ref = O.moe(h.to(F64), w64, m)
    s = torch.sigmoid(h.to(F64) @ w64["router"].T)
    idx, wts, _ = ms.route(h.to(dev), w["router"].to(dev), None, top, 1.0, score="sigmoid")
    assert torch.equal(idx.cpu().long().sort(dim=-1).values, torch.topk(s, top).indices.sort(dim=-1).values)
    close(wts, s.gather(1, idx.cpu().long()), torch.float32)
    moe = SparseMoE(W, E, top, F, None, shared_intermediate_size=shared, dtype=dt, device=torch.device(dev),
                    score="sigmoid", weight_on_input=True, shared_gated=False)
    with torch.no_grad():
        moe.router.linear_router.weight.copy_(w["router"])
        moe.experts.gate_up_proj.weight.copy_(torch.stack([torch.cat([w[f"e{e}.gate"].T, w[f"e{e}.up"].T], dim=1) for e in range(E)]))
        moe.experts.down_proj.weight.copy_(torch.stack([w[f"e{e}.down"].T for e in range(E)]))
        if shared:
            moe.shared.gate_up_proj.weight.copy_(torch.cat([w["shared.gate"].T, w["shared.up"].T], dim=1)[None])
            moe.shared.down_proj.weight.copy_(w["shared.down"].T[None])
    out_weighted = sum(s.gather(1, torch.topk(s, top).indices)[:, j: j + 1] * torch.stack(
        [O.glu(h[t: t + 1].to(F64), O.sub(w64, f"e{int(torch.topk(s[t], top).indices[j])}."), O.silu)[0] for t in range(N)])
        for j in range(top)) + (O.glu(h.to(F64), O.sub(w64, "shared."), O.silu) if shared else 0.0)
    assert float((out_weighted - ref).abs().max()) > 0.05
    for path in ("pairs", "sorted"):
        close(moe(h.to(dev), path=path), ref, dt, scale=3.0)


@case
def test_gelu_gated_activation_from_a_wider_row(dev, dt):
    torch.manual_seed(3)
    N, F = 9, 20
    src = (torch.randn(N, 2 * F + 9) * 2).to(dt)
    act = ms.glu_bias(src.to(dev), 2, F + 7, F, act="gelu_tanh")
    s64 = src.to(F64)
    close(act, O.gelu_tanh(s64[:, 2: 2 + F]) * s64[:, F + 7: 2 * F + 7], dt, scale=6.0)
    big = (torch.randn(N, 48) * 2).to(dt)                                          # the vectorised form: aligned columns
    close(ms.glu_bias(big.to(dev), 0, 24, 24, act="gelu_tanh"), O.gelu_tanh(big.to(F64)[:, :24]) * big.to(F64)[:, 24:], dt,
          scale=6.0)


@case
def test_unit_head_norm_with_a_silu_gate_and_no_weight(dev, dt):
    torch.manual_seed(5)
    N, H, Dv = 7, 3, 10
    o = torch.randn(N, H, Dv) * 5
    src = torch.randn(N, H * Dv + 6).to(dt)
    got = ml.head_norm_gate(o.to(dev), src.to(dev), 4, H, Dv, None, 1e-5, True, dt, gate_act="silu")
    close(got, O.rms(o.to(F64), 1e-5).reshape(N, -1) * O.silu(src.to(F64)[:, 4: 4 + H * Dv]), dt, scale=3.0)


def test_cache_and_state_hold_an_entry_per_layer_run():
    cfg = tiny_vufasun()
    model = VufasunInferenceModel(cfg, InferenceConfig(batch_size=2, max_batch_size=2, seq_len=16, max_context_length=16))
    kc = model.init_kv_cache()
    runs = cfg.layer_runs()
    assert runs == [0, 1, 0, 1, 2] and kc.num_layers == 5 and cfg.num_hidden_layers == 5
    a, left, r = cfg.layers[0].mixer, cfg.layers[1].mixer.left, cfg.layers[1].mixer.right
    assert kc.layer(0)[0].shape == (2, a.kv_heads, 16, a.dim) and kc.layer(2)[1].shape == (2, a.kv_heads, 16, a.vdim)
    assert kc.layer(1)[0].shape == (2, left.kv_heads, 16, left.dim)
    assert kc.state(1)["S"].shape == (2, r.heads, r.dim, r.vdim) and kc.state(3)["S"].data_ptr() != kc.state(1)["S"].data_ptr()
    assert kc.layer(0)[0].data_ptr() != kc.layer(2)[0].data_ptr() and 0 not in kc.states and 4 not in kc.states
    seq = model.layer_sequence()
    assert seq[0] is seq[2] and seq[1] is seq[3] and len(seq) == 5


def test_checkpoint_names_round_trip_and_the_fused_projection_layout():
    cfg = tiny_vufasun()
    ic = InferenceConfig(batch_size=1, max_batch_size=1, seq_len=8, max_context_length=8)
    model = VufasunInferenceModel(cfg, ic)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if not name.endswith(("in_proj.weight", "gate_up_proj.weight", "correction")) or "experts" in name or "shared" in name:
                p.copy_(torch.randn_like(p))
    sd = export_vufasun_state_dict(model)
    assert "l1.mix.left.q.norm" in sd and "l0.mix.sink" in sd and "l1.hc2.mix" in sd and "l0.hc2.in" not in sd
    back = convert_vufasun_state_dict(sd, cfg)
    model2 = VufasunInferenceModel(cfg, ic)
    missing, unexpected = model2.load_state_dict(back, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    again = export_vufasun_state_dict(model2)
    assert set(again) == set(sd)
    for k in sd:
        assert torch.equal(again[k], sd[k]), k
    assert VufasunConfig.from_dict(cfg.to_dict(), torch.float32).to_dict() == cfg.to_dict()
    for L in cfg.layers:                                            # every part of the fused projection starts aligned
        cols, n_out = in_proj_columns(L)
        assert n_out % 8 == 0 and all(at % 8 == 0 for at, _ in cols.values())
    with pytest.raises(ValueError):
        VufasunConfig.from_dict(config(layers=[layer("attention", heads=3, kv_heads=2)]))
    with pytest.raises(ValueError):
        VufasunConfig.from_dict(config(layers=[layer("parallel", right=dict(decay=[0.5]))]))
    with pytest.raises(ValueError):
        VufasunConfig.from_dict(config(loop=(1, 9, 2)))
    with pytest.raises(ValueError):
        VufasunConfig.from_dict(config(layers=[{"type": "window", "mixer": {}, "mlp": None}]))


# ---- the model through the framework -----------------------------------------------------------------------------------
@case
@pytest.mark.parametrize("cfg", [config(), ODD, PLAIN, FIVE], ids=["mixed", "odd", "plain", "five"])
def test_prefill_matches_oracle_and_token_by_token_decoding(dev, dt, cfg):
    toks = tokens_of(cfg, 45, 1)
    model, sd = build(cfg, dev, dt, seed=2)                   # a seed without near ties among the router scores
    streams = []
    ref = O.forward(cfg, sd, toks, layer_outputs=streams)
    want = list(range(45))
    seen = []
    model.layer_probe = lambda i, x: seen.append(x.detach().to("cpu", F64))
    whole = replay(model, [([{"id": "a", "tokens": toks, "want": want}], ["a"])])["a"]
    model.layer_probe = None
    risky = O.close_calls(cfg, sd, toks)
    check_rows(whole, ref, want, dt, risky=risky)
    assert len(seen) == len(streams) == len(O.layer_runs(cfg))
    rows = [p for p in want if dt == torch.float32 or p not in risky]      # bf16 may swap an expert at a nearly tied score
    for got, exp in zip(seen, streams):                       # the sum of the streams after every layer run
        assert float((got[0] - exp)[rows].abs().max()) <= (2e-3 if dt == torch.float32 else 0.08 * float(exp.abs().max()) + 0.5)
    steps = [([{"id": "b", "tokens": toks[:1], "want": [0]}], [])]
    steps += [([{"id": "b", "tokens": [t], "want": [0]}], []) for t in toks[1:]]
    check_rows(replay(model, steps)["b"], ref, want, dt, risky=risky)


@case
@pytest.mark.parametrize("portion", [2, 5, 16, 70])
def test_portions_of_a_prompt(dev, dt, portion):
    """Portions of 2 .. 70 tokens (the last size takes the chunk-wise recurrence, whose second portion starts inside a
    chunk of the sequence), every position checked."""
    cfg = config()
    n = 41 if portion < 70 else 150
    toks = tokens_of(cfg, n, 6)
    model, sd = build(cfg, dev, dt, seq_len=160)
    ref = O.forward(cfg, sd, toks)
    steps, places = [], []
    for lo in range(0, n, portion):
        part = toks[lo:lo + portion]
        steps.append(([{"id": "p", "tokens": part, "want": list(range(len(part)))}], []))
        places += list(range(lo, lo + len(part)))
    check_rows(replay(model, steps)["p"], ref, places, dt, risky=O.close_calls(cfg, sd, toks))


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
    # two new requests take the lines that a and c gave back: stale keys and a stale retention state lie in them
    steps.append(([{"id": k, "tokens": toks[k][:lens[k]], "want": [0, lens[k] - 1]} for k in "de"], []))
    for s in range(6):
        steps.append(([{"id": k, "tokens": [toks[k][lens[k] + s]], "want": [0]} for k in "de"], []))
    got = replay(model, steps)
    risky = {k: O.close_calls(cfg, sd, v) for k, v in toks.items()}
    check_rows(got["a"], ref["a"], [0], dt)
    for k in "bc":
        check_rows(got[k], ref[k], [lens[k] - 1, lens[k], lens[k] + 1, lens[k] + 2], dt, risky=risky[k])
    for k in "de":
        check_rows(got[k], ref[k], [0, lens[k] - 1] + [lens[k] + s for s in range(6)], dt, risky=risky[k])


@case
def test_long_decoding_over_a_small_page_pool(dev, dt):
    """85 decoded tokens after a prompt of 5 on pages of 8 rows from a pool that two lines could not both fill: every page
    border is crossed while decoding, and the recurrence runs 85 single steps."""
    cfg = config()
    toks = tokens_of(cfg, 90, 4)
    model, sd = build(cfg, dev, dt, lines=2, paged=True, pages=14, page_size=8)
    ref = O.forward(cfg, sd, toks)
    steps = [([{"id": "x", "tokens": toks[:5], "want": [4]}], [])]
    steps += [([{"id": "x", "tokens": [t], "want": [0]}], []) for t in toks[5:]]
    check_rows(replay(model, steps)["x"], ref, list(range(4, 90)), dt, risky=O.close_calls(cfg, sd, toks))
    # the pages go back to the pool and a second request gets them in another order
    steps = [([{"id": "y", "tokens": toks[20:50], "want": [29]}], ["x"])]
    steps += [([{"id": "y", "tokens": [t], "want": [0]}], []) for t in toks[50:60]]
    check_rows(replay_on(model, steps)["y"], O.forward(cfg, sd, toks[20:60]), list(range(29, 40)), dt,
               risky=O.close_calls(cfg, sd, toks[20:60]))


def replay_on(model, steps):
    """As ``replay`` on a model whose cache was used before: a fresh replayer over the same cache (all lines free)."""
    model.kv_cache.reset() if model.kv_cache.pool is not None else None
    return replay(model, steps)


@case
def test_a_key_far_back_and_the_sink_both_show_in_the_logits(dev, dt):
    """One sink-attention layer: only token id 5, at position 1, has a non-zero embedding column 1, which the first key
    dimension reads, while the first query dimension reads column 0, shared by all tokens: that key takes most of the
    softmax mass of every later query, 280 positions on as well (the oracle says by how much the logits move without it),
    in a long prompt step, in a portion at an offset and while decoding.  The sink's share shows at the first token, whose
    only other term is its own key."""
    cfg = config(layers=[layer("attention", mlp=None, heads=2, kv_heads=1, scale=1.0, rot={"base": 10000.0, "dims": 4})],
                 streams=2, loop=None)
    sd = O.random_weights(cfg, seed=3)
    D = 16
    sd["embed"][:, 0], sd["embed"][:, 1] = 1.0, 0.0
    sd["embed"][5, 1] = 4.0
    sd["l0.norm1"][:] = 1.0
    sd["l0.mix.k"][D - 1] = 0.0                                  # an un-rotated dimension carries the planted score
    sd["l0.mix.k"][D - 1, 1] = 6.0
    for h in range(2):
        sd["l0.mix.q"][h * D + D - 1] = 0.0
        sd["l0.mix.q"][h * D + D - 1, 0] = 3.0
    sd["l0.mix.sink"][:] = 2.0
    toks = [t if t != 5 else 6 for t in tokens_of(cfg, 300, 9)]
    toks[1] = 5
    ref = O.forward(cfg, sd, toks)
    moved = list(toks)
    moved[1] = 6
    assert rel_err(O.forward(cfg, sd, moved)[290].float(), ref[290]) > 0.1
    no_sink = dict(sd)
    no_sink["l0.mix.sink"] = torch.full((2,), -30.0)
    assert rel_err(O.forward(cfg, no_sink, toks[:1])[0].float(), ref[0]) > 0.02     # the first token shares with the sink alone
    model, _ = build(cfg, dev, dt, sd=sd, seq_len=320, lines=2)
    steps = [([{"id": "f", "tokens": toks[:200], "want": [0, 1, 2, 199]}], []),
             ([{"id": "f", "tokens": toks[200:280], "want": [0, 79]}], [])]
    steps += [([{"id": "f", "tokens": [t], "want": [0]}], []) for t in toks[280:]]
    check_rows(replay(model, steps)["f"], ref, [0, 1, 2, 199, 200, 279] + list(range(280, 300)), dt, strict=1e-3)


@case
def test_a_token_far_back_lives_on_in_the_retention_state(dev, dt):
    """One parallel layer whose retention heads decay slowly: moving one early token changes the logits 280 positions later
    (the oracle says by how much), through the chunk-wise step, a portion at an offset and the single-token steps."""
    cfg = config(layers=[layer("parallel", mlp=None, right=dict(decay=[0.9995, 0.999, 0.9999]))], streams=2, loop=None)
    sd = O.random_weights(cfg, seed=4)
    sd["l0.mix.left.out"][:] = 0.05                              # the attention branch hardly speaks
    sd["l0.mix.right.k"] *= 0.05                                 # every token writes little ...
    sd["embed"][:, 1] = 0.0
    sd["embed"][5, 1] = 8.0
    sd["l0.mix.right.k"][:, 1] = 2.0                             # ... but token 5, at position 1, writes a lot
    sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    toks = [t if t != 5 else 6 for t in tokens_of(cfg, 300, 9)]
    toks[1] = 5
    ref = O.forward(cfg, sd, toks)
    moved = list(toks)
    moved[1] = 6
    assert rel_err(O.forward(cfg, sd, moved)[290].float(), ref[290]) > 0.1
    model, _ = build(cfg, dev, dt, sd=sd, seq_len=320, lines=2)
    steps = [([{"id": "f", "tokens": toks[:200], "want": [0, 1, 2, 199]}], []),
             ([{"id": "f", "tokens": toks[200:280], "want": [0, 79]}], [])]
    steps += [([{"id": "f", "tokens": [t], "want": [0]}], []) for t in toks[280:]]
    check_rows(replay(model, steps)["f"], ref, [0, 1, 2, 199, 200, 279] + list(range(280, 300)), dt, strict=1e-3)


@case
def test_sizes_of_the_tensor_core_and_wide_register_kernels_through_the_model(dev, dt):
    """Key sizes 64 / 128 (the attention's tensor-core kernels in bf16, the widest register slices of the recurrence),
    grouped heads, four streams, prompts of 70 and 130 tokens in one batch (in bf16 the sink-free left branch then runs on
    the tcgen05 flash-attention kernel, next to a padded row), a portion at an offset, decoding."""
    big_left = dict(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, rot={"base": 1e4, "dims": 64})
    cfg = config(layers=[layer("parallel", left=big_left, right=dict(heads=2, dim=128, vdim=64, decay=[0.98, 0.999],
                                                                      rot={"base": 1e4, "dims": 128}), mlp=None),
                         layer("attention", heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, rot={"base": 1e4, "dims": 32}, mlp=MOE),
                         layer("attention", heads=2, kv_heads=1, dim=128, vdim=64, scale=0.09, rot={"base": 1e4, "dims": 64})],
                 width=64, vocab=80, streams=4, loop=(0, 1, 2))
    model, sd = build(cfg, dev, dt, lines=2, seq_len=200)
    a, b = tokens_of(cfg, 170, 51), tokens_of(cfg, 80, 52)
    ra, rb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    steps = [([{"id": "a", "tokens": a[:130], "want": [0, 47, 48, 129]}, {"id": "b", "tokens": b[:70], "want": [69]}], []),
             ([{"id": "a", "tokens": a[130:160], "want": [0, 29]}], [])]
    steps += [([{"id": "a", "tokens": [a[160 + s]], "want": [0]}, {"id": "b", "tokens": [b[70 + s]], "want": [0]}], [])
              for s in range(6)]
    got = replay(model, steps)
    check_rows(got["a"], ra, [0, 47, 48, 129, 130, 159] + list(range(160, 166)), dt, strict=1e-3, risky=O.close_calls(cfg, sd, a))
    check_rows(got["b"], rb, [69] + list(range(70, 76)), dt, strict=1e-3, risky=O.close_calls(cfg, sd, b))


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
    best = [O.forward(cfg, sd, p)[-1].topk(3).indices.tolist() for p in prompts]      # bf16 may swap near-equal logits
    for b, p in enumerate(prompts):
        got = out[b, len(p):len(p) + 6].tolist()
        assert got == want[b] or not strict, (got, want[b])
        assert got[0] in best[b]
    from neuronx_distributed_llama3_2_b200.inference.continuous_batching import ContinuousBatcher

    model2, _ = build(cfg, dev, dt, lines=2, sd=sd, paged=True, pages=9, page_size=4, seq_len=32)
    cb = ContinuousBatcher(model2)
    rids = [cb.submit(torch.tensor(p), 6) for p in prompts]
    res = cb.run()
    for rid, w, top3 in zip(rids, want, best):
        assert res[rid][:6] == w or not strict, (res[rid], w)
        assert res[rid][0] in top3


@case
def test_runner_buckets_match_oracle_greedy(dev, dt):
    from neuronx_distributed_llama3_2_b200.inference import VufasunRunner

    cfg = config()
    sd = O.random_weights(cfg, seed=12)
    vc = VufasunConfig.from_dict(cfg, torch_dtype=dt).with_checkpoint_shapes(sd)
    ic = InferenceConfig(batch_size=3, max_context_length=32, seq_len=64, buckets=[16, 32], max_new_tokens=5,
                         use_cuda_graphs=dev == "cuda")
    runner = VufasunRunner(vc, ic, checkpoint_loader=lambda: convert_vufasun_state_dict(sd, vc), device=torch.device(dev))
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
        assert got[0] in O.forward(cfg, sd, p)[-1].topk(3).indices.tolist()
        assert got == w or dt != torch.float32, (got, w)


def test_registry_and_command_line_replay(tmp_path):
    """``bin/trace_run`` on a model directory: family chosen from config.json, sink and norm tensors found in the
    checkpoint, steps on stdin, logits in files."""
    from safetensors.torch import save_file

    from neuronx_distributed_llama3_2_b200.inference.registry import families

    assert "vufasun" in families()
    cfg = json.loads(json.dumps(ODD))
    sd = O.random_weights(cfg, seed=8)
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in sd.items()}, str(mdir / "model.safetensors"))
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

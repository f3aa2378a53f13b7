"""Serving throughput of the Gekazen family next to the closest existing family (the Mixtral-style MoE decoder) at equal
layer sizes, plus the like-for-like kernels of the two in isolation with their roofline fractions.

Random-init bf16 weights, synthetic token ids.  Every number is CUDA-event time on the launching stream after >= 3
warm-up runs, with a write through a buffer larger than L2 between timed runs; peaks come from ``MEASURED_PEAKS.json``
(measured copy bandwidth and cuBLAS bf16 throughput) when the file is present.
"""
from __future__ import annotations

import ctypes
import json
import os
import statistics
from typing import Callable, Dict, List

import torch

from ..models.gekazen import GekazenConfig
from ..models.mixtral import MixtralConfig
from ..ops import _lib
from ..ops import activation as act_ops
from ..ops import attention as attn_ops
from ..ops import moe_sparse  # noqa: F401
from ..ops import norm as norm_ops
from ..ops import window_attention as wa
from .config import InferenceConfig
from .model import GekazenInferenceModel, MixtralInferenceModel

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

SIZES = [
    dict(name="w2048-d128", width=2048, layers=4, heads=16, kv_heads=4, dim=128, experts=8, top=2, ff=2048, window=1024,
         keep_first=4, prefill_batch=4, prompt=2048, decode_batch=16),
    dict(name="w4096-d128", width=4096, layers=2, heads=32, kv_heads=8, dim=128, experts=8, top=2, ff=4096, window=2048,
         keep_first=4, prefill_batch=2, prompt=4096, decode_batch=32),
    dict(name="w1024-d64", width=1024, layers=4, heads=16, kv_heads=16, dim=64, experts=16, top=4, ff=512, window=512,
         keep_first=2, prefill_batch=8, prompt=1024, decode_batch=64),
]
VOCAB = 8192


def peaks() -> Dict[str, float]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class _Timer:
    def __init__(self, device):
        self.flush = torch.empty(192 << 20, dtype=torch.uint8, device=device)      # > 126 MB of L2

    def __call__(self, fn: Callable[[], None], steps: int, warmup: int) -> float:
        """Median milliseconds of ``fn`` over ``steps`` runs."""
        for _ in range(max(warmup, 3)):
            fn()
        times = []
        for _ in range(steps):
            _lib.lib().nxd_l2_flush(_lib.ptr(self.flush), ctypes.c_size_t(self.flush.numel()), _lib.stream_ptr())
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return statistics.median(times)


def gekazen_config(s: dict) -> GekazenConfig:
    layer = {"type": "attention",
             "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                       "scale": s["dim"] ** -0.5, "mask": {"size": s["window"], "keep_first": s["keep_first"]}},
             "mlp": {"kind": "moe", "expert": {"ff": s["ff"], "limit": 7.0},
                     "router": {"experts": s["experts"], "identity": 0, "scale": 1.0, "top": s["top"]}, "shared": None}}
    return GekazenConfig.from_dict({"architecture": "Gekazen", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5},
                                    "layers": [layer] * s["layers"]}, torch_dtype=torch.bfloat16)


def mixtral_config(s: dict) -> MixtralConfig:
    return MixtralConfig(vocab_size=VOCAB, hidden_size=s["width"], intermediate_size=s["ff"],
                         num_hidden_layers=s["layers"], num_attention_heads=s["heads"],
                         num_key_value_heads=s["kv_heads"], head_dim=s["dim"], rope_scaling=None,
                         max_position_embeddings=s["prompt"] + 64, tie_word_embeddings=False,
                         num_local_experts=s["experts"], num_experts_per_tok=s["top"], capacity_factor=None,
                         sequence_parallel_enabled=False, torch_dtype=torch.bfloat16)


def _serve(model, s: dict, timer: _Timer, steps: int, warmup: int, dev) -> Dict[str, float]:
    Bp, T, Bd = s["prefill_batch"], s["prompt"], s["decode_batch"]
    ids = torch.randint(1, VOCAB, (Bp, T), device=dev)
    pos = torch.arange(T, device=dev).unsqueeze(0).expand(Bp, T).contiguous()
    lines = torch.arange(Bp, dtype=torch.int32, device=dev)
    last = torch.full((Bp,), T - 1, device=dev)
    pre = timer(lambda: model.forward_infer(ids, pos, seq_ids=lines, last_token_index=last), steps, warmup)
    # every decode line holds T tokens of context: fill the lines Bp at a time, then step at position T
    for lo in range(0, Bd, Bp):
        n = min(Bp, Bd - lo)
        model.forward_infer(ids[:n], pos[:n], seq_ids=torch.arange(lo, lo + n, dtype=torch.int32, device=dev),
                            last_token_index=last[:n])
    tok = torch.randint(1, VOCAB, (Bd, 1), device=dev)
    dpos = torch.full((Bd, 1), T, device=dev)
    dl = torch.arange(Bd, dtype=torch.int32, device=dev)
    dec = timer(lambda: model.forward_infer(tok, dpos, seq_ids=dl), steps, warmup)
    return {"prefill_ms": pre, "prefill_tokens_per_s": Bp * T / pre * 1e3, "decode_ms": dec,
            "decode_tokens_per_s": Bd / dec * 1e3}


def serve_case(s: dict, steps: int, warmup: int, dev) -> dict:
    timer = _Timer(dev)
    out = {"size": {k: v for k, v in s.items()}}
    ic = dict(batch_size=s["decode_batch"], max_batch_size=s["decode_batch"], max_context_length=s["prompt"],
              seq_len=s["prompt"] + 64, is_continuous_batching=True, use_cuda_graphs=False)
    for name, make in (("gekazen", lambda: GekazenInferenceModel(gekazen_config(s), InferenceConfig(**ic), device=dev)),
                       ("mixtral", lambda: MixtralInferenceModel(mixtral_config(s), InferenceConfig(**ic), device=dev))):
        torch.manual_seed(0)
        model = make()
        model.init_kv_cache(device=dev)
        out[name] = _serve(model, s, timer, steps, warmup, dev)
        del model
        torch.cuda.empty_cache()
    out["gekazen_over_mixtral"] = {k: out["gekazen"][k] / out["mixtral"][k]
                                   for k in ("prefill_tokens_per_s", "decode_tokens_per_s")}
    return out


def kernel_cases(s: dict, steps: int, warmup: int, dev) -> List[dict]:
    """The attention and norm kernels of both families on the shapes of ``s``, alone, with roofline fractions."""
    pk = peaks()
    timer = _Timer(dev)
    B, T, H, G, D = s["prefill_batch"], s["prompt"], s["heads"], s["kv_heads"], s["dim"]
    W, win, keep, Bd = s["width"], s["window"], s["keep_first"], s["decode_batch"]
    bf = torch.bfloat16
    rows = []

    def row(kernel, like, ms, flops=None, nbytes=None):
        r = {"kernel": kernel, "like": like, "ms": ms}
        if flops is not None:
            r["tflops"] = flops / ms / 1e9
            r["of_peak"] = r["tflops"] / pk["bf16_tflops"]
        if nbytes is not None:
            r["gbs"] = nbytes / ms / 1e6
            r["of_peak"] = r["gbs"] / pk["hbm_gbs"]
        r["peak"] = pk["source"]
        rows.append(r)

    # prefill attention: visible (query, key) pairs only are counted as work
    q = torch.randn(B, T, H, D, device=dev, dtype=bf)
    ck = torch.randn(max(B, Bd), G, T + 64, D, device=dev, dtype=bf)
    cv = torch.randn(max(B, Bd), G, T + 64, D, device=dev, dtype=bf)
    zero = torch.zeros(B, dtype=torch.int32, device=dev)
    slopes = wa.distance_slopes(H, device=dev)
    i = torch.arange(T).reshape(T, 1)
    j = torch.arange(T).reshape(1, T)
    pairs_win = int(((j <= i) & ((i - j < win) | (j < keep))).sum())
    pairs_causal = T * (T + 1) // 2
    ms = timer(lambda: wa.window_attention_prefill(q, ck, cv, zero, D ** -0.5, win, keep, slopes), steps, warmup)
    row("window_attn_prefill_mma (window, kept tokens, bias)", "prefill attention", ms, flops=4.0 * D * pairs_win * H * B)
    ms = timer(lambda: wa.window_attention_prefill(q, ck, cv, zero, D ** -0.5, None, 0, slopes), steps, warmup)
    row("window_attn_prefill_mma (plain causal, bias)", "prefill attention", ms, flops=4.0 * D * pairs_causal * H * B)
    qh = q.permute(0, 2, 1, 3)
    kh, vh = ck[:B, :, :T], cv[:B, :, :T]
    ms = timer(lambda: wa.window_attention_tc(qh, kh, vh, D ** -0.5, win, keep, slopes), steps, warmup)
    row("windowed flash attention (tcgen05; window, kept tokens, bias)", "prefill attention", ms,
        flops=4.0 * D * pairs_win * H * B)
    ms = timer(lambda: wa.window_attention_tc(qh, kh, vh, D ** -0.5, None, 0, slopes), steps, warmup)
    row("windowed flash attention (tcgen05; plain causal, bias)", "prefill attention", ms,
        flops=4.0 * D * pairs_causal * H * B)
    ms = timer(lambda: attn_ops.flash_attn_func(qh, kh, vh, causal=True), steps, warmup)
    row("flash attention forward (tcgen05, plain causal)", "prefill attention", ms, flops=4.0 * D * pairs_causal * H * B)
    # decode attention: bytes of the cache rows that have to be read
    qd = torch.randn(Bd, H, D, device=dev, dtype=bf)
    posd = torch.full((Bd,), T, dtype=torch.int32, device=dev)
    seen = min(T + 1, win) + min(keep, max(T + 1 - win, 0))
    ms = timer(lambda: wa.window_attention_decode(qd, ck, cv, posd, D ** -0.5, win, keep, slopes), steps, warmup)
    row("window_attn_decode", "decode attention", ms, nbytes=2.0 * seen * G * 2 * D * Bd)
    lens = torch.full((Bd,), T + 1, dtype=torch.int32, device=dev)
    ms = timer(lambda: attn_ops.decode_attention(qd, ck, cv, lens), steps, warmup)
    row("decode attention (full context)", "decode attention", ms, nbytes=2.0 * (T + 1) * G * 2 * D * Bd)
    # norms on the prefill activations
    N = B * T
    x32 = torch.randn(N, W, device=dev)
    y = torch.randn(N, W, device=dev, dtype=bf)
    w32 = torch.zeros(W, device=dev)
    ms = timer(lambda: norm_ops.post_norm_residual_(x32, y, w32, 1e-5, bf), steps, warmup)
    row("post-norm + fp32 residual (+ bf16 copy)", "norm", ms, nbytes=float(N * W * (2 + 4 + 4 + 2)))
    xb, rb, wb = y, torch.randn(N, W, device=dev, dtype=bf), torch.ones(W, device=dev, dtype=bf)
    ms = timer(lambda: norm_ops.fused_add_rms_norm(xb, rb, wb, 1e-5), steps, warmup)
    row("fused add + RMSNorm (bf16 residual)", "norm", ms, nbytes=float(N * W * 2 * 4))
    # q/k normalisation + cache write against rotation + cache write
    n_out = (H + 2 * G) * D
    qkv = torch.randn(B, T, n_out, device=dev, dtype=bf)
    ms = timer(lambda: wa.qk_norm_cache_write(qkv, ck, cv, zero, H, G, D, D, 1e-5), steps, warmup)
    row("unit-RMS q/k + cache write", "projection epilogue", ms, nbytes=float(2 * N * n_out * 2))
    return rows


def run(steps: int = 10, warmup: int = 3, device=None, sizes=None) -> dict:
    dev = device or torch.device("cuda", torch.cuda.current_device())
    before = _lib.kernel_launches()
    out = {"metric": "Gekazen vs Mixtral-style decoder, serving throughput at equal layer sizes", "dtype": "bf16",
           "data": "synthetic token ids, random-init weights", "steps": steps, "warmup": max(warmup, 3),
           "l2": "192 MB written between timed runs", "peaks": peaks(), "cases": [], "kernels": {}}
    for s in (sizes or SIZES):
        out["cases"].append(serve_case(s, steps, warmup, dev))
        out["kernels"][s["name"]] = kernel_cases(s, steps, warmup, dev)
    out["gpu_launches"] = _lib.kernel_launches() - before
    return out


# ---- Rasodra (chunked attention + recurrent matrix memory + latent attention, dense feed-forward) next to the Llama
# decoder at equal width, heads, head size, layer count and feed-forward parameters -----------------------------------------
HYBRID_SIZES = [
    dict(name="w2048", width=2048, heads=16, kv_heads=4, dim=128, chunk=1024, rec_heads=4, rec_dim=128, rec_vdim=256,
         lat_dim=128, lat_rot=64, lat_vdim=128, rank=512, ff=8192, prefill_batch=4, prompt=2048, decode_batch=16),
    dict(name="w4096", width=4096, heads=32, kv_heads=8, dim=128, chunk=2048, rec_heads=8, rec_dim=256, rec_vdim=512,
         lat_dim=128, lat_rot=64, lat_vdim=128, rank=512, ff=12288, prefill_batch=2, prompt=4096, decode_batch=32),
    dict(name="w1024", width=1024, heads=16, kv_heads=4, dim=64, chunk=512, rec_heads=4, rec_dim=64, rec_vdim=128,
         lat_dim=64, lat_rot=32, lat_vdim=64, rank=256, ff=4096, prefill_batch=8, prompt=1024, decode_batch=64),
]


def rasodra_config(s: dict):
    from ..models.rasodra import RasodraConfig

    ff = {"kind": "dense", "ff": s["ff"]}
    att = {"type": "attention", "mlp": ff,
           "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                     "scale": s["dim"] ** -0.5, "mask": {"size": s["chunk"]}, "rot": {"dims": s["dim"], "base": 500000.0}}}
    rec = {"type": "mlstm", "mlp": None,
           "mixer": {"heads": s["rec_heads"], "dim": s["rec_dim"], "vdim": s["rec_vdim"], "gate_cap": 15.0}}
    lat = {"type": "latent_attention", "mlp": ff,
           "mixer": {"heads": s["heads"], "dim": s["lat_dim"], "rot_dim": s["lat_rot"], "vdim": s["lat_vdim"],
                     "kv_rank": s["rank"], "scale": (s["lat_dim"] + s["lat_rot"]) ** -0.5,
                     "rot": {"dims": s["lat_rot"], "base": 1000000.0}}}
    return RasodraConfig.from_dict({"architecture": "Rasodra", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6},
                                    "layers": [att, rec, lat, lat]}, torch_dtype=torch.bfloat16)


def llama_like_config(s: dict):
    from ..models.llama import LlamaConfig

    # three matrices of (width x i) against two of (width x ff): i = 2/3 ff keeps the feed-forward parameters equal
    inter = (2 * s["ff"] // 3 + 127) // 128 * 128
    return LlamaConfig(vocab_size=VOCAB, hidden_size=s["width"], intermediate_size=inter, num_hidden_layers=4,
                       num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"], head_dim=s["dim"],
                       rope_scaling=None, max_position_embeddings=s["prompt"] + 64, tie_word_embeddings=False,
                       sequence_parallel_enabled=False, torch_dtype=torch.bfloat16)


def hybrid_serve_case(s: dict, steps: int, warmup: int, dev) -> dict:
    from .hybrid import RasodraInferenceModel
    from .model import LlamaInferenceModel

    timer = _Timer(dev)
    out = {"size": dict(s)}
    ic = dict(batch_size=s["decode_batch"], max_batch_size=s["decode_batch"], max_context_length=s["prompt"],
              seq_len=s["prompt"] + 64, is_continuous_batching=True, use_cuda_graphs=False)
    for name, make in (("rasodra", lambda: RasodraInferenceModel(rasodra_config(s), InferenceConfig(**ic), device=dev)),
                       ("llama", lambda: LlamaInferenceModel(llama_like_config(s), InferenceConfig(**ic), device=dev))):
        torch.manual_seed(0)
        model = make()
        model.init_kv_cache(device=dev)
        out[name] = _serve(model, s, timer, steps, warmup, dev)
        del model
        torch.cuda.empty_cache()
    out["rasodra_over_llama"] = {k: out["rasodra"][k] / out["llama"][k]
                                 for k in ("prefill_tokens_per_s", "decode_tokens_per_s")}
    return out


def hybrid_kernel_cases(s: dict, steps: int, warmup: int, dev) -> List[dict]:
    """The mixers' own kernels on the shapes of ``s``, alone, with roofline fractions, next to the like kernel of the
    Llama decoder (flash attention forward, decode attention over the full context, fused add + RMSNorm)."""
    from ..ops import latent_attention as la
    from ..ops import mlstm as ml
    from ..ops import rope as rope_ops

    pk = peaks()
    timer = _Timer(dev)
    bf = torch.bfloat16
    B, T, H, G, D, W, Bd = s["prefill_batch"], s["prompt"], s["heads"], s["kv_heads"], s["dim"], s["width"], s["decode_batch"]
    rows = []

    def row(kernel, like, ms, flops=None, nbytes=None):
        r = {"kernel": kernel, "like": like, "ms": ms, "peak": pk["source"]}
        if flops is not None:
            r["tflops"] = flops / ms / 1e9
            r["of_peak"] = r["tflops"] / pk["bf16_tflops"]
        if nbytes is not None:
            r["gbs"] = nbytes / ms / 1e6
            r["of_peak"] = r["gbs"] / pk["hbm_gbs"]
        rows.append(r)

    S = T + 64
    zero = torch.zeros(B, dtype=torch.int32, device=dev)
    i = torch.arange(T).reshape(T, 1)
    j = torch.arange(T).reshape(1, T)
    pairs_chunk = int(((j <= i) & (i // s["chunk"] == j // s["chunk"])).sum())
    pairs_causal = T * (T + 1) // 2
    # chunked attention, prefill and decode
    q = torch.randn(B, T, H, D, device=dev, dtype=bf)
    ck = torch.randn(max(B, Bd), G, S, D, device=dev, dtype=bf)
    cv = torch.randn(max(B, Bd), G, S, D, device=dev, dtype=bf)
    ms = timer(lambda: wa.window_attention_prefill(q, ck, cv, zero, D ** -0.5, chunk=s["chunk"]), steps, warmup)
    row("chunked attention prefill (mma.sync, over the cache)", "prefill attention", ms, flops=4.0 * D * pairs_chunk * H * B)
    if T % s["chunk"] == 0:
        nch, size = T // s["chunk"], s["chunk"]
        qx = q.reshape(B * nch, size, H, D).permute(0, 2, 1, 3)
        kx = ck[:B, :, :T].transpose(1, 2).contiguous().reshape(B * nch, size, G, D).permute(0, 2, 1, 3)
        vx = cv[:B, :, :T].transpose(1, 2).contiguous().reshape(B * nch, size, G, D).permute(0, 2, 1, 3)
        ms = timer(lambda: attn_ops.flash_attn_func(qx, kx, vx, softmax_scale=D ** -0.5, causal=True), steps, warmup)
        row("chunked attention prefill (tcgen05, chunks as batch rows: prompts from position 0)", "prefill attention", ms,
            flops=4.0 * D * pairs_chunk * H * B)
    qh, kh, vh = q.permute(0, 2, 1, 3), ck[:B, :, :T], cv[:B, :, :T]
    ms = timer(lambda: attn_ops.flash_attn_func(qh, kh, vh, causal=True), steps, warmup)
    row("flash attention forward (tcgen05, plain causal)", "prefill attention", ms, flops=4.0 * D * pairs_causal * H * B)
    qd = torch.randn(Bd, H, D, device=dev, dtype=bf)
    posd = torch.full((Bd,), T, dtype=torch.int32, device=dev)
    seen = T % s["chunk"] + 1
    ms = timer(lambda: wa.window_attention_decode(qd, ck, cv, posd, D ** -0.5, chunk=s["chunk"]), steps, warmup)
    row("chunked attention decode (rows of the query's chunk)", "decode attention", ms, nbytes=2.0 * seen * G * 2 * D * Bd)
    posm = torch.full((Bd,), T - 1, dtype=torch.int32, device=dev)
    ms = timer(lambda: wa.window_attention_decode(qd, ck, cv, posm, D ** -0.5, chunk=s["chunk"]), steps, warmup)
    row("chunked attention decode (a full chunk)", "decode attention", ms,
        nbytes=2.0 * ((T - 1) % s["chunk"] + 1) * G * 2 * D * Bd)
    lens = torch.full((Bd,), T + 1, dtype=torch.int32, device=dev)
    ms = timer(lambda: attn_ops.decode_attention(qd, ck, cv, lens), steps, warmup)
    row("decode attention (full context)", "decode attention", ms, nbytes=2.0 * (T + 1) * G * 2 * D * Bd)
    del ck, cv
    # latent attention: prefill over expanded heads, decode over the latent rows
    Dn, Dr, Dv, R = s["lat_dim"], s["lat_rot"], s["lat_vdim"], s["rank"]
    ql = torch.randn(B, T, H, Dn + Dr, device=dev, dtype=bf)
    kx = torch.randn(B, T, H, Dn + Dr, device=dev, dtype=bf).permute(0, 2, 1, 3)
    vx = torch.randn(B, T, H, Dv, device=dev, dtype=bf).permute(0, 2, 1, 3)
    sinks = torch.zeros(H, device=dev)
    ms = timer(lambda: wa.window_attention_prefill(ql, kx, vx, zero, 0.07, sinks=sinks), steps, warmup)
    row("latent attention prefill (expanded heads, sink)", "prefill attention", ms,
        flops=2.0 * (Dn + Dr + Dv) * pairs_causal * H * B)
    cl = torch.randn(Bd, 1, S, R + Dr, device=dev, dtype=bf)
    qa = torch.randn(Bd, H, R + Dr, device=dev, dtype=bf)
    ms = timer(lambda: wa.window_attention_decode(qa, cl, cl[..., :R], posd, 0.07, sinks=sinks), steps, warmup)
    row("latent attention decode (absorbed queries over latent rows)", "decode attention", ms,
        nbytes=2.0 * (T + 1) * (R + Dr) * Bd)
    proj = torch.randn(B, T, H * (Dn + Dr) + R + Dr, device=dev, dtype=bf)
    tables = rope_ops.build_interleaved_rope_cache(S, Dr, 1e6, device=dev)
    wn = torch.ones(R, device=dev)
    ms = timer(lambda: la.latent_prep(proj, 0, H * (Dn + Dr), None, cl, wn, tables, zero, H, Dn, Dr, R, 1e-6), steps, warmup)
    row("latent norm + rotations + cache row", "projection epilogue", ms,
        nbytes=2.0 * B * T * (2 * H * (Dn + Dr) + 2 * (R + Dr)))
    del cl
    # recurrent matrix memory
    Hr, Dk, Dvr = s["rec_heads"], s["rec_dim"], s["rec_vdim"]
    ld = 2 * Hr * Dk + 2 * Hr * Dvr
    pr = torch.randn(B, T, ld, device=dev, dtype=bf) * 0.3
    gi = torch.randn(B * T, Hr, device=dev)
    gf = -torch.rand(B * T, Hr, device=dev) * 0.1
    st = (torch.zeros(Bd, Hr, Dk, Dvr, device=dev), torch.zeros(Bd, Hr, Dk, device=dev), torch.zeros(Bd, Hr, device=dev))
    ms = timer(lambda: ml.mlstm_scan(pr, (0, Hr * Dk, 2 * Hr * Dk), gi, gf, st, zero, Hr, Dk, Dvr, Dk ** -0.5), steps, warmup)
    row("recurrent scan, prompt (token by token in registers; fp32 serving, short steps)", "prefill attention", ms,
        flops=4.0 * Dk * Dvr * Hr * B * T)
    ms = timer(lambda: ml.mlstm_chunkwise(pr, (0, Hr * Dk, 2 * Hr * Dk), gi, gf, st, zero, Hr, Dk, Dvr, Dk ** -0.5), steps,
               warmup)
    row("recurrent prompt, chunk-wise (fp32 matrix products; bf16 serving, steps of 64+ tokens)", "prefill attention", ms,
        flops=4.0 * Dk * Dvr * Hr * B * T)
    prd = torch.randn(Bd, 1, ld, device=dev, dtype=bf) * 0.3
    one = torch.ones(Bd, dtype=torch.int32, device=dev)
    ms = timer(lambda: ml.mlstm_scan(prd, (0, Hr * Dk, 2 * Hr * Dk), gi[:Bd], gf[:Bd], st, one, Hr, Dk, Dvr, Dk ** -0.5),
               steps, warmup)
    row("recurrent scan, one token (state read + written)", "decode attention", ms, nbytes=8.0 * Dk * Dvr * Hr * Bd)
    hh = torch.randn(B * T, W, device=dev, dtype=bf)
    gw = torch.randn(2 * Hr, W, device=dev, dtype=bf) * 0.02
    gb = torch.zeros(2 * Hr, device=dev)
    ms = timer(lambda: ml.mlstm_gates(hh, gw, gb, Hr, 15.0), steps, warmup)
    row("recurrent gates (fp32 dot products)", "norm", ms, nbytes=2.0 * B * T * W)
    # norms on the prefill activations
    N = B * T
    x32 = torch.randn(N, W, device=dev)
    y = torch.randn(N, W, device=dev, dtype=bf)
    w1, w2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
    ms = timer(lambda: norm_ops.norm_chain_(x32, y, w1, w2, 1e-6, bf), steps, warmup)
    row("post-norm + fp32 residual + next pre-norm", "norm", ms, nbytes=float(N * W * (2 + 4 + 4 + 2)))
    rb, wb = torch.randn(N, W, device=dev, dtype=bf), torch.ones(W, device=dev, dtype=bf)
    ms = timer(lambda: norm_ops.fused_add_rms_norm(y, rb, wb, 1e-5), steps, warmup)
    row("fused add + RMSNorm (bf16 residual)", "norm", ms, nbytes=float(N * W * 2 * 4))
    qk = torch.randn(B, T, (H + G) * D, device=dev, dtype=bf)
    ck2 = torch.zeros(B, G, S, D, device=dev, dtype=bf)
    cv2 = torch.zeros(B, G, S, D, device=dev, dtype=bf)
    t2 = rope_ops.build_interleaved_rope_cache(S, D, 5e5, device=dev)
    wq = torch.ones(D, device=dev)
    ms = timer(lambda: wa.qk_norm_cache_write(qk, ck2, cv2, zero, H, G, D, D, 1e-6, q_weight=wq, k_weight=wq, rope=t2,
                                              value_from_key=True), steps, warmup)
    row("q/k norm + rotation + cache write", "projection epilogue", ms, nbytes=2.0 * N * (2 * H * D + 3 * G * D))
    return rows


def run_hybrid(steps: int = 10, warmup: int = 3, device=None, sizes=None) -> dict:
    dev = device or torch.device("cuda", torch.cuda.current_device())
    before = _lib.kernel_launches()
    out = {"metric": "Rasodra vs Llama decoder, serving throughput at equal layer sizes", "dtype": "bf16",
           "data": "synthetic token ids, random-init weights", "steps": steps, "warmup": max(warmup, 3),
           "l2": "192 MB written between timed runs", "peaks": peaks(), "cases": [], "kernels": {}}
    for s in (sizes or HYBRID_SIZES):
        out["cases"].append(hybrid_serve_case(s, steps, warmup, dev))
        out["kernels"][s["name"]] = hybrid_kernel_cases(s, steps, warmup, dev)
    out["gpu_launches"] = _lib.kernel_launches() - before
    return out


# ---- Gogalix (gated delta rule + differential window attention on a gated parallel residual) next to the closest existing
# family, Rasodra (recurrent matrix memory + attention over the cache, fp32 stream), at equal width, heads, head size,
# layer count and feed-forward parameters ---------------------------------------------------------------------------------
def gogalix_config(s: dict):
    from ..models.gogalix import GogalixConfig

    # three matrices of (width x f) against Rasodra's two of (width x ff): f = 2/3 ff keeps the parameters equal
    ff = {"kind": "dense", "ff": (2 * s["ff"] // 3 + 127) // 128 * 128}
    half = s["dim"] // 2                        # two maps of half the head size: the query / key rows of a plain head
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": half, "vdim": s["dim"], "scale": half ** -0.5,
           "diff": 0.5, "mask": {"size": s["chunk"]}}
    rec = {"heads": s["rec_heads"], "kv_heads": s["rec_heads"], "dim": s["rec_dim"], "vdim": s["rec_vdim"], "conv": 4}
    return GogalixConfig.from_dict({
        "architecture": "Gogalix", "vocab": VOCAB, "width": s["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
        "layers": [{"type": "attention", "mixer": att, "mlp": ff},
                   {"type": "delta", "mixer": rec, "mlp": None},
                   {"type": "attention", "mixer": dict(att, kv_from=0), "mlp": ff},
                   {"type": "channel_delta", "mixer": dict(rec, rank=64), "mlp": ff}]}, torch_dtype=torch.bfloat16)


def delta_serve_case(s: dict, steps: int, warmup: int, dev) -> dict:
    from .hybrid import GogalixInferenceModel, RasodraInferenceModel

    timer = _Timer(dev)
    out = {"size": dict(s)}
    ic = dict(batch_size=s["decode_batch"], max_batch_size=s["decode_batch"], max_context_length=s["prompt"],
              seq_len=s["prompt"] + 64, is_continuous_batching=True, use_cuda_graphs=False)
    for name, make in (("gogalix", lambda: GogalixInferenceModel(gogalix_config(s), InferenceConfig(**ic), device=dev)),
                       ("rasodra", lambda: RasodraInferenceModel(rasodra_config(s), InferenceConfig(**ic), device=dev))):
        torch.manual_seed(0)
        model = make()
        model.init_kv_cache(device=dev)
        out[name] = _serve(model, s, timer, steps, warmup, dev)
        del model
        torch.cuda.empty_cache()
    out["gogalix_over_rasodra"] = {k: out["gogalix"][k] / out["rasodra"][k]
                                   for k in ("prefill_tokens_per_s", "decode_tokens_per_s")}
    return out


def delta_kernel_cases(s: dict, steps: int, warmup: int, dev) -> List[dict]:
    """Gogalix's own kernels on the shapes of ``s``, alone, with roofline fractions, each next to the like kernel of the
    Rasodra family (recurrent scan / step, attention over the cache, norm chain, projection epilogue)."""
    from ..ops import delta_rule as dr
    from ..ops import mlstm as ml

    pk = peaks()
    timer = _Timer(dev)
    bf = torch.bfloat16
    B, T, H, G, D, W, Bd = s["prefill_batch"], s["prompt"], s["heads"], s["kv_heads"], s["dim"], s["width"], s["decode_batch"]
    rows = []

    def row(kernel, like, ms, flops=None, nbytes=None):
        r = {"kernel": kernel, "like": like, "ms": ms, "peak": pk["source"]}
        if flops is not None:
            r["tflops"] = flops / ms / 1e9
            r["of_peak"] = r["tflops"] / pk["bf16_tflops"]
        if nbytes is not None:
            r["gbs"] = nbytes / ms / 1e6
            r["of_peak"] = r["gbs"] / pk["hbm_gbs"]
        rows.append(r)

    S, N = T + 64, B * T
    zero = torch.zeros(B, dtype=torch.int32, device=dev)
    win = s["chunk"]
    i = torch.arange(T).reshape(T, 1)
    j = torch.arange(T).reshape(1, T)
    pairs_win = int(((j <= i) & (i - j < win)).sum())
    pairs_chunk = int(((j <= i) & (i // win == j // win)).sum())
    # differential attention: 2H query heads of D/2 over 2G key heads and G value heads of D
    Dh = D // 2
    q2 = torch.randn(B, T, 2 * H, Dh, device=dev, dtype=bf)
    ck2 = torch.randn(max(B, Bd), 2 * G, S, Dh, device=dev, dtype=bf)
    cv2 = torch.randn(max(B, Bd), G, S, D, device=dev, dtype=bf)
    ms = timer(lambda: wa.window_attention_prefill(q2, ck2, cv2, zero, Dh ** -0.5, win, value_heads=G), steps, warmup)
    row("differential attention prefill (two maps as heads, window, over the cache)", "prefill attention", ms,
        flops=2.0 * (Dh + D) * pairs_win * 2 * H * B)
    q1 = torch.randn(B, T, H, D, device=dev, dtype=bf)
    ck1 = torch.randn(max(B, Bd), G, S, D, device=dev, dtype=bf)
    ms = timer(lambda: wa.window_attention_prefill(q1, ck1, cv2, zero, D ** -0.5, chunk=win), steps, warmup)
    row("chunked attention prefill over the cache (the like kernel)", "prefill attention", ms,
        flops=4.0 * D * pairs_chunk * H * B)
    qd2 = torch.randn(Bd, 2 * H, Dh, device=dev, dtype=bf)
    posd = torch.full((Bd,), T, dtype=torch.int32, device=dev)
    seen = min(win, T + 1)
    ms = timer(lambda: wa.window_attention_decode(qd2, ck2, cv2, posd, Dh ** -0.5, win, value_heads=G), steps, warmup)
    row("differential attention decode (rows of the window; values read by both maps)", "decode attention", ms,
        nbytes=2.0 * seen * G * (2 * Dh + D) * Bd)
    qd1 = torch.randn(Bd, H, D, device=dev, dtype=bf)
    posm = torch.full((Bd,), T - 1, dtype=torch.int32, device=dev)
    ms = timer(lambda: wa.window_attention_decode(qd1, ck1, cv2, posm, D ** -0.5, chunk=win), steps, warmup)
    row("chunked attention decode, a full chunk (the like kernel)", "decode attention", ms,
        nbytes=2.0 * ((T - 1) % win + 1) * G * 2 * D * Bd)
    maps = torch.randn(N, 2 * H, D, device=dev, dtype=bf)
    lv = [torch.randn(Dh, device=dev) * 0.1 for _ in range(4)]
    ms = timer(lambda: wa.diff_attention_combine(maps, *lv, 0.5, 1e-6), steps, warmup)
    row("a1 - lambda a2 + head norm", "norm", ms, nbytes=2.0 * N * 3 * H * D)
    wide = torch.randn(B, T, 2 * H * Dh + 2 * G * Dh + G * D, device=dev, dtype=bf)
    ckw, cvw = torch.zeros(B, 2 * G, S, Dh, device=dev, dtype=bf), torch.zeros(B, G, S, D, device=dev, dtype=bf)
    ms = timer(lambda: wa.qk_norm_cache_write(wide, ckw, cvw, zero, 2 * H, 2 * G, Dh, D, 1e-6, normalize=False,
                                              value_heads=G), steps, warmup)
    row("query copy + cache write of both maps", "projection epilogue", ms, nbytes=2.0 * N * (4 * H * Dh + 4 * G * Dh + 2 * G * D))
    del q2, ck2, cv2, q1, ck1, maps, wide, ckw, cvw
    # gated delta rule
    Hr, Dk, Dvr, taps = s["rec_heads"], s["rec_dim"], s["rec_vdim"], 4
    C = 2 * Hr * Dk + Hr * Dvr
    proj = torch.randn(B, T, C, device=dev, dtype=bf) * 0.3
    cw = torch.randn(C, taps, device=dev) * 0.3
    cst = torch.zeros(max(B, Bd), taps - 1, C, device=dev)
    ms = timer(lambda: dr.delta_prep(proj, (0, Hr * Dk, 2 * Hr * Dk), cw, cst, zero, Hr, Hr, Dk, Dvr, Dk ** -0.5), steps, warmup)
    row("short convolution + silu + unit norm + convolution state", "projection epilogue", ms, nbytes=float(N * C * (2 + 4)))
    qn, kn, vn = dr.delta_prep(proj, (0, Hr * Dk, 2 * Hr * Dk), cw, cst, zero, Hr, Hr, Dk, Dvr, Dk ** -0.5)
    St = torch.zeros(max(B, Bd), Hr, Dk, Dvr, device=dev)
    a_log = torch.full((Hr,), -3.0, device=dev)
    for per_channel in (False, True):
        na = Hr * Dk if per_channel else Hr
        apre, bpre, dtb = torch.randn(N, na, device=dev), torch.randn(N, Hr, device=dev), torch.zeros(na, device=dev)
        tag = "one decay per key channel" if per_channel else "one decay per head"
        ms = timer(lambda: dr.delta_scan(qn, kn, vn, apre, 0, bpre, 0, a_log, dtb, St, zero, per_channel), steps, warmup)
        row(f"gated delta rule, prompt, {tag} (token by token, state slice in registers)", "prefill attention", ms,
            flops=6.0 * Dk * Dvr * Hr * B * T)
        one = torch.ones(Bd, dtype=torch.int32, device=dev)
        qd, kd, vd = (x[:1].expand(Bd, *x.shape[1:])[:, :1].contiguous() for x in (qn, kn, vn))
        ms = timer(lambda: dr.delta_scan(qd, kd, vd, apre[:Bd], 0, bpre[:Bd], 0, a_log, dtb, St, one, per_channel), steps, warmup)
        row(f"gated delta rule, one token, {tag} (state read + written)", "decode attention", ms,
            nbytes=8.0 * Dk * Dvr * Hr * Bd)
    ld = 2 * Hr * Dk + 2 * Hr * Dvr
    pr = torch.randn(B, T, ld, device=dev, dtype=bf) * 0.3
    gi, gf = torch.randn(N, Hr, device=dev), -torch.rand(N, Hr, device=dev) * 0.1
    st = (torch.zeros(Bd, Hr, Dk, Dvr, device=dev), torch.zeros(Bd, Hr, Dk, device=dev), torch.zeros(Bd, Hr, device=dev))
    ms = timer(lambda: ml.mlstm_scan(pr, (0, Hr * Dk, 2 * Hr * Dk), gi, gf, st, zero, Hr, Dk, Dvr, Dk ** -0.5), steps, warmup)
    row("matrix-memory scan, prompt, token by token (the like kernel)", "prefill attention", ms, flops=4.0 * Dk * Dvr * Hr * B * T)
    ms = timer(lambda: ml.mlstm_chunkwise(pr, (0, Hr * Dk, 2 * Hr * Dk), gi, gf, st, zero, Hr, Dk, Dvr, Dk ** -0.5), steps,
               warmup)
    row("matrix-memory prompt, chunk-wise (the like kernel of long bf16 steps)", "prefill attention", ms,
        flops=4.0 * Dk * Dvr * Hr * B * T)
    prd = torch.randn(Bd, 1, ld, device=dev, dtype=bf) * 0.3
    one = torch.ones(Bd, dtype=torch.int32, device=dev)
    ms = timer(lambda: ml.mlstm_scan(prd, (0, Hr * Dk, 2 * Hr * Dk), gi[:Bd], gf[:Bd], st, one, Hr, Dk, Dvr, Dk ** -0.5),
               steps, warmup)
    row("matrix-memory scan, one token (the like kernel)", "decode attention", ms, nbytes=8.0 * Dk * Dvr * Hr * Bd)
    o = torch.randn(N, Hr, Dvr, device=dev)
    gsrc = torch.randn(N, Hr * Dvr, device=dev, dtype=bf)
    wn = torch.ones(Hr * Dvr, device=dev)
    ms = timer(lambda: ml.head_norm_gate(o, gsrc, 0, Hr, Dvr, wn, 1e-6, True, bf, gate_act="silu"), steps, warmup)
    row("head norm * weight * silu gate", "norm", ms, nbytes=float(N * Hr * Dvr * (4 + 2 + 2)))
    del proj, qn, kn, vn, pr, o, gsrc
    # the residual update
    x32 = torch.randn(N, W, device=dev)
    y1, y2 = torch.randn(N, W, device=dev, dtype=bf), torch.randn(N, W, device=dev, dtype=bf)
    gate = torch.randn(N, 2 * W, device=dev, dtype=bf)
    vecs = [torch.randn(W, device=dev) for _ in range(5)]
    wnext = torch.ones(1, device=dev)
    ms = timer(lambda: norm_ops.gated_residual_norm_(x32, y1, y2, vecs[0], gate, (0, W), vecs[1], vecs[2], vecs[3], vecs[4],
                                                     wnext, 1e-6, bf), steps, warmup)
    row("gated residual of both sublayers + layer scale + next norm", "norm", ms, nbytes=float(N * W * (4 + 4 + 2 + 2 + 4 + 2)))
    w1, w2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
    ms = timer(lambda: norm_ops.norm_chain_(x32, y1, w1, w2, 1e-6, bf), steps, warmup)
    row("post-norm + fp32 residual + next pre-norm (the like kernel)", "norm", ms, nbytes=float(N * W * (2 + 4 + 4 + 2)))
    F = (2 * s["ff"] // 3 + 127) // 128 * 128
    src = torch.randn(N, 2 * F, device=dev, dtype=bf)
    gb, ub = torch.zeros(F, device=dev), torch.zeros(F, device=dev)
    ms = timer(lambda: moe_sparse.glu_bias(src, 0, F, F, gb, ub), steps, warmup)
    row("silu(gate + b) * (up + b) from the fused projection", "activation", ms, nbytes=2.0 * N * 3 * F)
    ms = timer(lambda: act_ops.swiglu(src), steps, warmup)
    row("swiglu (the like kernel of the Llama decoder)", "activation", ms, nbytes=2.0 * N * 3 * F)
    return rows


def run_delta(steps: int = 10, warmup: int = 3, device=None, sizes=None) -> dict:
    dev = device or torch.device("cuda", torch.cuda.current_device())
    before = _lib.kernel_launches()
    out = {"metric": "Gogalix vs Rasodra, serving throughput at equal layer sizes", "dtype": "bf16",
           "data": "synthetic token ids, random-init weights", "steps": steps, "warmup": max(warmup, 3),
           "l2": "192 MB written between timed runs", "peaks": peaks(), "cases": [], "kernels": {}}
    for s in (sizes or HYBRID_SIZES):
        out["cases"].append(delta_serve_case(s, steps, warmup, dev))
        out["kernels"][s["name"]] = delta_kernel_cases(s, steps, warmup, dev)
    out["gpu_launches"] = _lib.kernel_launches() - before
    return out


# ---- Vufasun next to Gogalix ------------------------------------------------------------------------------------------------
VUFASUN_STREAMS = 2


def vufasun_config(s: dict):
    from ..models.vufasun import VufasunConfig

    # gate, up and down of (width x f), as in Gogalix's dense feed-forward: the same f keeps the parameters equal
    ff = {"kind": "dense", "ff": (2 * s["ff"] // 3 + 127) // 128 * 128}
    rot = {"base": 500000.0, "dims": s["dim"] // 2}
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
           "rot": rot}
    left = dict(att, rot=dict(rot, scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}))
    decay = [1.0 - 2.0 ** (-5 - 3.0 * h / max(s["rec_heads"] - 1, 1)) for h in range(s["rec_heads"])]
    right = {"heads": s["rec_heads"], "dim": s["rec_dim"], "vdim": s["rec_vdim"], "decay": decay,
             "rot": {"base": 500000.0, "dims": s["rec_dim"]}}
    par = {"left": left, "right": right}
    return VufasunConfig.from_dict({
        "architecture": "Vufasun", "vocab": VOCAB, "width": s["width"], "streams": VUFASUN_STREAMS, "norm": {"eps": 1e-6},
        "layers": [{"type": "parallel", "mixer": par, "mlp": ff},
                   {"type": "attention", "mixer": att, "mlp": ff},
                   {"type": "parallel", "mixer": par, "mlp": ff}]}, torch_dtype=torch.bfloat16)


def retention_serve_case(s: dict, steps: int, warmup: int, dev) -> dict:
    from .hybrid import GogalixInferenceModel, VufasunInferenceModel

    timer = _Timer(dev)
    out = {"size": dict(s)}
    ic = dict(batch_size=s["decode_batch"], max_batch_size=s["decode_batch"], max_context_length=s["prompt"],
              seq_len=s["prompt"] + 64, is_continuous_batching=True, use_cuda_graphs=False)
    for name, make in (("vufasun", lambda: VufasunInferenceModel(vufasun_config(s), InferenceConfig(**ic), device=dev)),
                       ("gogalix", lambda: GogalixInferenceModel(gogalix_config(s), InferenceConfig(**ic), device=dev))):
        torch.manual_seed(0)
        model = make()
        model.init_kv_cache(device=dev)
        out[name] = _serve(model, s, timer, steps, warmup, dev)
        out[name]["parameters"] = sum(p.numel() for p in model.parameters())
        del model
        torch.cuda.empty_cache()
    out["vufasun_over_gogalix"] = {k: out["vufasun"][k] / out["gogalix"][k]
                                   for k in ("prefill_tokens_per_s", "decode_tokens_per_s")}
    return out


def retention_kernel_cases(s: dict, steps: int, warmup: int, dev) -> List[dict]:
    """Vufasun's own kernels on the shapes of ``s``, alone, with roofline fractions, each next to the like kernel of the
    Gogalix / Rasodra families (recurrent scan / step, attention over the cache, residual update, projection epilogue)."""
    from ..ops import hyper_connection as hc_ops
    from ..ops import mlstm as ml
    from ..ops import retention as rt
    from ..ops import rope as rope_ops

    pk = peaks()
    timer = _Timer(dev)
    bf = torch.bfloat16
    B, T, H, G, D, W, Bd = s["prefill_batch"], s["prompt"], s["heads"], s["kv_heads"], s["dim"], s["width"], s["decode_batch"]
    rows = []

    def row(kernel, like, ms, flops=None, nbytes=None):
        r = {"kernel": kernel, "like": like, "ms": ms, "peak": pk["source"]}
        if flops is not None:
            r["tflops"] = flops / ms / 1e9
            r["of_peak"] = r["tflops"] / pk["bf16_tflops"]
        if nbytes is not None:
            r["gbs"] = nbytes / ms / 1e6
            r["of_peak"] = r["gbs"] / pk["hbm_gbs"]
        rows.append(r)

    S, N = T + 64, B * T
    zero = torch.zeros(B, dtype=torch.int32, device=dev)
    pairs = T * (T + 1) // 2
    # softmax attention with the sink term, next to the same kernels without it
    q = torch.randn(B, T, H, D, device=dev, dtype=bf)
    ck = torch.randn(max(B, Bd), G, S, D, device=dev, dtype=bf)
    cv = torch.randn(max(B, Bd), G, S, D, device=dev, dtype=bf)
    sink = torch.randn(H, device=dev)
    for name, sk in (("softmax attention prefill with a sink term, over the cache", sink),
                     ("causal attention prefill over the cache (the like kernel)", None)):
        ms = timer(lambda: wa.window_attention_prefill(q, ck, cv, zero, D ** -0.5, sinks=sk), steps, warmup)
        row(name, "prefill attention", ms, flops=4.0 * D * pairs * H * B)
    qd = torch.randn(Bd, H, D, device=dev, dtype=bf)
    posd = torch.full((Bd,), T, dtype=torch.int32, device=dev)
    for name, sk in (("softmax attention decode with a sink term", sink), ("causal attention decode (the like kernel)", None)):
        ms = timer(lambda: wa.window_attention_decode(qd, ck, cv, posd, D ** -0.5, sinks=sk), steps, warmup)
        row(name, "decode attention", ms, nbytes=2.0 * (T + 1) * G * 2 * D * Bd)
    n_qkv = H * D + 2 * G * D
    wide = torch.randn(B, T, n_qkv, device=dev, dtype=bf)
    ckw, cvw = torch.zeros(B, G, S, D, device=dev, dtype=bf), torch.zeros(B, G, S, D, device=dev, dtype=bf)
    rope = rope_ops.build_interleaved_rope_cache(S, D // 2, 500000.0, device=dev, scaling=(8.0, 1.0, 4.0, 8192))
    qw, kw = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
    ms = timer(lambda: wa.qk_norm_cache_write(wide, ckw, cvw, zero, H, G, D, D, 1e-6, normalize=True, q_weight=qw,
                                              k_weight=kw, rope=rope, rope_layout="halves", whole_norm=True), steps, warmup)
    row("whole-projection q / k norm + rotation of halves + cache write", "projection epilogue", ms,
        nbytes=2.0 * N * (2 * H * D + 4 * G * D))
    ms = timer(lambda: wa.qk_norm_cache_write(wide, ckw, cvw, zero, H, G, D, D, 1e-6, normalize=False, rope=rope,
                                              rope_layout="halves"), steps, warmup)
    row("rotation of halves + cache write (sink-attention layers)", "projection epilogue", ms,
        nbytes=2.0 * N * (2 * H * D + 4 * G * D))
    ms = timer(lambda: wa.qk_norm_cache_write(wide, ckw, cvw, zero, H, G, D, D, 1e-6, normalize=True), steps, warmup)
    row("per-head unit norm + cache write (the like kernel)", "projection epilogue", ms,
        nbytes=2.0 * N * (2 * H * D + 4 * G * D))
    del q, ck, cv, wide, ckw, cvw
    # retention next to the matrix-memory kernels
    Hr, Dk, Dvr = s["rec_heads"], s["rec_dim"], s["rec_vdim"]
    ld = 2 * Hr * Dk + 2 * Hr * Dvr
    pr = torch.randn(B, T, ld, device=dev, dtype=bf) * 0.3
    dec = torch.full((Hr,), 0.99, device=dev)
    st = torch.zeros(max(B, Bd), Hr, Dk, Dvr, device=dev)
    rrope = rope_ops.build_interleaved_rope_cache(S, Dk, 500000.0, device=dev)
    offs = (0, Hr * Dk, 2 * Hr * Dk)
    flops = 4.0 * Dk * Dvr * Hr * B * T
    if rt.chunkwise_applies(Dk, Dvr):
        ms = timer(lambda: rt.retention_chunkwise(pr, offs, dec, st, zero, Hr, Dk, Dvr, Dk ** -0.5, rope=rrope), steps, warmup)
        row("retention prompt, chunk-wise (rotation inside)", "prefill attention", ms, flops=flops)
    ms = timer(lambda: rt.retention_scan(pr, offs, dec, st, zero, Hr, Dk, Dvr, Dk ** -0.5, rope=rrope), steps, warmup)
    row("retention prompt, token by token (state slice in registers, rotation inside)", "prefill attention", ms, flops=flops)
    gi, gf = torch.randn(N, Hr, device=dev), -torch.rand(N, Hr, device=dev) * 0.1
    mst = (torch.zeros(max(B, Bd), Hr, Dk, Dvr, device=dev), torch.zeros(max(B, Bd), Hr, Dk, device=dev),
           torch.zeros(max(B, Bd), Hr, device=dev))
    ms = timer(lambda: ml.mlstm_scan(pr, offs, gi, gf, mst, zero, Hr, Dk, Dvr, Dk ** -0.5), steps, warmup)
    row("matrix-memory scan, prompt, token by token (the like kernel)", "prefill attention", ms, flops=flops)
    ms = timer(lambda: ml.mlstm_chunkwise(pr, offs, gi, gf, mst, zero, Hr, Dk, Dvr, Dk ** -0.5), steps, warmup)
    row("matrix-memory prompt, chunk-wise (the like kernel of long bf16 steps)", "prefill attention", ms, flops=flops)
    prd = torch.randn(Bd, 1, ld, device=dev, dtype=bf) * 0.3
    at = torch.full((Bd,), T, dtype=torch.int32, device=dev)
    ms = timer(lambda: rt.retention_scan(prd, offs, dec, st, at, Hr, Dk, Dvr, Dk ** -0.5, rope=rrope), steps, warmup)
    row("retention, one token (state read + written)", "decode attention", ms, nbytes=8.0 * Dk * Dvr * Hr * Bd)
    ms = timer(lambda: ml.mlstm_scan(prd, offs, gi[:Bd], gf[:Bd], mst, at, Hr, Dk, Dvr, Dk ** -0.5), steps, warmup)
    row("matrix-memory scan, one token (the like kernel)", "decode attention", ms, nbytes=8.0 * Dk * Dvr * Hr * Bd)
    o = torch.randn(N, Hr, Dvr, device=dev)
    ms = timer(lambda: ml.head_norm_gate(o, pr.view(N, ld), 2 * Hr * Dk + Hr * Dvr, Hr, Dvr, None, 1e-6, True, bf,
                                         gate_act="silu"), steps, warmup)
    row("unit head norm * silu gate", "norm", ms, nbytes=float(N * Hr * Dvr * (4 + 2 + 2)))
    del pr, o
    # the stream update next to the gated residual of the parallel-residual family
    St = VUFASUN_STREAMS
    xs = torch.randn(N, St, W, device=dev)
    y1, y2 = torch.randn(N, W, device=dev, dtype=bf), torch.randn(N, W, device=dev, dtype=bf)
    mix, ow, iw = torch.eye(St, device=dev), torch.ones(St, device=dev), torch.ones(St, device=dev)
    wn, wa_, wb = torch.ones(W, device=dev), torch.ones(W, device=dev), torch.ones(W, device=dev)
    ms = timer(lambda: hc_ops.hc_step(xs, y1, mix, ow, iw, wn, 1e-6, bf), steps, warmup)
    row(f"stream write + mixing + next read and norm ({St} streams)", "norm", ms, nbytes=float(N * W * (8 * St + 2 + 2)))
    ms = timer(lambda: hc_ops.hc_step(xs, y1, mix, ow, iw, wn, 1e-6, bf, y2=y2, branch_w=(wa_, wb)), steps, warmup)
    row(f"the same with the mean of two normed branches ({St} streams)", "norm", ms, nbytes=float(N * W * (8 * St + 4 + 2)))
    x32 = torch.randn(N, W, device=dev)
    gate = torch.randn(N, 2 * W, device=dev, dtype=bf)
    vecs = [torch.randn(W, device=dev) for _ in range(5)]
    wnext = torch.ones(1, device=dev)
    ms = timer(lambda: norm_ops.gated_residual_norm_(x32, y1, y2, vecs[0], gate, (0, W), vecs[1], vecs[2], vecs[3], vecs[4],
                                                     wnext, 1e-6, bf), steps, warmup)
    row("gated residual of both sublayers + layer scale + next norm (the like kernel)", "norm", ms,
        nbytes=float(N * W * (4 + 4 + 2 + 2 + 4 + 2)))
    del xs, x32, gate
    F = (2 * s["ff"] // 3 + 127) // 128 * 128
    src = torch.randn(N, 2 * F, device=dev, dtype=bf)
    ms = timer(lambda: moe_sparse.glu_bias(src, 0, F, F, act="gelu_tanh"), steps, warmup)
    row("gelu_tanh(gate) * up from the fused projection", "activation", ms, nbytes=2.0 * N * 3 * F)
    gb, ub = torch.zeros(F, device=dev), torch.zeros(F, device=dev)
    ms = timer(lambda: moe_sparse.glu_bias(src, 0, F, F, gb, ub), steps, warmup)
    row("silu(gate + b) * (up + b) from the fused projection (the like kernel)", "activation", ms, nbytes=2.0 * N * 3 * F)
    return rows


def run_retention(steps: int = 10, warmup: int = 3, device=None, sizes=None) -> dict:
    dev = device or torch.device("cuda", torch.cuda.current_device())
    before = _lib.kernel_launches()
    out = {"metric": "Vufasun vs Gogalix, serving throughput at equal layer sizes", "dtype": "bf16",
           "data": "synthetic token ids, random-init weights", "steps": steps, "warmup": max(warmup, 3),
           "l2": "192 MB written between timed runs", "peaks": peaks(), "cases": [], "kernels": {}}
    for s in (sizes or HYBRID_SIZES):
        out["cases"].append(retention_serve_case(s, steps, warmup, dev))
        out["kernels"][s["name"]] = retention_kernel_cases(s, steps, warmup, dev)
    out["gpu_launches"] = _lib.kernel_launches() - before
    return out

#!/usr/bin/env python
"""Vufasun inference: build the runner for a model directory (``config.json`` + ``model.safetensors``) or for the small
built-in configuration with random weights, trace the buckets, generate, optionally benchmark.

    python examples/inference/run_vufasun.py --model_dir /path/to/model --batch_size 4 --max_new_tokens 64
    python examples/inference/run_vufasun.py --tiny --benchmark
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from neuronx_distributed_llama3_2_b200.inference import VufasunRunner, InferenceConfig  # noqa: E402
from neuronx_distributed_llama3_2_b200.inference.checkpoint import load_state_dict  # noqa: E402
from neuronx_distributed_llama3_2_b200.models import VufasunConfig, convert_vufasun_state_dict, tiny_vufasun  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_dir", default=None, help="folder with config.json and model.safetensors")
    ap.add_argument("--tiny", action="store_true", help="the small built-in configuration with random weights")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--batch_size", type=int, default=2)
    ap.add_argument("--max_context_length", type=int, default=256)
    ap.add_argument("--seq_len", type=int, default=512)
    ap.add_argument("--max_new_tokens", type=int, default=16)
    ap.add_argument("--top_k", type=int, default=1)
    ap.add_argument("--no_cuda_graphs", action="store_true")
    ap.add_argument("--benchmark", action="store_true")
    args = ap.parse_args()
    dtype = torch.float32 if (args.dtype == "float32" or not torch.cuda.is_available()) else torch.bfloat16
    if args.model_dir:
        raw = load_state_dict(args.model_dir)
        cfg = VufasunConfig.from_json(args.model_dir, torch_dtype=dtype).with_checkpoint_shapes(raw)
        loader = lambda: convert_vufasun_state_dict(raw, cfg)  # noqa: E731
    elif args.tiny:
        cfg, loader = tiny_vufasun(torch_dtype=dtype), None
    else:
        ap.error("give --model_dir or --tiny")
    ic = InferenceConfig(batch_size=args.batch_size, max_context_length=args.max_context_length, seq_len=args.seq_len,
                         max_new_tokens=args.max_new_tokens, top_k=args.top_k, do_sample=args.top_k > 1,
                         use_cuda_graphs=not args.no_cuda_graphs)
    runner = VufasunRunner(cfg, ic, checkpoint_loader=loader)
    runner.trace()
    T = min(32, args.max_context_length)
    prompts = torch.randint(1, cfg.vocab_size, (args.batch_size, T), device=runner.device)
    out = runner.generate(prompts, max_new_tokens=args.max_new_tokens)
    print("generated token ids:", out[0, T:].tolist())
    if args.benchmark:
        print(json.dumps(runner.benchmark_sampling(prompt_len=T, new_tokens=args.max_new_tokens, n_runs=5), indent=1))
    runner.close()


if __name__ == "__main__":
    main()

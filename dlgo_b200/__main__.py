"""Command line: ``python -m dlgo_b200 <command> ...``.

Option names follow the reference's example programs where it has them:
``--ctx``, ``--max-tokens`` and ``--temp`` (examples/simple_chat/main.go:19-22),
and its generation options ``top-k``, ``top-p``, ``seed``, ``greedy``
(dlgo.go:213-240).  Prompts are token ids.

    python -m dlgo_b200 generate MODEL --prompt-ids 1,2,3 [--max-tokens 256] [--temp 0.7] [--ctx N]
    python -m dlgo_b200 info MODEL
    python -m dlgo_b200 random-model --config CONFIG.json --seed 0 --out DIR
    python -m dlgo_b200 build
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _parse_ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def _add_generation_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("model", help="model folder (config.json + model.safetensors)")
    p.add_argument("--prompt-ids", action="append", default=[],
                   help="token ids of one prompt, comma or space separated (repeat for a batch)")
    p.add_argument("--prompt-file", help="file with one prompt per line (token ids)")
    p.add_argument("--ctx", type=int, default=0, help="runtime context length in tokens (0 = the model's)")
    p.add_argument("--max-tokens", type=int, default=256, help="max tokens to generate per prompt")
    p.add_argument("--temp", type=float, default=0.7, help="sampling temperature (0 = greedy)")
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--repetition-penalty", type=float, default=1.1)
    p.add_argument("--seed", type=int, default=-1, help="sampler seed (-1 = from the clock)")
    p.add_argument("--greedy", action="store_true", help="argmax decoding")
    p.add_argument("--stop-token-ids", default="", help="extra stop tokens")
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--stream", action="store_true", help="print tokens as they are produced")
    p.add_argument("--bench", action="store_true", help="print prompt tokens, output tokens, prefill ms, tok/s")
    p.add_argument("--profile", action="store_true",
                   help="time every kernel (CUDA events, no CUDA graphs) and print the totals; also DLGO_PROFILE=1")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--max-batch", type=int, default=64)


def _cmd_generate(a: argparse.Namespace) -> int:
    from .api import load_llm

    prompts = [_parse_ids(t) for t in a.prompt_ids]
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts += [_parse_ids(line) for line in f if line.strip()]
    if not prompts:
        print("error: no prompt (use --prompt-ids or --prompt-file)", file=sys.stderr)
        return 2
    if a.ctx < 0 or a.max_tokens <= 0 or a.temp < 0:
        print("error: --ctx must be >= 0, --max-tokens > 0 and --temp >= 0", file=sys.stderr)
        return 2
    import os
    profile = a.profile or os.environ.get("DLGO_PROFILE", "") not in ("", "0")
    llm = load_llm(a.model, a.ctx, dtype=a.dtype, device=a.device, max_batch=a.max_batch, cuda_graphs=not profile)
    print(f"Model: {llm.model_info()}", file=sys.stderr)
    if profile:
        from .csrc import kernels
        kernels.profile_start()
    opts = dict(max_tokens=a.max_tokens, temperature=a.temp, top_k=a.top_k, top_p=a.top_p, min_p=a.min_p,
                repetition_penalty=a.repetition_penalty, seed=a.seed, greedy=a.greedy,
                stop_token_ids=_parse_ids(a.stop_token_ids), ignore_eos=a.ignore_eos)
    if a.stream:
        llm.generate_stream(prompts, lambda r, t: print(f"{r}\t{t}", flush=True), **opts)
    elif a.bench:
        res = llm.benchmark(prompts, **opts)
        for out in res.tokens:
            print(" ".join(str(t) for t in out))
        print(f"{res} | prompt tokens: {res.prompt_tokens}", file=sys.stderr)
    else:
        for out in llm.generate(prompts, **opts):
            print(" ".join(str(t) for t in out))
    if profile:
        rows = kernels.profile_stop()
        whole = sum(ms for _, _, ms in rows) or 1.0
        print(f"{'kernel entry point':28s} {'launches':>9s} {'ms':>10s} {'share':>7s}", file=sys.stderr)
        for name, n, ms in rows:
            print(f"{name:28s} {n:9d} {ms:10.3f} {100 * ms / whole:6.1f}%", file=sys.stderr)
    return 0


def _cmd_info(a: argparse.Namespace) -> int:
    from .config import load_config
    cfg = load_config(a.model)
    print(json.dumps(cfg.to_dict(), indent=2))
    return 0


def _cmd_random_model(a: argparse.Namespace) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    with open(a.config) as f:
        cfg = config_from_dict(json.load(f))
    write_random_model(cfg, a.seed, a.out, std=a.std,
                       dtype=torch.float32 if a.store == "float32" else torch.bfloat16, device=a.device)
    print(a.out)
    return 0


def _cmd_build(a: argparse.Namespace) -> int:
    from .csrc import build
    for name, path in build.build_all().items():
        print(f"{name}: {path}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dlgo_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate tokens for one or more prompts")
    _add_generation_options(g)
    g.set_defaults(fn=_cmd_generate)
    i = sub.add_parser("info", help="print a model folder's configuration")
    i.add_argument("model")
    i.set_defaults(fn=_cmd_info)
    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--store", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--device", default="cpu")
    r.set_defaults(fn=_cmd_random_model)
    b = sub.add_parser("build", help="compile every CUDA kernel library for sm_100a")
    b.set_defaults(fn=_cmd_build)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())

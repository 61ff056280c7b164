"""The `tq` command line, after the reference's (src/main.rs:23-187).

Kept subcommands and options, with their names, short forms, defaults and
meanings: `chat MODEL` (-n/--max-tokens 512, -t/--temperature 0.7, --top-p
0.9, --top-k 40, --repeat-penalty 1.1, --model-path), `bench MODEL`
(-n/--tokens 100, --json, --prompt; greedy, tok/s = emitted tokens / wall time
including the prompt, TTFT = time to the first token, src/main.rs:1116-1151),
`perplexity FILE` (-m/--model, --model-path; token by token,
src/engine.rs:467-529), `list`, `doctor`.  `run` is an alias of `chat` that
generates once instead of reading turns from the terminal.  Not kept: serve,
pull, rm, calibrate, ablate, --cpu, --tq-bits (servers, downloads and cache
compression are outside this library; there is no CPU path).

Prompts are token ids (`--prompt-ids 1,2,3` or `--prompt-file` with ids
separated by spaces or commas); `--prompt TEXT` works when the model folder
has a tokenizer.json.  MODEL is a model folder or, with --random-weights, the
name of a shape (`tq list`).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import sys
import time
from typing import Optional

from .sampling import GenerationParams

BENCH_PROMPT = "Explain the theory of relativity in simple terms. Include examples."   # src/main.rs:934-936


def _add_model_args(p: argparse.ArgumentParser, positional: bool = True) -> None:
    if positional:
        p.add_argument("model", help="model folder, or a shape name with --random-weights")
    else:
        p.add_argument("-m", "--model", default=None, help="model folder or shape name")
    p.add_argument("--model-path", default=None, help="model folder (overrides MODEL)")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--random-weights", action="store_true", help="random weights for MODEL's configuration")
    p.add_argument("--seed", type=int, default=0, help="seed of sampling (and of random weights)")
    p.add_argument("--max-context", type=int, default=None)


def _add_sampling_args(p: argparse.ArgumentParser, max_tokens_default: int = 512) -> None:
    p.add_argument("-n", "--max-tokens", type=int, default=max_tokens_default, help="max tokens per response")
    p.add_argument("-t", "--temperature", type=float, default=0.7, help="temperature; <= 0 is arg-max")
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--repeat-penalty", type=float, default=1.1)


def _add_prompt_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--prompt-ids", action="append", default=None,
                   help="token ids, comma separated; repeat the option for a batch of prompts")
    p.add_argument("--prompt-file", default=None, help="file with one prompt of token ids per line")
    p.add_argument("--prompt", action="append", default=None, help="text prompt (needs tokenizer.json)")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tq", description="Qwen2.5 generation on one B200")
    sub = ap.add_subparsers(dest="command")
    for name in ("chat", "run"):
        p = sub.add_parser(name, help="generate from prompts" if name == "run" else "interactive generation")
        _add_model_args(p)
        _add_sampling_args(p)
        _add_prompt_args(p)
    p = sub.add_parser("bench", help="time generation (greedy)")
    _add_model_args(p)
    p.add_argument("-n", "--tokens", type=int, default=100, help="tokens to generate per run")
    p.add_argument("--json", action="store_true", help="output results as JSON")
    _add_prompt_args(p)
    p = sub.add_parser("perplexity", help="token-by-token perplexity of a file of token ids")
    _add_model_args(p, positional=False)
    p.add_argument("file", help="file of token ids (or text, with tokenizer.json)")
    sub.add_parser("list", help="list the named shapes")
    sub.add_parser("doctor", help="check the GPU, nvcc and the CUDA library")
    return ap


def _parse_ids(text: str) -> list[int]:
    return [int(t) for t in re.split(r"[\s,]+", text.strip()) if t]


def _tokenizer(folder: Optional[str]):
    if folder and os.path.isfile(os.path.join(folder, "tokenizer.json")):
        from tokenizers import Tokenizer
        return Tokenizer.from_file(os.path.join(folder, "tokenizer.json"))
    return None


def _model_location(args) -> str:
    loc = args.model_path or args.model
    if not loc:
        raise SystemExit("tq: no model given")
    return loc


def _load(args):
    from .api import load
    return load(_model_location(args), dtype=args.dtype, random_weights=args.random_weights, seed=args.seed,
                max_context=args.max_context)


def _prompts(args, tok, default_text: Optional[str] = None) -> list[list[int]]:
    prompts: list[list[int]] = []
    for s in args.prompt_ids or []:
        prompts.append(_parse_ids(s))
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_parse_ids(line) for line in f if line.strip()]
    texts = list(args.prompt or [])
    if not prompts and not texts and default_text is not None and tok is not None:
        texts = [default_text]
    for t in texts:
        if tok is None:
            raise SystemExit("tq: --prompt needs a tokenizer.json in the model folder; use --prompt-ids")
        prompts.append(tok.encode(t, add_special_tokens=False).ids)     # src/engine.rs:342-344
    return prompts


def _params(args) -> GenerationParams:
    return GenerationParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                            top_k=args.top_k, repeat_penalty=args.repeat_penalty, seed=args.seed)


def cmd_run(args, interactive: bool) -> int:
    engine = _load(args)
    tok = _tokenizer(_model_location(args) if not args.random_weights else None)
    prompts = _prompts(args, tok)
    if not prompts and interactive:
        print("tq chat: enter a prompt per line (token ids, or text with a tokenizer); empty line ends",
              file=sys.stderr)
        for line in sys.stdin:
            line = line.strip()
            if not line:
                break
            ids = _parse_ids(line) if re.fullmatch(r"[\d\s,]+", line) else (
                tok.encode(line, add_special_tokens=False).ids if tok else None)
            if ids is None:
                print("tq: text needs a tokenizer.json; give token ids", file=sys.stderr)
                continue
            _emit(engine.generate([ids], _params(args)), tok)
        return 0
    if not prompts:
        raise SystemExit("tq: no prompt (use --prompt-ids, --prompt-file or --prompt)")
    _emit(engine.generate(prompts, _params(args)), tok)
    return 0


def _emit(results, tok) -> None:
    for r in results:
        if tok is not None:
            print(tok.decode(r.tokens, skip_special_tokens=True))
        else:
            print(",".join(str(t) for t in r.tokens))


def cmd_bench(args) -> int:
    import torch
    engine = _load(args)
    tok = _tokenizer(_model_location(args) if not args.random_weights else None)
    prompts = _prompts(args, tok, BENCH_PROMPT)
    if not prompts:
        g = torch.Generator().manual_seed(args.seed)
        prompts = [torch.randint(0, engine.vocab_size, (32,), generator=g).tolist()]
    params = GenerationParams.greedy(args.tokens, seed=args.seed, stop_token_ids=())   # src/main.rs:947-951
    engine.generate(prompts, GenerationParams.greedy(2, stop_token_ids=()))           # warm-up (builds, allocates)
    torch.cuda.synchronize()
    first: list[float] = []
    t0 = time.perf_counter()
    res = engine.generate(prompts, params,
                          on_token=lambda i, t: first.append(time.perf_counter()) if not first else None)
    torch.cuda.synchronize()
    total = time.perf_counter() - t0
    n = sum(len(r.tokens) for r in res)
    out = {"model": _model_location(args), "dtype": args.dtype, "batch": len(prompts),
           "prompt_tokens": [len(p) for p in prompts], "tokens": n, "total_secs": total,
           "tok_per_sec": n / total if total > 0 else 0.0, "ttft_secs": (first[0] - t0) if first else None}
    if args.json:
        print(json.dumps(out))
    else:
        print(f"{out['tok_per_sec']:.1f} tok/s, {total:.2f}s total, TTFT {out['ttft_secs']:.3f}s "
              f"({n} tokens, batch {len(prompts)})")
    return 0


def perplexity(engine, tokens: list[int], progress=None) -> float:
    """exp(mean negative log-likelihood) of tokens[1:], fed one token at a
    time; the log-sum-exp is done in float64 (src/engine.rs:467-544)."""
    import torch
    from .engine import StepRow
    if len(tokens) < 2:
        raise ValueError("Text too short for perplexity (need >= 2 tokens)")
    slot = engine.new_sequence()
    total = 0.0
    try:
        for t in range(len(tokens) - 1):
            logits = engine.step([StepRow(slot, [tokens[t]], [0])])[0].to(torch.float64)
            total += float(torch.logsumexp(logits, 0) - logits[tokens[t + 1]])
            if progress and (t + 1) % 100 == 0:
                progress(t + 1, len(tokens) - 1, math.exp(total / (t + 1)))
    finally:
        engine.release(slot)
    return math.exp(total / (len(tokens) - 1))


def cmd_perplexity(args) -> int:
    engine = _load(args)
    tok = _tokenizer(_model_location(args) if not args.random_weights else None)
    with open(args.file) as f:
        text = f.read()
    ids = _parse_ids(text) if re.fullmatch(r"[\d\s,]+", text) else (
        tok.encode(text, add_special_tokens=False).ids if tok else None)
    if ids is None:
        raise SystemExit("tq: a text file needs a tokenizer.json in the model folder")
    ppl = perplexity(engine, ids, lambda i, n, p: print(f"  [{i}/{n}] PPL: {p:.3f}", file=sys.stderr))
    print(f"Final perplexity: {ppl:.3f} ({len(ids) - 1} tokens)")
    return 0


def cmd_list() -> int:
    from .config import named_shape, shape_names
    for n in shape_names():
        c = named_shape(n)
        print(f"{n}: {c['num_hidden_layers']} layers, hidden {c['hidden_size']}, heads {c['num_attention_heads']}"
              f"/{c['num_key_value_heads']}, vocab {c['vocab_size']}")
    return 0


def cmd_doctor() -> int:
    import torch
    from .csrc import build
    ok = torch.cuda.is_available()
    print(f"CUDA device: {torch.cuda.get_device_name(0) if ok else 'none'}")
    try:
        print(f"C++ compiler: {build.find_cxx()}")
        print(f"host runtime: {build.build('host')}")
    except build.BuildError as e:
        print(f"host runtime: FAILED\n{e}")
        ok = False
    try:
        print(f"nvcc: {build.find_nvcc()}")
        print(f"CUDA library: {build.build('core')}")
    except build.BuildError as e:
        print(f"CUDA library: FAILED\n{e}")
        ok = False
    return 0 if ok else 1


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command in ("chat", "run"):
        return cmd_run(args, interactive=args.command == "chat")
    if args.command == "bench":
        return cmd_bench(args)
    if args.command == "perplexity":
        return cmd_perplexity(args)
    if args.command == "list":
        return cmd_list()
    if args.command == "doctor":
        return cmd_doctor()
    build_parser().print_help()
    return 2

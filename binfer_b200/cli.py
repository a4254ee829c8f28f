"""Command line, in the manner of the reference's ``src/index.ts``.

Same option names and meanings where the reference has them (src/index.ts:9-54,
130-215): positional ``<model>`` and prompt, ``-p/--prompt``, ``--max-tokens``
(100), ``--temperature/--temp`` (0 = greedy), ``--top-k`` (0 = off), ``--top-p``
(1.0 = off), ``--bench`` (prompts of 128/256/512 tokens + 128 generated, :543-586),
``--profile``, ``--dtype``, ``--no-cuda-graphs``, ``-i/--input`` with
``-o/--output`` (one prompt per line, run as one batch, :592-740), ``-q``, ``-v``,
``-h``.  Unknown flags are refused before anything heavy is imported (:57-89).

A prompt is a list of token ids (``12,7,99`` or ``12 7 99``); text needs a
``tokenizer.json`` in the model folder.  ``--tp`` accepts only 1 or ``auto`` (this
engine runs on one GPU); ``--no-cache`` is accepted and has nothing to switch off;
``--chat`` and ``--use-template`` need a tokenizer.
"""
from __future__ import annotations

import os
import sys
import time
from typing import List, Optional

VALUE_FLAGS = {
    "--tp", "--max-tokens", "--dtype", "-p", "--prompt", "--trace", "--temperature", "--temp",
    "--top-k", "--top-p", "-i", "--input", "-o", "--output",
    # additions of this engine
    "--prompt-ids", "--seed", "--repetition-penalty", "--random-weights", "--kv-memory-gb",
    "--kv-pages", "--page-size", "--max-tokens-per-step", "--max-seq-len", "--max-batch-size",
}
BOOL_FLAGS = {
    "--chat", "--bench", "--profile", "--no-cache", "-q", "--quiet", "--help", "-h",
    "--verbose", "-v", "--no-cuda-graphs", "--use-template", "--ignore-eos",
    "--allow-unexpected-tensors",
}

USAGE = """
binfer_b200 - Qwen3 dense inference on one B200

Usage: bin/binfer <model> [prompt] [options]

Options:
  --tp <n|auto>            Tensor parallel degree (only 1 or auto: one GPU)
  --max-tokens <n>         Maximum tokens to generate (default: 100)
  --dtype <type>           bf16 or fp32 (default: bf16)
  -p, --prompt <p>         Prompt: token ids "1,2,3", or text if the model folder has tokenizer.json
  --prompt-ids <ids>       Prompt as token ids
  --chat                   Interactive chat mode (needs tokenizer.json)
  --bench                  Run benchmark (128/256/512-token prompts + 128 generated)
  --profile                Show timing breakdown summary
  --trace <file>           Write a JSON trace of step timings to file
  --no-cache               Accepted for compatibility (no shard cache on one GPU)
  -q, --quiet              Suppress loading output
  -v, --verbose            Show startup timing breakdown
  --no-cuda-graphs         Disable CUDA graph capture for decode
  --use-template           Apply chat template to prompt (needs tokenizer.json)
  --temperature <f>        Sampling temperature (default: 0 = greedy)
  --top-k <n>              Top-k sampling (default: 0 = disabled)
  --top-p <f>              Nucleus sampling threshold (default: 1.0 = disabled)
  --repetition-penalty <f> Penalty on generated tokens (default: 1.0 = disabled)
  --seed <n>               Seed of the sampling stream
  --ignore-eos             Do not stop at the end-of-sequence token
  -i, --input <file>       Input file with prompts (one per line), processed in batch
  -o, --output <file>      Output file for batch results (one per line)
  --random-weights <seed>  Draw random weights for the folder's config.json (no safetensors needed)
  --allow-unexpected-tensors  Warn about tensors the model does not use instead of refusing
  --kv-memory-gb <f>       Memory for the key/value cache (default: 0.9 of what is free
                           after loading, at most max-batch-size x max-seq-len tokens)
  --kv-pages <n>           Size of the cache in pages instead
  --page-size <n>          Tokens per cache page (default: 16)
  --max-tokens-per-step <n>  Token budget of one step (default: 2048)
  --max-seq-len <n>        Longest sequence (default: 4096)
  --max-batch-size <n>     Most requests running at once (default: 64)

Examples:
  bin/binfer /models/Qwen3-8B --prompt-ids 9707,11,1879 --max-tokens 50
  bin/binfer /models/Qwen3-8B -i prompts.txt -o outputs.txt --max-tokens 50
  bin/binfer /models/Qwen3-8B --bench --random-weights 0
"""


class CliError(SystemExit):
    pass


def pre_parse(argv: List[str]) -> Optional[int]:
    """--help and unknown flags, before any heavy import.  Returns an exit code or None."""
    if "--help" in argv or "-h" in argv:
        print(USAGE)
        return 0
    i = 0
    while i < len(argv):
        a = argv[i]
        if a.startswith("-") and not _is_number(a):
            if a not in VALUE_FLAGS and a not in BOOL_FLAGS:
                print(f"Error: Unknown flag '{a}'", file=sys.stderr)
                print("Run with --help to see available options.", file=sys.stderr)
                return 1
            if a in VALUE_FLAGS:
                i += 1
        i += 1
    return None


def _is_number(s: str) -> bool:
    try:
        float(s)
        return True
    except ValueError:
        return False


def parse_args(argv: List[str]) -> dict:
    a = dict(model=None, prompt=None, max_tokens=100, tp="auto", dtype="bf16", chat=False,
             bench=False, profile=False, trace=None, quiet=False, verbose=False, cuda_graphs=True,
             temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=None,
             ignore_eos=False, input=None, output=None, use_template=False, random_weights=None,
             kv_memory_gb=None, kv_pages=None, allow_unexpected_tensors=False, page_size=16, max_tokens_per_step=2048,
             max_seq_len=4096, max_batch_size=64)
    names = {"--max-tokens": ("max_tokens", int), "--tp": ("tp", str), "--dtype": ("dtype", str),
             "-p": ("prompt", str), "--prompt": ("prompt", str), "--prompt-ids": ("prompt", str),
             "--trace": ("trace", str), "--temperature": ("temperature", float),
             "--temp": ("temperature", float), "--top-k": ("top_k", int),
             "--top-p": ("top_p", float), "-i": ("input", str), "--input": ("input", str),
             "-o": ("output", str), "--output": ("output", str), "--seed": ("seed", int),
             "--repetition-penalty": ("repetition_penalty", float),
             "--random-weights": ("random_weights", int), "--kv-memory-gb": ("kv_memory_gb", float),
             "--kv-pages": ("kv_pages", int), "--page-size": ("page_size", int),
             "--max-tokens-per-step": ("max_tokens_per_step", int),
             "--max-seq-len": ("max_seq_len", int), "--max-batch-size": ("max_batch_size", int)}
    flags = {"--chat": "chat", "--bench": "bench", "--profile": "profile", "-q": "quiet",
             "--quiet": "quiet", "-v": "verbose", "--verbose": "verbose",
             "--use-template": "use_template", "--ignore-eos": "ignore_eos",
             "--allow-unexpected-tensors": "allow_unexpected_tensors"}
    i = 0
    while i < len(argv):
        t = argv[i]
        if t in names:
            if i + 1 >= len(argv):
                raise CliError(f"Error: {t} needs a value")
            key, conv = names[t]
            try:
                a[key] = conv(argv[i + 1])
            except ValueError:
                raise CliError(f"Error: bad value for {t}: {argv[i + 1]!r}")
            i += 2
            continue
        if t in flags:
            a[flags[t]] = True
        elif t == "--no-cuda-graphs":
            a["cuda_graphs"] = False
        elif t == "--no-cache":
            pass
        elif a["model"] is None:
            a["model"] = t
        elif a["prompt"] is None:
            a["prompt"] = t
        i += 1
    if a["model"] is None:
        raise CliError("Error: no model given\nRun with --help to see available options.")
    if str(a["tp"]) not in ("auto", "1"):
        raise CliError("Error: --tp must be 1 or auto: this engine runs on one GPU")
    if a["dtype"] not in ("bf16", "bfloat16", "fp32", "float32"):
        raise CliError("Error: --dtype must be bf16 or fp32")
    if a["input"] and not a["output"]:
        raise CliError("Error: -i/--input needs -o/--output")
    return a


class _Tokens:
    """Token ids in and out; text only when the folder has a tokenizer.json."""

    def __init__(self, model_dir: str):
        self.tok = None
        path = os.path.join(model_dir, "tokenizer.json")
        if os.path.exists(path):
            try:
                from tokenizers import Tokenizer
                self.tok = Tokenizer.from_file(path)
            except Exception:                       # noqa: BLE001 - optional convenience
                self.tok = None

    def encode(self, prompt: str) -> List[int]:
        s = prompt.replace(",", " ").split()
        if s and all(p.lstrip("-").isdigit() for p in s):
            return [int(p) for p in s]
        if self.tok is None:
            raise CliError("Error: a text prompt needs tokenizer.json in the model folder; "
                           "give token ids instead (for example --prompt-ids 1,2,3)")
        return self.tok.encode(prompt).ids

    def decode(self, ids: List[int]) -> str:
        if self.tok is None:
            return " ".join(str(i) for i in ids)
        return self.tok.decode(ids)


def _bench(engine, args, log) -> None:
    """src/index.ts:543-586: prompts of 128/256/512 tokens, 128 generated, batch 1."""
    import torch
    log("\nRunning benchmark...\n")
    vocab = engine.spec.vocab_size
    g = torch.Generator().manual_seed(0)
    for n in (128, 256, 512):
        ids = torch.randint(0, vocab, (n,), generator=g).tolist()
        t0 = time.perf_counter()
        out = engine.generate(ids, max_tokens=128, ignore_eos=True)
        dt = time.perf_counter() - t0
        print(f"Prompt: {n} tokens, Generated: {len(out)} tokens, Time: {dt:.2f}s, "
              f"Speed: {len(out) / dt:.1f} tok/s")


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    code = pre_parse(argv)
    if code is not None:
        return code
    try:
        args = parse_args(argv)
    except CliError as e:
        print(e, file=sys.stderr)
        return 1
    t_start = time.perf_counter()
    log = (lambda *a, **k: None) if args["quiet"] else (lambda *a, **k: print(*a, **k, flush=True))

    # heavy imports only now
    from .config.registry import load_config
    from .engine.engine import Engine
    from .profiling import Profiler

    if not os.path.isdir(args["model"]):
        print(f"Error: model folder {args['model']!r} not found (there is no network here; "
              f"give a local folder)", file=sys.stderr)
        return 1
    log(f"Loading {args['model']} ...")
    model = args["model"]
    kw = dict(dtype=args["dtype"], max_kv_memory_gb=args["kv_memory_gb"],
              num_pages=args["kv_pages"], page_size=args["page_size"],
              max_seq_len=args["max_seq_len"], max_batch_size=args["max_batch_size"],
              max_tokens_per_step=args["max_tokens_per_step"],
              cuda_graphs=args["cuda_graphs"] and not args["profile"] and not args["trace"])
    try:
        if args["random_weights"] is not None:
            engine = Engine(load_config(model), random_seed=args["random_weights"], **kw)
        else:
            engine = Engine(model, allow_unexpected_tensors=args["allow_unexpected_tensors"],
                            **kw)
    except (ValueError, FileNotFoundError, RuntimeError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    engine.warm_up()                  # the decode graphs, before the first request
    t_loaded = time.perf_counter()
    if args["verbose"]:
        log(f"  startup: {t_loaded - t_start:.2f}s (model + cache on device, decode graphs)")
    tokens = _Tokens(model)
    prof = Profiler(engine) if (args["profile"] or args["trace"]) else None
    sampling = dict(max_tokens=args["max_tokens"], temperature=args["temperature"],
                    top_k=args["top_k"], top_p=args["top_p"],
                    repetition_penalty=args["repetition_penalty"], seed=args["seed"],
                    ignore_eos=args["ignore_eos"])
    try:
        if args["bench"]:
            _bench(engine, args, log)
        elif args["input"]:
            with open(args["input"]) as f:
                prompts = [tokens.encode(line) for line in f.read().splitlines() if line.strip()]
            log(f"Processing {len(prompts)} prompts with true GPU batching...")
            t0 = time.perf_counter()
            outs = engine.generate(prompts, **sampling)
            dt = time.perf_counter() - t0
            total = sum(len(o) for o in outs)
            with open(args["output"], "w") as f:
                f.write("\n".join(tokens.decode(o) for o in outs) + "\n")
            log(f"\nCompleted {len(prompts)} prompts in {dt:.2f}s")
            log(f"Total: {total} tokens, {total / dt:.1f} tok/s")
            log(f"Results written to {args['output']}")
        elif args["chat"]:
            if tokens.tok is None:
                raise CliError("Error: --chat needs tokenizer.json in the model folder")
            while True:
                try:
                    line = input("> ")
                except (EOFError, KeyboardInterrupt):
                    break
                if not line.strip():
                    continue
                out = engine.generate(tokens.encode(line), **dict(sampling, max_tokens=512))
                print(tokens.decode(out))
        else:
            if args["prompt"] is None:
                raise CliError("Error: no prompt given (token ids, for example --prompt-ids 1,2,3)")
            ids = tokens.encode(args["prompt"])
            t0 = time.perf_counter()
            out = engine.generate(ids, **sampling)
            dt = time.perf_counter() - t0
            print(tokens.decode(out))
            log(f"[{len(out)} tokens, {dt:.2f}s, {len(out) / dt:.1f} tok/s]")
    except CliError as e:
        print(e, file=sys.stderr)
        return 1
    except (ValueError, RuntimeError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    if prof is not None:
        if args["profile"]:
            print(prof.report())
        if args["trace"]:
            prof.write_trace(args["trace"])
            log(f"Trace written to {args['trace']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())

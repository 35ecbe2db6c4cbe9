"""Command line in the manner of the reference's (Daisi.Llogos.Cli/Program.cs:444-576).

Same option names and meanings where the reference has them: ``--model/-m``, ``--prompt/-p``,
``--max-tokens/-n`` (256), ``--max-context`` (2048), ``--temperature/-t`` (0.7, 0 = greedy),
``--top-k`` (40), ``--top-p`` (0.9), ``--repeat-penalty`` (1.1), ``--seed``, ``--bench``,
``--help/-h``.  ``--model`` is a folder with config.json and safetensors.  Text is outside this
library: ``--prompt`` is turned into ids by a byte stand-in (``byte % vocab``) and output is token
ids; ``--prompt-ids`` and ``--prompt-file`` give ids directly.  ``--backend`` is replaced by ``--dtype``.
``--ignore-eos``, ``--min-p``, ``--typical-p``, ``--frequency-penalty`` and ``--presence-penalty`` set the
fields of the same meaning in the reference's GenerationParams (Inference/GenerationParams.cs:32-53).
"""
from __future__ import annotations

import argparse
import sys
import time


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="daisi-llogos", description="B200 inference for dense Llama / Qwen decoders")
    ap.add_argument("--model", "-m", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--prompt", "-p", help="prompt text (bytes stand in for tokens)")
    ap.add_argument("--prompt-ids", help="prompt as comma-separated token ids; ';' separates several prompts")
    ap.add_argument("--max-tokens", "-n", type=int, default=256, help="maximum tokens to generate (default 256)")
    ap.add_argument("--max-context", type=int, default=2048, help="maximum context length (default 2048)")
    ap.add_argument("--temperature", "-t", type=float, default=0.7, help="sampling temperature, 0 = greedy (default 0.7)")
    ap.add_argument("--top-k", type=int, default=40, help="top-k sampling, 0 = disabled (default 40)")
    ap.add_argument("--top-p", type=float, default=0.9, help="nucleus sampling (default 0.9)")
    ap.add_argument("--repeat-penalty", type=float, default=1.1, help="repetition penalty (default 1.1)")
    ap.add_argument("--seed", type=int, default=None, help="random seed for reproducibility")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="compute type")
    ap.add_argument("--bench", action="store_true", help="run benchmark (prefill + decode timing)")
    ap.add_argument("--random-config", help="config.json of a model to initialise randomly instead of --model")
    ap.add_argument("--batch", type=int, default=1, help="with --bench: copies of the prompt decoded together")
    ap.add_argument("--prompt-file", help="file with one prompt per line, token ids separated by commas or blanks")
    ap.add_argument("--ignore-eos", action="store_true",
                    help="never draw or stop at the end-of-sequence tokens (the reference's PreventEOS)")
    ap.add_argument("--min-p", type=float, default=0.0, help="min-p sampling, 0 = disabled (default 0)")
    ap.add_argument("--typical-p", type=float, default=1.0, help="typical-p sampling, 1 = disabled (default 1)")
    ap.add_argument("--frequency-penalty", type=float, default=0.0, help="frequency penalty (default 0)")
    ap.add_argument("--presence-penalty", type=float, default=0.0, help="presence penalty (default 0)")
    return ap


def _ids_from_text(text: str, vocab: int):
    return [b % vocab for b in text.encode("utf-8")] or [0]


def main(argv=None) -> int:
    args = _parser().parse_args(argv)
    if not args.model and not args.random_config:
        print("error: --model <folder> is required (or --random-config <config.json>)", file=sys.stderr)
        return 2
    from .api import LlogosModel
    from .sampling.params import GenerationParams

    t_load = time.perf_counter()
    kw = dict(dtype=args.dtype, max_context=args.max_context, max_batch=max(1, args.batch))
    if args.model:
        model = LlogosModel.load(args.model, **kw)
    else:
        import json
        with open(args.random_config) as f:
            model = LlogosModel.random(json.load(f), seed=args.seed or 0, **kw)
    load_ms = (time.perf_counter() - t_load) * 1e3
    vocab = model.model.spec.vocab_size

    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts = [[int(x) for x in line.replace(",", " ").split()] for line in f if line.strip()]
        if not prompts:
            print(f"error: {args.prompt_file} holds no prompt", file=sys.stderr)
            return 2
    elif args.prompt_ids:
        prompts = [[int(x) for x in part.split(",") if x.strip()] for part in args.prompt_ids.split(";")]
    else:
        text = args.prompt if args.prompt is not None else ("The meaning of life is" if args.bench else None)
        if text is None:
            print("error: --prompt <text>, --prompt-ids or --prompt-file is required unless --bench", file=sys.stderr)
            return 2
        prompts = [_ids_from_text(text, vocab)]

    if args.bench:
        prompts = [prompts[0]] * max(1, args.batch)
        greedy = GenerationParams.greedy_params(args.max_tokens, stop_tokens=())
        model.generate(prompts, GenerationParams.greedy_params(min(4, args.max_tokens), stop_tokens=()))   # warm-up
        r = model.generate(prompts, greedy)
        total_ms = (r.prefill_seconds + r.decode_seconds) * 1e3
        print("=== Benchmark Results ===", file=sys.stderr)
        print(f"  Prefill:  {r.prompt_tokens:6d} tokens in {r.prefill_seconds * 1e3:8.1f} ms  ({r.prefill_tokens_per_second:8.1f} tok/s)", file=sys.stderr)
        print(f"  Decode:   {r.generated_tokens:6d} tokens in {r.decode_seconds * 1e3:8.1f} ms  ({r.decode_tokens_per_second:8.1f} tok/s)", file=sys.stderr)
        print(f"  Total:    {r.prompt_tokens + r.generated_tokens:6d} tokens in {total_ms:8.1f} ms", file=sys.stderr)
        print(f"  Load:     {load_ms:8.1f} ms", file=sys.stderr)
        return 0

    params = GenerationParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                              top_p=args.top_p, repetition_penalty=args.repeat_penalty, seed=args.seed,
                              min_p=args.min_p, typical_p=args.typical_p, frequency_penalty=args.frequency_penalty,
                              presence_penalty=args.presence_penalty, prevent_eos=args.ignore_eos)
    first = [True] * len(prompts)

    def show(i, tok):
        if len(prompts) == 1:
            sys.stdout.write(("" if first[0] else " ") + str(tok))
            sys.stdout.flush()
            first[0] = False

    r = model.generate(prompts, params, on_token=show)
    if len(prompts) == 1:
        print()
    else:
        for toks in r.tokens:
            print(" ".join(str(t) for t in toks))
    print(f"\n[prefill: {r.prompt_tokens} tokens, {r.prefill_tokens_per_second:.1f} tok/s | "
          f"decode: {r.generated_tokens} tokens, {r.decode_tokens_per_second:.1f} tok/s]", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())

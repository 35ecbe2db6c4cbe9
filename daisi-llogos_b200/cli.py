"""Command line in the manner of the reference's (Daisi.Llogos.Cli/Program.cs:444-576).

Same option names and meanings where the reference has them: ``--model/-m``, ``--prompt/-p``,
``--max-tokens/-n`` (256), ``--max-context`` (2048), ``--temperature/-t`` (0.7, 0 = greedy),
``--top-k`` (40), ``--top-p`` (0.9), ``--repeat-penalty`` (1.1), ``--seed``, ``--bench``,
``--help/-h``.  ``--model`` is a folder with config.json and safetensors.  Text is outside this
library: ``--prompt`` is turned into ids by a byte stand-in (``byte % vocab``) and output is token
ids; ``--prompt-ids`` and ``--prompt-file`` give ids directly.  ``--backend`` is replaced by ``--dtype``.
``--ignore-eos``, ``--min-p``, ``--typical-p``, ``--frequency-penalty`` and ``--presence-penalty`` set the
fields of the same meaning in the reference's GenerationParams (Inference/GenerationParams.cs:32-53).

``--bench`` prints the reference's four lines (``Prefill:``, ``Decode:``, ``Total:``, ``Load:``,
Program.cs:283-297, which its dashboard parses) and, below them, what the reference does not measure: batch
and context, the bytes a decode step had to read, the operations of the prompt step, and both as fractions of
the measured peaks.  ``--batch``, ``--prompt-len`` (a number, or ``LOW:HIGH`` for lengths drawn uniformly per
sequence) and ``--context`` (decode until every sequence holds that many tokens) select the workload.
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
    ap.add_argument("--batch", type=int, default=1, help="with --bench: sequences decoded together")
    ap.add_argument("--prompt-len", help="with --bench: random prompts of this many tokens, or LOW:HIGH for lengths "
                                         "drawn uniformly per sequence (instead of --prompt)")
    ap.add_argument("--context", type=int, default=0,
                    help="with --bench: decode until every sequence holds this many tokens (sets --max-context)")
    ap.add_argument("--peaks", help="JSON file with hbm_gbs and bf16_tflops to compute the roofline fractions against")
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

    import json
    t_load = time.perf_counter()
    max_context = args.max_context
    if args.bench and args.context > 0:
        max_context = args.context
    if args.model:
        with open(f"{args.model}/config.json") as f:
            limit = json.load(f).get("max_position_embeddings")
    else:
        with open(args.random_config) as f:
            limit = json.load(f).get("max_position_embeddings")
    if isinstance(limit, int) and max_context > limit:
        if args.bench and args.context > 0 or "--max-context" in (argv if argv is not None else sys.argv):
            print(f"error: a context of {max_context} tokens exceeds the model's max_position_embeddings ({limit})", file=sys.stderr)
            return 2
        max_context = limit              # the default of 2048 gives way to a model with fewer positions
    kw = dict(dtype=args.dtype, max_context=max_context, max_batch=max(1, args.batch))
    if args.model:
        model = LlogosModel.load(args.model, **kw)
    else:
        with open(args.random_config) as f:
            model = LlogosModel.random(json.load(f), seed=args.seed or 0, **kw)
    load_ms = (time.perf_counter() - t_load) * 1e3
    vocab = model.model.spec.vocab_size

    if args.bench and args.prompt_len:
        import random
        lo, _, hi = args.prompt_len.partition(":")
        lo, hi = int(lo), int(hi or lo)
        if not 0 < lo <= hi < max_context:
            print(f"error: --prompt-len {args.prompt_len} must lie between 1 and the context ({max_context})", file=sys.stderr)
            return 2
        rng = random.Random(args.seed or 0)
        prompts = [[rng.randrange(vocab) for _ in range(rng.randint(lo, hi))] for _ in range(max(1, args.batch))]
    elif args.prompt_file:
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
        if not args.prompt_len:
            prompts = [prompts[0]] * max(1, args.batch)
        n_new = max_context if args.context > 0 else args.max_tokens          # with --context the cache's limit ends a sequence
        b = model.benchmark(prompts, n_new, peaks_file=args.peaks)
        total_ms = (b.prefill_seconds + b.decode_seconds) * 1e3
        # the reference's four lines (Daisi.Llogos.Cli/Program.cs:283-297)
        print("=== Benchmark Results ===", file=sys.stderr)
        print(f"  Prefill:  {b.prompt_tokens:6d} tokens in {b.prefill_seconds * 1e3:8.1f} ms  ({b.prefill_tokens_per_second:8.1f} tok/s)", file=sys.stderr)
        print(f"  Decode:   {b.generated_tokens:6d} tokens in {b.decode_seconds * 1e3:8.1f} ms  ({b.decode_tokens_per_second:8.1f} tok/s)", file=sys.stderr)
        print(f"  Total:    {b.prompt_tokens + b.generated_tokens:6d} tokens in {total_ms:8.1f} ms", file=sys.stderr)
        print(f"  Load:     {load_ms:8.1f} ms", file=sys.stderr)
        # beyond them: what the steps had to move and compute, against the measured peaks
        pk = b.peaks
        print(f"  Batch:    {b.batch} sequences, prompts of {min(b.prompt_lengths)} to {max(b.prompt_lengths)} tokens, "
              f"longest sequence at the end {max(b.final_lengths)} tokens", file=sys.stderr)
        if b.decode_seconds > 0 and b.decode_steps:
            print(f"  Decode step: {b.decode_seconds / b.decode_steps * 1e3:8.3f} ms mean over {b.decode_steps} steps, "
                  f"{b.decode_bytes_per_step / 1e9:7.3f} GB to read per step, {b.decode_gb_per_second:7.1f} GB/s = "
                  f"{100 * b.decode_fraction_of_copy_bandwidth:5.1f} % of {pk['hbm_gbs']:.0f} GB/s ({pk['source']} copy bandwidth)",
                  file=sys.stderr)
        if b.prefill_seconds > 0:
            print(f"  Prompt step: {b.prompt_step_flops / 1e12:8.3f} TFLOP, {b.prompt_tflops:7.1f} TFLOP/s = "
                  f"{100 * b.prompt_fraction_of_matrix_peak:5.1f} % of {pk['bf16_tflops']:.0f} TFLOP/s ({pk['source']} bfloat16 matrix "
                  f"throughput)", file=sys.stderr)
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

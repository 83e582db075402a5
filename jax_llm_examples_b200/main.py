"""Command line: generate from a model folder, or from a preset with seeded random weights.

The reference's ``llama4/main.py`` takes no options: the checkpoint path, the prompts, 32 greedy
decode steps and the tokenizer are constants in the file (llama4/main.py:42-80).  The same run here
is ``python -m jax_llm_examples_b200.main --model DIR --prompt "..."``, with those constants as
options; ``--max-new-tokens`` defaults to the reference's 32 steps and sampling to its argmax.
Option names follow the reference where it has them: ``--temperature`` / ``--top-k`` are
``sample_temp`` / ``sample_topk`` of gpt_oss (gpt_oss/gpt_oss_jax/model.py:1125), and the serving
mains' flags are argparse too (serving/main_serving_gemma4.py:163-171).
"""

from __future__ import annotations

import argparse
import random
import sys
import tempfile
import time
from pathlib import Path


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="jax_llm_examples_b200.main", description=__doc__.split("\n\n")[0])
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors (ckpt_path of llama4/main.py)")
    src.add_argument("--preset", help="a named configuration with random weights (see --seed)")
    ap.add_argument("--layers", type=int, help="with --preset: number of layers")
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights, random prompts and sampling")
    ap.add_argument("--write-model", metavar="DIR", help="with --preset: write the random model folder here and exit")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompt", action="append", default=[], help="text prompt (needs tokenizer.json in --model)")
    ap.add_argument("--prompt-ids", action="append", default=[], help='token ids, e.g. "1,2,3"')
    ap.add_argument("--random-prompts", type=int, default=0, help="number of random prompts")
    ap.add_argument("--prompt-len", type=int, default=32, help="length of each random prompt")
    ap.add_argument("--max-new-tokens", type=int, default=32, help="decode steps (32 in llama4/main.py)")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = argmax (the reference's Llama 4 decoding)")
    ap.add_argument("--top-k", type=int, default=0, help="sample among the k most likely tokens; 0 = all")
    ap.add_argument("--eos", type=int, action="append", default=None, help="token id that ends a request (default: config.json's)")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=None, help="cache pool in tokens (default: what the prompts need)")
    ap.add_argument("--num-pages", type=int, default=None, help="the same pool given in pages of --page-size tokens")
    ap.add_argument("--max-tokens-per-step", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--max-live", type=int, default=None, help="most requests in the cache at a time")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--profile-kernels", action="store_true",
                    help="time every kernel launch with CUDA events and print the times by kernel and by op group")
    args = ap.parse_args(argv)

    import jax_llm_examples_b200 as J

    if args.preset:
        overrides = {"num_hidden_layers": args.layers} if args.layers else {}
        cfg_json = J.preset(args.preset, **overrides)
        if args.write_model:
            J.write_random_model(args.write_model, cfg_json, args.seed)
            print(f"wrote {args.write_model}")
            return 0
        model = J.random_model(cfg_json, args.seed, args.dtype)
        model_dir = None
    else:
        model_dir = Path(args.model)
        model = J.load_model(model_dir, args.dtype)

    prompts: list[list[int]] = [[int(t) for t in s.replace(" ", "").split(",") if t] for s in args.prompt_ids]
    tokenizer = None
    if args.prompt:
        if model_dir is None or not (model_dir / "tokenizer.json").is_file():
            ap.error("--prompt needs a model folder with tokenizer.json; use --prompt-ids or --random-prompts")
        from .tokenizer import encode_chat, load_tokenizer

        tokenizer = load_tokenizer(model_dir / "tokenizer.json", model_dir / "tokenizer_config.json")
        prompts += [encode_chat(tokenizer, text) for text in args.prompt]
    rng = random.Random(args.seed)
    prompts += [[rng.randrange(model.vocab_size) for _ in range(args.prompt_len)] for _ in range(args.random_prompts)]
    if not prompts:
        ap.error("no prompts: give --prompt, --prompt-ids or --random-prompts")

    eos = tuple(args.eos) if args.eos is not None else tuple(getattr(model.config, "eos_token_ids", ()) or ())
    params = J.SamplingParams(temperature=args.temperature, top_k=args.top_k, seed=args.seed,
                              max_new_tokens=args.max_new_tokens, eos_token_ids=eos)
    ps = args.page_size
    if args.num_pages is not None and args.max_tokens is None:
        args.max_tokens = args.num_pages * ps
    max_tokens = args.max_tokens or sum(-(-(len(p) + args.max_new_tokens) // ps) * ps for p in prompts)
    gen = J.Generator(model, max_tokens=max_tokens, page_size=ps, max_slots=max(len(prompts), 1),
                      max_tokens_per_step=args.max_tokens_per_step, max_live=args.max_live, seed=args.seed,
                      profile="kernels" if args.profile_kernels else args.verbose)
    t0 = time.time()
    outputs = gen.generate(prompts, params)
    dt = time.time() - t0
    print("Responses:")
    for p, o in zip(prompts, outputs):
        print(tokenizer.decode(o) if tokenizer else " ".join(map(str, o)))
        print("-" * 80)
    if args.profile_kernels:
        print("time by kernel entry point:\n" + gen.kernel_timer.report("kernel"), file=sys.stderr)
        print("time by op group:\n" + gen.kernel_timer.report("scope"), file=sys.stderr)
    if args.verbose:
        n = sum(map(len, outputs))
        print(f"{n} tokens in {dt:.3f} s ({n / dt:.1f} tok/s), {gen.scheduler.step_count} steps, "
              f"{sum(r.preemptions for r in gen.scheduler.finished)} preemptions", file=sys.stderr)
        pre = [(p_, t) for p_, d, t in gen.step_times if p_ > 0]
        dec = [(d, t) for p_, d, t in gen.step_times if p_ == 0 and d > 0]
        if pre:
            print(f"steps with prompt tokens: {sum(p_ for p_, _ in pre)} tokens in {sum(t for _, t in pre):.3f} s "
                  f"({sum(p_ for p_, _ in pre) / sum(t for _, t in pre):.0f} tok/s)", file=sys.stderr)
        if dec:
            print(f"decode-only steps: {len(dec)} steps, {sum(d for d, _ in dec)} tokens in {sum(t for _, t in dec):.3f} s "
                  f"({sum(d for d, _ in dec) / sum(t for _, t in dec):.1f} tok/s, {1e3 * sum(t for _, t in dec) / len(dec):.2f} ms/step)",
                  file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())

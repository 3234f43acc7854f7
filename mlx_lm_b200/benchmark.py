"""``python -m mlx_lm_b200 benchmark``: prompt and generation speed of a model folder, with the options and the
report of mlx-lm's benchmark (mlx_lm/benchmark.py:13-180): seeded random prompt tokens, end-of-sequence
disabled, one warm-up run, then ``--num-trials`` timed runs and their averages.  A batch of one runs through
``stream_generate``, larger batches through ``batch_generate``."""

from __future__ import annotations

import argparse
import time

import torch

from .generate import batch_generate, load, stream_generate


def setup_arg_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="mlx_lm_b200.benchmark", description="LLM benchmarking script")
    p.add_argument("--model", type=str, required=True, help="The path to the local model directory.")
    p.add_argument("--prompt-tokens", "-p", default=512, type=int, help="Length of prompt")
    p.add_argument("--generation-tokens", "-g", default=1024, type=int, help="Length of completion")
    p.add_argument("--batch-size", "-b", default=1, type=int, help="Batch size")
    p.add_argument("--num-trials", "-n", default=5, type=int, help="Number of timing trials")
    p.add_argument("--prefill-step-size", default=2048, type=int, help="Tokens of a prompt run per step")
    p.add_argument("--delay", type=float, default=0, help="Seconds to wait between trials")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    return p


def main(argv=None) -> None:
    args = setup_arg_parser().parse_args(argv)
    model, tokenizer, config = load(args.model, return_config=True, dtype=args.dtype)
    tokenizer.eos_token_ids = set()      # no early stop
    g = torch.Generator().manual_seed(0)
    vocab = int(config["vocab_size"])
    prompts = torch.randint(0, vocab, (args.batch_size, args.prompt_tokens), generator=g).tolist()

    def single_bench():
        response = None
        for response in stream_generate(model, tokenizer, prompts[0], max_tokens=args.generation_tokens,
                                        prefill_step_size=args.prefill_step_size):
            pass
        return response

    def batch_bench():
        return batch_generate(model, tokenizer, prompts, max_tokens=args.generation_tokens,
                              prefill_step_size=args.prefill_step_size, completion_batch_size=args.batch_size,
                              prefill_batch_size=args.batch_size).stats

    bench = single_bench if args.batch_size == 1 else batch_bench
    print("Running warmup..")
    bench()
    keys = ["prompt_tps", "generation_tps", "peak_memory"]
    print(f"Timing with prompt_tokens={args.prompt_tokens}, generation_tokens={args.generation_tokens}, "
          f"batch_size={args.batch_size}.")
    responses = []
    for i in range(args.num_trials):
        if args.delay > 0:
            time.sleep(args.delay)
        tic = time.perf_counter()
        r = bench()
        toc = time.perf_counter()
        responses.append(r)
        print(f"Trial {i + 1}:  " + ", ".join(f"{k}={getattr(r, k):.3f}" for k in keys) + f", total_time={toc - tic:.3f}")
    print("Averages: " + ", ".join(f"{k}={sum(getattr(r, k) for r in responses) / len(responses):.3f}" for k in keys))


if __name__ == "__main__":
    main()

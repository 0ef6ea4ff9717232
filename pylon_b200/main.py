"""Command line of the engine: token ids in, token ids out.

raun6k/Pylon's ``main.py`` starts its HTTP server and takes no flags; its options are
``PYLON_*`` environment variables (src/pylon/main.py:13-46, src/pylon/config.py:87-112).
This engine has no server, so the command line generates directly; the engine options keep
Pylon's names (``--prefill-chunk-size`` for ``PYLON_PREFILL_CHUNK_SIZE`` and so on, and the
environment variables themselves are read as defaults), and the sampling options are the
fields of Pylon's ``Sampling`` (src/pylon/api/types.py:6-9).

    python main.py --model DIR --prompt-ids prompts.json --max-new-tokens 32 --temperature 0
    python main.py --random-weights config.json --seed 0 --write-model DIR     # random-weights mode
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path
from typing import Optional, Sequence


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="pylon_b200", description="Generate token ids with a Qwen3 model on one B200.")
    source = parser.add_argument_group("model")
    source.add_argument("--model", help="folder with config.json and model.safetensors")
    source.add_argument("--random-weights", metavar="CONFIG_JSON", help="a config.json; weights are drawn from --seed")
    source.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    source.add_argument("--write-model", metavar="DIR", help="with --random-weights: write the model folder there (and exit if no prompts are given)")
    source.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="bfloat16: serving kernels; float32: everything in true 32-bit")
    prompts = parser.add_argument_group("prompts (token ids)")
    prompts.add_argument("--prompt-ids", metavar="FILE", help="JSON: a list of token-id lists ('-' reads standard input)")
    prompts.add_argument("--prompt-len", type=int, help="instead of a file: random prompts of this many tokens")
    prompts.add_argument("--num-prompts", type=int, default=1, help="how many random prompts")
    sampling = parser.add_argument_group("sampling (raun6k/Pylon's Sampling fields)")
    sampling.add_argument("--max-new-tokens", type=int, default=256)
    sampling.add_argument("--temperature", type=float, default=0.2)
    sampling.add_argument("--top-p", type=float, default=0.95)
    sampling.add_argument("--sample-seed", type=int, default=None, help="seed of the draws (each request gets its own stream)")
    sampling.add_argument("--ignore-eos", action="store_true", help="generate max-new-tokens tokens whatever is drawn")
    engine = parser.add_argument_group("engine (raun6k/Pylon's PYLON_* options; the environment variables are the defaults)")
    engine.add_argument("--prefill-chunk-size", type=int, default=None, help="PYLON_PREFILL_CHUNK_SIZE: prompt tokens per step")
    engine.add_argument("--max-batch-size", type=int, default=None, help="PYLON_MAX_BATCH_SIZE: requests running at a time")
    engine.add_argument("--max-queue-size", type=int, default=None, help="PYLON_MAX_QUEUE_SIZE: requests waiting at a time")
    engine.add_argument("--max-gpu-utilization", type=float, default=None, help="PYLON_MAX_GPU_UTILIZATION: share of GPU memory the engine may use")
    engine.add_argument("--admit-skip", type=int, default=None, help="PYLON_ADMIT_SKIP: how many waiting requests may pass one that does not fit")
    graphs = engine.add_mutually_exclusive_group()
    graphs.add_argument("--cuda-graphs", dest="cuda_graphs", action="store_true", default=None, help="PYLON_CUDA_GRAPHS: replay decode steps from CUDA graphs")
    graphs.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false")
    ahead = engine.add_mutually_exclusive_group()
    ahead.add_argument("--run-ahead", dest="run_ahead", action="store_true", default=None,
                       help="PYLON_B200_RUN_AHEAD: queue the next step before waiting for the last one's tokens (the default)")
    ahead.add_argument("--no-run-ahead", dest="run_ahead", action="store_false")
    engine.add_argument("--page-size", type=int, default=None, help="tokens per cache page (default 256)")
    engine.add_argument("--max-cache-tokens", type=int, default=None, help="size of the cache pool in tokens (default: from free memory)")
    engine.add_argument("--max-context", type=int, default=None, help="longest request, prompt plus new tokens")
    return parser


def read_prompts(args: argparse.Namespace, vocab_size: int) -> list[list[int]]:
    if args.prompt_ids:
        text = sys.stdin.read() if args.prompt_ids == "-" else Path(args.prompt_ids).read_text()
        data = json.loads(text)
        if data and isinstance(data[0], int):
            data = [data]
        return [[int(token) for token in prompt] for prompt in data]
    if args.prompt_len:
        import numpy as np

        rng = np.random.default_rng(args.seed)
        return [rng.integers(0, vocab_size, size=args.prompt_len).tolist() for _ in range(args.num_prompts)]
    return []


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if bool(args.model) == bool(args.random_weights):
        print("give exactly one of --model and --random-weights", file=sys.stderr)
        return 2

    from pylon_b200.config import EngineConfig
    from pylon_b200.config.registry import architecture_of

    scratch = None
    model_dir = args.model
    if args.random_weights:
        from pylon_b200.weights import write_random_model

        data = json.loads(Path(args.random_weights).read_text())
        model_config = architecture_of(data).config_class.from_dict(data)
        if args.write_model:
            model_dir = args.write_model
        else:
            scratch = tempfile.TemporaryDirectory(prefix="pylon_b200_random_")
            model_dir = scratch.name
        write_random_model(model_config, args.seed, model_dir, dtype="bfloat16")
        print(f"wrote random model (seed {args.seed}) to {model_dir}", file=sys.stderr)
    vocab_size = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    prompts = read_prompts(args, vocab_size)
    if not prompts:
        if args.random_weights and args.write_model:
            return 0
        print("no prompts: give --prompt-ids FILE or --prompt-len N", file=sys.stderr)
        return 2

    import torch

    if not torch.cuda.is_available():
        print("pylon_b200 needs a CUDA device (NVIDIA B200); none is visible", file=sys.stderr)
        return 1
    from pylon_b200.engine import Engine
    from pylon_b200.sampling import SamplingParams

    config = EngineConfig.from_env(
        None, dtype=args.dtype, prefill_chunk_size=args.prefill_chunk_size, max_batch_size=args.max_batch_size,
        max_queue_size=args.max_queue_size, max_gpu_utilization=args.max_gpu_utilization, admit_skip=args.admit_skip,
        cuda_graphs=args.cuda_graphs, run_ahead=args.run_ahead, page_size=args.page_size, max_cache_tokens=args.max_cache_tokens, max_context=args.max_context,
        seed=args.sample_seed,
    )
    engine = Engine(model_dir, config)
    params = SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_p=args.top_p,
                            seed=args.sample_seed, ignore_eos=args.ignore_eos)
    # one seed for all: give each request its own stream derived from it
    per_prompt = [params if args.sample_seed is None else SamplingParams(**{**params.__dict__, "seed": args.sample_seed + i}) for i in range(len(prompts))]
    results = engine.generate(prompts, per_prompt)
    for index, result in enumerate(results):
        print(json.dumps({
            "request": index, "prompt_tokens": result.prompt_tokens, "output_ids": result.output_ids, "finish_reason": result.finish_reason,
            "queue_seconds": round(result.queue_seconds, 6), "prefill_seconds": round(result.prefill_seconds, 6),
            "first_token_seconds": None if result.first_token_seconds is None else round(result.first_token_seconds, 6),
            "elapsed_seconds": round(result.elapsed_seconds, 6),
        }))
    if scratch is not None:
        scratch.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())

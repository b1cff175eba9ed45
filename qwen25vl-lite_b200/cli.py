"""Command line of the engine: ``qwen25vl-lite generate ...`` (also ``python -m
qwen25vl_lite.cli``), in the manner of the reference's CLI (src/qwen25vl_lite/cli.py:630-786).

``generate`` keeps the reference's option names and meanings where this engine has the
feature: ``--model --dtype --num-blocks --block-size --max-num-seqs
--max-num-batched-tokens --max-model-len --no-chunked-prefill --prompt-token-ids
--temperature --top-p --max-tokens`` (cli.py:634-673, 706-713); as there, a missing
``--prompt-token-ids`` prints a message and exits with 2 and the result is the printed list
of generated ids (cli.py:267-278).  Added: ``--top-k --min-p --seed --ignore-eos``;
``--random-weights --weights-seed S`` (``--model`` then only has to hold a config.json: the
weights are drawn on the device from the seed); ``random-model`` (writes a model folder from a
config and a seed), ``replay`` (trace replay) and ``bench`` (one prefill and a run of decode
steps, timed).  The reference's quantisation, vision, prefix-cache, backend and server options
have no counterpart here.
"""

from __future__ import annotations

import argparse
import json
import sys


def _add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True, help="folder with config.json and safetensors")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    p.add_argument("--num-blocks", type=int, default=2048)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--max-num-seqs", type=int, default=8)
    p.add_argument("--max-num-batched-tokens", type=int, default=4096)
    p.add_argument("--max-model-len", type=int, default=32768)
    p.add_argument("--no-chunked-prefill", action="store_true")
    p.add_argument("--random-weights", action="store_true",
                   help="draw the weights from --weights-seed; --model then names a config.json or a folder with one")
    p.add_argument("--weights-seed", type=int, default=0)


def _llm(args):
    from .engine.llm import LLM

    options = dict(dtype=args.dtype, device=args.device, num_blocks=args.num_blocks, block_size=args.block_size,
                   max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
                   max_model_len=args.max_model_len, enable_chunked_prefill=not args.no_chunked_prefill)
    if args.random_weights:
        from .config.text_config import read_config_json
        return LLM(random_config=read_config_json(args.model), weights_seed=args.weights_seed, **options)
    return LLM(args.model, **options)


def cmd_generate(args) -> int:
    if not args.prompt_token_ids:
        print("--prompt-token-ids is required (this CLI does not bundle a tokenizer)", file=sys.stderr)
        return 2
    from .sampling.params import SamplingParams

    ids = [int(t) for t in args.prompt_token_ids.split(",")]
    llm = _llm(args)
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                            max_tokens=args.max_tokens, seed=args.seed, ignore_eos=args.ignore_eos)
    outs = llm.generate([ids], params)
    print(outs[0].output_token_ids)
    return 0


def cmd_random_model(args) -> int:
    from .weights.random_init import write_random_model

    with open(args.config, "r", encoding="utf-8") as fh:
        config = json.load(fh)
    write_random_model(args.out, config, args.seed, args.storage_dtype)
    print(args.out)
    return 0


def cmd_bench(args) -> int:
    from .engine.benchmark import quick_bench

    need = args.batch * (-(-(args.prompt_len + args.steps + 16) // args.block_size))
    args.num_blocks = max(args.num_blocks, need)
    args.max_num_seqs = max(args.max_num_seqs, args.batch)
    args.max_num_batched_tokens = max(args.max_num_batched_tokens, args.prompt_len)
    args.max_model_len = max(args.max_model_len, args.prompt_len + args.steps + 16)
    print(json.dumps(quick_bench(_llm(args), args.batch, args.prompt_len, args.steps)))
    return 0


def cmd_replay(args) -> int:
    from .engine.trace import make_runner, replay

    runner = make_runner(args.model, args.dtype, args.max_tokens, args.page_size, device=args.device)
    with (open(args.trace, "r", encoding="utf-8") if args.trace != "-" else sys.stdin) as fh:
        replay(fh, runner, args.out)
    return 0


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="qwen25vl-lite", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    p = sub.add_parser("generate", help="one-shot generation from token ids")
    _add_engine_options(p)
    p.add_argument("--prompt-token-ids", default=None, help='comma-separated ids, e.g. "1,2,3"')
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--ignore-eos", action="store_true")
    p.set_defaults(func=cmd_generate)

    p = sub.add_parser("bench", help="time one prefill and a run of decode steps; prints one JSON line")
    _add_engine_options(p)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--prompt-len", type=int, default=2048)
    p.add_argument("--steps", type=int, default=64)
    p.set_defaults(func=cmd_bench, dtype="bfloat16")

    p = sub.add_parser("random-model", help="write a model folder with random weights")
    p.add_argument("--config", required=True, help="a config.json")
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--storage-dtype", default="bfloat16", choices=["float32", "bfloat16"])
    p.set_defaults(func=cmd_random_model)

    p = sub.add_parser("replay", help="feed a trace of token ids through the model and write logits")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--trace", default="-", help="file of JSON lines, or - for standard input")
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, default=4096)
    p.add_argument("--page-size", type=int, default=16)
    p.set_defaults(func=cmd_replay)
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return int(args.func(args))


if __name__ == "__main__":
    sys.exit(main())

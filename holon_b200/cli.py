"""Command line: `holon-b200 generate | random-model | prebuild | models`.

The engine's flags are made from `EngineConfig`'s fields, one flag per field with the field's help line, as the
reference makes `holon serve`'s (core/holon/core/cli.py:52-98); `prebuild` and `models` keep the reference's names
(cli.py:434-456). The reference serves over HTTP and has no one-shot generation command; `generate` stands where
`serve` stands there, takes the sampling settings by their `SamplingParams` names and prints token ids (there is no
tokenizer in this engine).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys

from .config.engine import EngineConfig


def _add_engine_flags(ap: argparse.ArgumentParser) -> None:
    for f in dataclasses.fields(EngineConfig):
        if f.name == "model":
            continue
        flag, help_ = "--" + f.name.replace("_", "-"), f.metadata.get("help", "")
        if f.type in ("bool", bool):
            ap.add_argument(flag, action=argparse.BooleanOptionalAction, default=f.default, help=help_)
        else:
            kind = {"int": int, "float": float, "int | None": int, "str": str}.get(str(f.type), str)
            ap.add_argument(flag, type=kind, default=f.default, help=f"{help_} (default: {f.default})")


def _engine_config(args) -> EngineConfig:
    names = [f.name for f in dataclasses.fields(EngineConfig)]
    return EngineConfig(**{n: getattr(args, n) for n in names})


def _prompts(args) -> list[list[int]]:
    prompts = [[int(t) for t in p.replace(",", " ").split()] for p in args.prompt_ids or []]
    if args.prompt_file:
        with (sys.stdin if args.prompt_file == "-" else open(args.prompt_file)) as f:
            prompts += [json.loads(line) for line in f if line.strip()]
    if not prompts:
        raise SystemExit("generate: give --prompt-ids or --prompt-file")
    return prompts


def cmd_generate(args) -> int:
    import torch
    from .engine import Engine, SamplingParams
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                            max_tokens=args.max_tokens, ignore_eos=args.ignore_eos, seed=args.sampling_seed,
                            stop_token_ids=tuple(args.stop_token_ids or ()), n=args.n, logprobs=args.logprobs,
                            prompt_logprobs=args.prompt_logprobs)
    with torch.inference_mode():
        engine = Engine(_engine_config(args))
        print(f"holon-b200: {engine.memory_report()}", file=sys.stderr, flush=True)
        prompts = _prompts(args)
        if args.n == 1 and args.logprobs is None and args.prompt_logprobs is None:
            for prompt, tokens in zip(prompts, engine.generate(prompts, params)):
                print(json.dumps({"prompt_ids": prompt, "token_ids": tokens}), flush=True)
        else:                                  # several sequences a prompt, or log-probabilities: the streaming calls
            rids = [engine.add(p, params, rid=str(i)) for i, p in enumerate(prompts)]
            out = {(rid, j): {"prompt": i, "index": j, "token_ids": []} for i, rid in enumerate(rids) for j in range(args.n)}
            while engine.has_work():
                for d in engine.step():
                    o = out[(d.rid, d.index)]
                    o["token_ids"] += d.token_ids
                    o["finish_reason"] = d.finish_reason
                    if d.cached_tokens is not None:
                        o["cached_tokens"] = d.cached_tokens
                    for name, lp in (("logprobs", d.logprobs), ("prompt_logprobs", d.prompt_logprobs)):
                        if lp is not None:
                            have = o.setdefault(name, {"token": [], "top_ids": [], "top": []})
                            have["token"] += lp.token
                            have["top_ids"] += lp.top_ids
                            have["top"] += lp.top
            for key in sorted(out, key=lambda k: (int(k[0]), k[1])):
                print(json.dumps(out[key]), flush=True)
        print(f"holon-b200: {json.dumps(engine.stats())}", file=sys.stderr)
        engine.close()
    return 0


def cmd_random_model(args) -> int:
    from .weights import RandomSource, write_model_folder
    with open(args.config) as f:
        config = json.load(f)
    folder = write_model_folder(RandomSource(config, args.seed), args.out)
    print(folder)
    return 0


def cmd_prebuild(args) -> int:
    from .kernels.build import library_path
    print(library_path(create=True))
    return 0


def cmd_models(args) -> int:
    from . import models  # noqa: F401
    from .config.registry import architectures
    print("\n".join(architectures()))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="holon-b200", description="Qwen3 dense inference on one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate token ids for prompts given as token ids")
    g.add_argument("model", help=EngineConfig.__dataclass_fields__["model"].metadata["help"])
    _add_engine_flags(g)
    g.add_argument("--prompt-ids", action="append", help="a prompt as token ids, e.g. '5,17,3' (repeatable)")
    g.add_argument("--prompt-file", help="a file of JSON lists of token ids, one prompt a line ('-': standard input)")
    g.add_argument("--max-tokens", type=int, default=16, help="tokens to generate per prompt")
    g.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--sampling-seed", type=int, default=None, help="SamplingParams.seed of every prompt")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--stop-token-ids", type=int, nargs="*")
    g.add_argument("--n", type=int, default=1, help="sequences per prompt (SamplingParams.n); more than one prints one "
                                                    "line a sequence with its index")
    g.add_argument("--logprobs", type=int, default=None, help="top-k log-probabilities per generated token (0: the token's own)")
    g.add_argument("--prompt-logprobs", type=int, default=None, help="the same per prompt token")
    g.set_defaults(run=cmd_generate)
    r = sub.add_parser("random-model", help="write a model folder (config.json, model.safetensors) with seeded random weights")
    r.add_argument("config", help="a config.json to take the sizes from")
    r.add_argument("out", help="folder to write")
    r.add_argument("--seed", type=int, default=0)
    r.set_defaults(run=cmd_random_model)
    sub.add_parser("prebuild", help="compile the CUDA kernels for sm_100a now").set_defaults(run=cmd_prebuild)
    sub.add_parser("models", help="list the registered architectures").set_defaults(run=cmd_models)
    args = ap.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())

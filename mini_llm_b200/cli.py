"""Command line: complete prompts with a model folder.

In the manner of the reference's ``scripts/complete.py``: the same options with
the same meanings and defaults (``--model``, ``--max-new-tokens 64``,
``--temperature 0.8`` with ``<= 0`` meaning greedy, ``--top-p 0.95``,
``--device``; :45-59), the same interactive commands (``/clear``, ``/history``,
``/exit``, ``/quit``; :156-180), and prompts trimmed from the left to
``n_positions - max_new_tokens`` tokens (:92-110).  That script generates
through another library; this one generates through the engine.  A tokenizer
is no part of the engine: prompts are token ids (``--prompt-ids 1,2,3`` or a
line of numbers), and text only if the model folder holds a ``tokenizer.json``
and the ``tokenizers`` package is installed.

    python -m mini_llm_b200.cli --model DIR --prompt-ids 464,3290,318 --temperature 0
    python -m mini_llm_b200.cli --random config.json --weights-seed 0 --prompt-ids 1,2,3

The second form needs no weights file: it writes a model folder with seeded random weights
for the given ``config.json`` into a temporary folder first.
"""

from __future__ import annotations

import argparse
import os
import sys


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(prog="mini_llm_b200", description="Complete prompts with the local model")
    parser.add_argument("--model", default="models/gpt2", help="Model directory")
    parser.add_argument("--max-new-tokens", type=int, default=64)
    parser.add_argument("--temperature", type=float, default=0.8)
    parser.add_argument("--top-p", type=float, default=0.95)
    parser.add_argument("--device", default="auto", choices=("auto", "cpu", "cuda"), help="Inference device")
    parser.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    parser.add_argument("--seed", type=int, default=0, help="seed of the sampler")
    parser.add_argument("--prompt-ids", action="append", default=[],
                        help="a prompt as comma-separated token ids (may be given more than once)")
    parser.add_argument("--prompt", action="append", default=[], help="a prompt as text (needs a tokenizer.json)")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-tokens-per-step", type=int, default=2048)
    parser.add_argument("--plain-kernels", action="store_true")
    parser.add_argument("--random", metavar="CONFIG.json",
                        help="instead of --model: write a model folder with random weights for this config.json "
                             "into a temporary folder and complete with it")
    parser.add_argument("--weights-seed", type=int, default=0, help="seed of --random's weights")
    parser.add_argument("--recipe", default="gpt2", choices=("gpt2", "varied"), help="how --random fills the tensors")
    return parser.parse_args(argv)


def random_model_folder(args) -> str:
    """A temporary model folder (config.json, model.safetensors) for ``--random``."""
    import atexit
    import json
    import shutil
    import tempfile
    from .config import config_from_dict
    from .weights import write_random_model
    with open(args.random) as handle:
        raw = json.load(handle)
    folder = tempfile.mkdtemp(prefix="mini_llm_b200-random-")
    atexit.register(shutil.rmtree, folder, ignore_errors=True)
    write_random_model(config_from_dict(raw), args.weights_seed, folder, recipe=args.recipe)
    return folder


def choose_device(requested: str) -> str:
    import torch
    if requested == "cpu":
        raise SystemExit("this engine has no CPU path: run with --device cuda on a CUDA device")
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device is available and this engine has no CPU path")
    return "cuda:0"


def load_tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def parse_ids(text: str) -> list:
    return [int(part) for part in text.replace(",", " ").split()]


def trim_prompt(ids: list, max_input_tokens: int) -> list:
    return ids if len(ids) <= max_input_tokens else ids[-max_input_tokens:]


def complete(llm, tokenizer, ids: list, args) -> tuple:
    limit = llm.engine.max_positions - args.max_new_tokens
    if limit < 1:
        raise SystemExit(f"--max-new-tokens {args.max_new_tokens} leaves no room for a prompt in "
                         f"{llm.engine.max_positions} positions")
    ids = trim_prompt(ids, limit)
    (tokens,) = llm.generate([ids], args.max_new_tokens, args.temperature, args.top_p, args.seed, llm.eos_token_id)
    text = tokenizer.decode(tokens) if tokenizer is not None else None
    return tokens, text


def main(argv=None) -> int:
    args = parse_args(argv)
    device = choose_device(args.device)
    from .generate import LLM
    if args.random:
        args.model = random_model_folder(args)
    llm = LLM(args.model, dtype=args.dtype, device=device, page_size=args.page_size,
              max_tokens_per_step=args.max_tokens_per_step, plain_kernels=args.plain_kernels)
    tokenizer = load_tokenizer(args.model)
    prompts = [parse_ids(p) for p in args.prompt_ids]
    for text in args.prompt:
        if tokenizer is None:
            raise SystemExit("--prompt needs a tokenizer.json in the model folder; give --prompt-ids instead")
        prompts.append(tokenizer.encode(text).ids)
    if prompts:
        for ids in prompts:
            tokens, text = complete(llm, tokenizer, ids, args)
            print(text if text is not None else " ".join(str(t) for t in tokens))
        return 0

    history = []
    print("Type a prompt" + (" (text, or token ids)" if tokenizer else " as token ids") +
          ". Commands: /clear /history /exit", file=sys.stderr)
    while True:
        try:
            line = input("> ").strip()
        except EOFError:
            break
        if not line:
            continue
        if line in ("/exit", "/quit"):
            break
        if line == "/clear":
            history.clear()
            continue
        if line == "/history":
            for prompt, completion in history:
                print(f"{prompt} -> {completion}")
            continue
        try:
            ids = parse_ids(line)
        except ValueError:
            if tokenizer is None:
                print("no tokenizer.json in the model folder: type token ids", file=sys.stderr)
                continue
            ids = tokenizer.encode(line).ids
        tokens, text = complete(llm, tokenizer, ids, args)
        shown = text if text is not None else " ".join(str(t) for t in tokens)
        print(shown)
        history.append((line, shown))
    return 0


if __name__ == "__main__":
    sys.exit(main())

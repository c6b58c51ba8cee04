"""Command line: ``tesseract --model-path DIR`` generates from token-id prompts.

The reference's binary takes ``--model-path``, ``--device``, ``--max-queue``,
``--max-running``, ``--max-batch-tokens``, ``--prefill-chunk-tokens``,
``--max-sequence-length`` and ``--kv-capacity-tokens``, each with a ``TESSERACT_*``
environment fallback (src/config.rs:139-186), and then serves HTTP.  Serving is not part
of this package; with the same options this command generates instead, taking what the
reference's request body carries (``max_tokens``, ``temperature``, ``top_p``, ``seed``,
src/api/openai.rs:70-96) as flags.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import sys
import tempfile
import time


def _env(name: str, default):
    value = os.environ.get("TESSERACT_" + name)
    return type(default)(value) if value is not None else default


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="tesseract", description="Generate tokens with a model folder (config.json, model.safetensors) on one B200.")
    p.add_argument("--model-path", default=os.environ.get("TESSERACT_MODEL_PATH"),
                   help="folder with config.json and model.safetensors [TESSERACT_MODEL_PATH]")
    p.add_argument("--device", type=int, default=_env("DEVICE", 0))
    p.add_argument("--max-queue", type=int, default=_env("MAX_QUEUE", 256))
    p.add_argument("--max-running", type=int, default=_env("MAX_RUNNING", 32))
    p.add_argument("--max-batch-tokens", type=int, default=_env("MAX_BATCH_TOKENS", 4096))
    p.add_argument("--prefill-chunk-tokens", type=int, default=_env("PREFILL_CHUNK_TOKENS", 512))
    p.add_argument("--max-sequence-length", type=int, default=_env("MAX_SEQUENCE_LENGTH", 131072))
    p.add_argument("--kv-capacity-tokens", type=int, default=_env("KV_CAPACITY_TOKENS", 32768))
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--random-weights", type=int, metavar="SEED", default=None,
                   help="write seeded random weights for --config into a temporary model folder and use it")
    p.add_argument("--config", help="config.json to use with --random-weights")
    p.add_argument("--prompt", action="append", default=[], help="text prompt (needs tokenizer.json); repeatable")
    p.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeatable")
    p.add_argument("--prompt-file", action="append", default=[], metavar="FILE",
                   help="one prompt per line: token ids separated by commas or blanks (a line that is not all "
                        "numbers is a text prompt and needs tokenizer.json); repeatable")
    p.add_argument("--random-prompt", type=int, action="append", default=[], metavar="LEN",
                   help="a prompt of LEN random token ids; repeatable")
    p.add_argument("--max-tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--no-cuda-graphs", action="store_true")
    p.add_argument("--check-weights", action="store_true",
                   help="after loading, read the final norm's weight back from the device and compare it with the "
                        "checkpoint bit by bit (the reference's checkpoint report, src/cuda/dense_decoder.rs:1429-1463)")
    p.add_argument("--json", action="store_true", help="one JSON object per request on standard output")
    p.add_argument("--plugin", action="append", default=[], metavar="MODULE",
                   help="import MODULE first (it registers parts or an architecture) [TESSERACT_PLUGINS]; repeatable")
    p.add_argument("--print-plan", action="store_true",
                   help="print which kernel every operation of this model takes at each row count, then exit")
    return p


def read_prompt_file(path: str):
    """One prompt per non-empty line: a list of token ids, or the line itself as text."""
    prompts = []
    with open(path, encoding="utf-8") as handle:
        for line in handle:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            fields = line.replace(",", " ").split()
            if all(f.lstrip("-").isdigit() for f in fields):
                prompts.append([int(f) for f in fields])
            else:
                prompts.append(line)
    return prompts


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from . import LLM, SamplingParams
    from .config import load_plugins

    load_plugins(args.plugin)

    model_path = args.model_path
    scratch = None
    if args.random_weights is not None:
        if not args.config:
            print("--random-weights needs --config", file=sys.stderr)
            return 2
        from .weights.random_init import write_random_model

        with open(args.config) as handle:
            config = json.load(handle)
        scratch = tempfile.TemporaryDirectory(prefix="tesseract_random_")
        model_path = write_random_model(scratch.name, config, args.random_weights)
    if not model_path:
        print("--model-path (or TESSERACT_MODEL_PATH) is required", file=sys.stderr)
        return 2
    llm = LLM(model_path, dtype=args.dtype, device=args.device, max_queue=args.max_queue,
              max_running=args.max_running, max_batch_tokens=args.max_batch_tokens,
              prefill_chunk_tokens=args.prefill_chunk_tokens, max_sequence_length=args.max_sequence_length,
              kv_capacity_tokens=args.kv_capacity_tokens, page_size=args.page_size,
              cuda_graphs=not args.no_cuda_graphs)
    if args.print_plan:
        from . import plan

        print(plan.describe(llm.model, context=min(args.max_sequence_length, llm.model.spec.max_positions),
                            page_size=args.page_size))
        return 0
    if args.check_weights:
        from .engine.loading import check_upload

        print(f"weights checked: {check_upload(llm.model, model_path)} matches the checkpoint", file=sys.stderr)
    vocab = llm.model.spec.vocab_size
    prompts = list(args.prompt)
    prompts += [[int(t) for t in ids.split(",") if t.strip()] for ids in args.prompt_ids]
    for path in args.prompt_file:
        prompts += read_prompt_file(path)
    rng = random.Random(args.seed or 0)
    prompts += [[rng.randrange(vocab) for _ in range(n)] for n in args.random_prompt]
    if not prompts:
        print("no prompt given (--prompt, --prompt-ids, --prompt-file or --random-prompt)", file=sys.stderr)
        return 2
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                            seed=args.seed, ignore_eos=args.ignore_eos)
    started = time.time()
    outputs = llm.generate(prompts, params)
    elapsed = time.time() - started
    for out in outputs:
        if args.json:
            print(json.dumps({"request": out.request_id, "token_ids": out.token_ids, "text": out.text,
                              "finish_reason": out.finish_reason, "usage": out.usage}))
        else:
            print(f"[{out.request_id}] {out.finish_reason}: " + (out.text if out.text is not None
                                                                else " ".join(map(str, out.token_ids))))
    total = sum(len(o.token_ids) for o in outputs)
    print(f"{total} tokens in {elapsed:.3f} s ({total / max(elapsed, 1e-9):.1f} tok/s)", file=sys.stderr)
    if scratch is not None:
        scratch.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Command line in the reference's manner (src/kipp_cli.c): prompts are
evaluated, then tokens are sampled and fed back one at a time, all of it by the
library's scheduler (the loop every front end shares), so several prompts run
beside one another.

Options the reference has keep their names and meanings (usage text
src/kipp_cli.c:571-610): --model, --decode, --temperature, --top-p, --top-k,
--min-p, --seed, --top, --ctx.  The prompt is token ids (there is no
tokenizer here): --prompt-ids (repeat it for several prompts), --prompt-file or
--random-prompt.  --backend
and --kv-quant have one value each here (cuda, the compute dtype's cache), so
--dtype stands in their place.  Output: ``generated\\t<ids>`` on stdout, the
final top-N logits as ``rank\\tid\\tlogit``, and on stderr the line
``KIPP_METRIC backend=... prefill_tokens=... prefill_seconds=...
decode_tokens=... decode_seconds=...`` (src/kipp_cli.c:1213-1217).
"""
from __future__ import annotations

import argparse
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="kipp", description="Qwen3 dense inference on one B200")
    ap.add_argument("--model", help="folder with config.json and *.safetensors")
    ap.add_argument("--random", metavar="PRESET|CONFIG.json",
                    help="instead of --model: a preset name (tiny-a, tiny-b, qwen3-4b, qwen3-8b, qwen3-32b) or a "
                         "config.json, filled with random weights")
    ap.add_argument("--weights-seed", type=int, default=None,
                    help="seed of the random weights (default: the preset's, else 0)")
    prompt = ap.add_mutually_exclusive_group(required=True)
    prompt.add_argument("--prompt-ids", action="append",
                        help="comma-separated token ids; give it again for another prompt (they run together)")
    prompt.add_argument("--prompt-file", help="file of little-endian uint32 token ids")
    prompt.add_argument("--random-prompt", type=int, metavar="LEN", help="LEN seeded random token ids")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="compute precision (default bfloat16; float32 = true 32-bit path)")
    ap.add_argument("--decode", type=int, default=0, help="greedy/sampled tokens to generate")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy argmax (default)")
    ap.add_argument("--top-p", type=float, default=1.0, help="nucleus mass, 0 < F <= 1 (default 1)")
    ap.add_argument("--top-k", type=int, default=0, help="keep N highest logits (0 = off)")
    ap.add_argument("--min-p", type=float, default=0.0, help="min prob vs top, 0 <= F <= 1 (0 = off)")
    ap.add_argument("--seed", type=int, default=1, help="nonzero sampling seed (default 1)")
    ap.add_argument("--top", type=int, default=10, help="final top-N logits to print (default 10)")
    ap.add_argument("--ctx", "--max-context", dest="ctx", type=int, default=None,
                    help="session capacity in tokens (default prompt + decode)")
    ap.add_argument("--kv-block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--kv-blocks", type=int, default=None,
                    help="pages of the cache pool (default: what the capacity needs)")
    ap.add_argument("--chunk", type=int, default=2048, help="largest prompt portion of one step")
    ap.add_argument("--max-batch-tokens", type=int, default=None,
                    help="tokens one step may hold (default: --chunk); sizes the activation buffers")
    ap.add_argument("--stop-token", type=int, action="append", default=None,
                    help="token id that ends decoding (default: the config's eos_token_id)")
    ap.add_argument("--policy", default="reserve", choices=["reserve", "preempt"],
                    help="when pages run out: admit only what can never run out (reserve, default), or admit "
                         "early and put the youngest request back (preempt)")
    ap.add_argument("--device", default="cuda:0")
    return ap


def _prompts(args, vocab: int) -> list:
    if args.prompt_ids is not None:
        return [[int(t) for t in ids.replace(" ", "").split(",") if t] for ids in args.prompt_ids]
    if args.prompt_file is not None:
        import numpy as np
        return [np.fromfile(args.prompt_file, dtype="<u4").astype("int64").tolist()]
    import torch
    g = torch.Generator().manual_seed(args.seed)
    return [torch.randint(0, vocab, (args.random_prompt,), generator=g).tolist()]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if (args.model is None) == (args.random is None):
        print("kipp: give exactly one of --model and --random", file=sys.stderr)
        return 2
    if args.decode < 0 or args.decode > (1 << 20):
        print("kipp: --decode must be between 0 and 2^20", file=sys.stderr)
        return 2
    if args.temperature > 0 and args.seed == 0:
        print("kipp: --seed must be nonzero", file=sys.stderr)
        return 2
    import numpy as np
    from .config.registry import config_from_dict, load_config
    from .engine.llm import LLM
    from .engine.scheduler import Request
    from .sampling.params import SamplingParams

    init = {}
    if args.model is not None:
        config = load_config(args.model)
    else:
        import json
        from .config.presets import load_preset, preset_names
        if args.random in preset_names():
            cfg_dict, init = load_preset(args.random)
            config = config_from_dict(cfg_dict)
        else:
            try:
                with open(args.random) as f:
                    config = config_from_dict(json.load(f))
            except FileNotFoundError:
                print(f"kipp: --random {args.random}: neither a preset ({', '.join(preset_names())}) nor a file",
                      file=sys.stderr)
                return 2
        if args.weights_seed is None:
            args.weights_seed = int(init.get("seed", 0))
    prompts = _prompts(args, config.vocab_size)
    if not prompts or any(not p for p in prompts):
        print("kipp: the prompt is empty", file=sys.stderr)
        return 2
    # one more token than asked for is sampled (and dropped) when the final logits are wanted:
    # they are the logits the token after the last generated one is sampled from
    extra = 1 if args.top > 0 and len(prompts) == 1 and args.decode > 0 else 0
    longest = max(len(p) for p in prompts)
    capacity = args.ctx or (longest + args.decode + extra)
    if longest + args.decode > capacity:
        print(f"kipp: prompt ({longest}) + decode ({args.decode}) exceeds --ctx {capacity}", file=sys.stderr)
        return 2
    if longest + args.decode + extra > capacity:
        extra = 0
    if args.max_batch_tokens is not None and args.max_batch_tokens < 1:
        print("kipp: --max-batch-tokens must be positive", file=sys.stderr)
        return 2
    if args.max_batch_tokens is not None:
        args.chunk = min(args.chunk, args.max_batch_tokens)
    page = args.kv_block_size
    cache_tokens = sum(-(-(len(p) + args.decode + extra) // page) * page for p in prompts)
    if args.kv_blocks is not None:
        cache_tokens = args.kv_blocks * page
        if cache_tokens < -(-capacity // page) * page and args.policy == "reserve":
            print(f"kipp: --kv-blocks {args.kv_blocks} x {page} tokens cannot hold {capacity}", file=sys.stderr)
            return 2
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                            min_p=args.min_p, seed=args.seed or 1)
    try:
        params.validate()
    except ValueError as e:
        print(f"kipp: {e}", file=sys.stderr)
        return 2
    llm = LLM(args.model if args.model is not None else config, dtype=args.dtype, device=args.device,
              kv_block_size=page, kv_tokens=cache_tokens, ctx=capacity, max_requests=max(len(prompts), 1),
              max_batch_tokens=max(args.max_batch_tokens or args.chunk, 1), chunk=args.chunk, policy=args.policy,
              seed=args.weights_seed or 0, stop_token_ids=tuple(args.stop_token or ()),
              **({"sigma": init.get("sigma"), "norm_jitter": init.get("norm_jitter", 0.1)}
                 if args.model is None else {}))
    total = sum(len(p) for p in prompts)
    print(f"kipp: evaluating {total} token{'' if total == 1 else 's'} of {config.architecture} on cuda "
          f"({args.dtype})", file=sys.stderr)
    sched = llm.new_scheduler()
    requests = []
    for i, prompt in enumerate(prompts):
        sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                            seed=(params.seed + i) or 1)
        requests.append(Request(id=i, prompt=prompt, max_new_tokens=args.decode + extra, sampling=sp,
                                stop_token_ids=llm.stop_token_ids))
        sched.add(requests[-1])
    llm.run(sched, record_steps=True)
    prefill_seconds = sum(s["seconds"] for s in llm.step_log if s["prefill"])
    decode_seconds = sum(s["seconds"] for s in llm.step_log if not s["prefill"])
    generated = 0
    for r in requests:
        out = r.output[:args.decode]
        generated += len(out)
        if args.decode:
            print("generated\t" + " ".join(str(t) for t in out))
    if args.top > 0 and len(prompts) == 1:
        logits = llm.engine.last_logits()
        if logits is not None and logits.shape[0] == 1:
            order = np.argsort(-logits[0], kind="stable")[:min(args.top, logits.shape[1])]
            for rank, i in enumerate(order.tolist(), 1):
                print(f"{rank}\t{i}\t{float(logits[0, i]):.9g}")
    print(f"KIPP_METRIC backend=cuda prefill_tokens={total} prefill_seconds={prefill_seconds:.9f} "
          f"decode_tokens={generated} decode_seconds={decode_seconds:.9f}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())

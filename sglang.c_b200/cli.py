"""Command line in the manner of the reference's `sglc` one-shot path
(apps/sglc.c:264-312,486-514): same option names and defaults where it has
them.  There is no tokenizer here, so the prompt is given as token ids."""
import argparse
import atexit
import json
import os
import shutil
import sys
import tempfile
import time


def parse_ids(text):
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit("the prompt must be token ids separated by commas or spaces "
                         "(this engine has no tokenizer)")


def build_parser():
    ap = argparse.ArgumentParser(
        prog="sglc", description="generate from a model folder (config.json, model.safetensors) on one GPU")
    ap.add_argument("--model", help="model folder")
    ap.add_argument("--prompt", help="prompt as token ids, e.g. \"464, 3616, 286\"")
    ap.add_argument("--prompt-ids", help="same as --prompt")
    ap.add_argument("--prompt-file", help="file with token ids")
    ap.add_argument("--max-new", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--device", default="cuda", help="cuda or cuda:N (this engine runs on the GPU only)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--pages", type=int, default=None, help="pages in the cache pool")
    ap.add_argument("--chunk", type=int, default=512, help="largest prompt portion per step")
    ap.add_argument("--token-budget", type=int, default=2048, help="most tokens per step")
    ap.add_argument("--native", action="store_true",
                    help="the engine behind the C interface (loader, scheduler and step in C++); same ids")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="write a random model folder from --config and use it")
    ap.add_argument("--config", help="config.json for --random-weights")
    ap.add_argument("--init", default="standard", choices=["standard", "varied"])
    ap.add_argument("--save-model", help="where --random-weights writes the folder (default: temporary)")
    return ap


def main(argv=None):
    from . import log
    args = build_parser().parse_args(argv)
    log.set_level(log.DEBUG if args.verbose else log.INFO)
    if args.device not in ("cuda", "auto") and not args.device.startswith("cuda:"):
        raise SystemExit(f"unknown --device '{args.device}' (this engine runs on cuda only)")
    device = "cuda:0" if args.device in ("cuda", "auto") else args.device
    model_dir = args.model
    if args.random_weights is not None:
        if not args.config:
            raise SystemExit("--random-weights needs --config <config.json>")
        from .config import resolve_architecture
        from .weights import write_random_model
        with open(args.config) as f:
            d = json.load(f)
        arch = resolve_architecture(d)
        cfg = arch.config_class.from_dict(d)
        model_dir = args.save_model
        if not model_dir:
            model_dir = tempfile.mkdtemp(prefix="sglc_random_")
            atexit.register(shutil.rmtree, model_dir, True)
        write_random_model(model_dir, arch, cfg, args.random_weights, scheme=args.init)
        log.info(f"wrote random weights (seed {args.random_weights}) to {model_dir}")
    if not model_dir:
        build_parser().print_usage(sys.stderr)
        return 1
    text = args.prompt or args.prompt_ids
    if args.prompt_file:
        with open(args.prompt_file) as f:
            text = f.read()
    if not text:
        raise SystemExit("give the prompt's token ids with --prompt, --prompt-ids or --prompt-file")
    prompt = parse_ids(text)

    from .engine import generate, sched_new
    from .sampling import SamplingParams
    t0 = time.time()
    need = len(prompt) + args.max_new + 1
    s = sched_new(model_dir, seed=args.seed, dtype=args.dtype, device=device, page_size=args.page_size,
                  n_pages=args.pages, max_tokens=None if args.pages else max(need, 64) + args.page_size,
                  max_requests=4, max_step_tokens=args.token_budget, prefill_chunk=args.chunk,
                  token_budget=args.token_budget, native=args.native)
    st = s.get_stats()
    mb = (st.weight_bytes if args.native else s.engine.model.weight_bytes) / 1e6
    log.debug(f"model loaded in {time.time() - t0:.2f}s ({mb:.1f} MB of weights, {st.pool_pages} pages of "
              f"{args.page_size})")
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                        min_p=args.min_p, repetition_penalty=args.repetition_penalty,
                        ignore_eos=args.ignore_eos, seed=args.seed)
    t1 = time.time()
    out = generate(s, prompt, sp, args.max_new)
    dt = time.time() - t1
    print(" ".join(str(t) for t in prompt + out))
    n = len(out)
    log.info(f"generated {n} tokens in {dt:.2f}s ({n / dt if dt > 0 else 0:.1f} tok/s, "
             f"{dt * 1000 / max(n, 1):.0f} ms/tok)")
    st = s.get_stats()
    log.debug("stats: " + ", ".join(f"{k}={getattr(st, k)}" for k in ("n_steps", "prefill_tokens", "decode_tokens",
                                                                       "n_finished", "n_preempt", "pool_free")))
    return 0


if __name__ == "__main__":
    sys.exit(main())

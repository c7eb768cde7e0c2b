"""forge-cli: one-shot generation from the command line, with the reference's option names
(src/cli/cli_args.cpp:11-82, 84-216): -m/--model, -p/--prompt, -n/--n-predict, --temp, --top-k, --top-p,
--repeat-penalty, --seed, --no-stream, --info, -v, -h; the same defaults (temperature 0.7, top-k 40,
top-p 0.9, repeat penalty 1.1, n-predict 256, -1 meaning 256; temperature 0 means greedy).

The reference tokenizes -p with the tokenizer stored in its GGUF file; a safetensors folder has none, so
here -p takes token ids ("1,15,27" or "1 15 27"), as does --prompt-file.  Options that select what this
engine does not have (-ngl, -t, -b, --kv-cache-dtype, --mmproj, --image, -i, --system-prompt) are refused
with a message.  Ours only: --dtype, --random-weights CONFIG.json, --page-size, --kv-pages, --max-tokens-per-step.
"""
import argparse
import json
import sys
import tempfile
import time


def parse_ids(text):
    parts = text.replace(",", " ").split()
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit("Error: this build has no tokenizer; give -p as token ids, e.g. -p \"1 15 27\"")


def build_parser():
    ap = argparse.ArgumentParser(prog="forge-cli", description="Forge CLI (B200 engine) - LLaMA inference")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("-p", "--prompt", help="prompt as token ids")
    ap.add_argument("--prompt-file", help="file with prompt token ids")
    ap.add_argument("-n", "--n-predict", type=int, default=-1, help="tokens to predict (default 256, -1 = 256)")
    ap.add_argument("--temp", "--temperature", dest="temp", type=float, default=0.7, help="0 = greedy")
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--repeat-penalty", type=float, default=1.1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-stream", action="store_true")
    ap.add_argument("--info", action="store_true", help="show model info and exit")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--random-weights", metavar="CONFIG.json", help="make a random model from this config")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page (8, 16, 32 or 64)")
    ap.add_argument("--kv-pages", type=int, default=None, help="pages of the cache (default: sized from the free device memory)")
    ap.add_argument("--max-tokens-per-step", type=int, default=2048, help="longer prompts are run in portions of this many tokens")
    for flag in ("-ngl", "--n-gpu-layers", "-t", "--threads", "-b", "--batch-size", "--kv-cache-dtype", "--mmproj",
                 "--image", "--system-prompt"):
        ap.add_argument(flag, dest="unsupported_" + flag.strip("-").replace("-", "_"), default=None, metavar="X",
                        help="(the reference's option; not part of this engine, refused)")
    ap.add_argument("-i", "--interactive", action="store_true")
    ap.add_argument("--bench", action="store_true", help="prefill of 32/128/512 tokens and 128 decode steps, timed")
    return ap


def run_benchmark(model, verbose=False):
    """The reference's built-in benchmark (src/cli/forge_cli.cpp:242-321): prefill of 32, 128 and 512 dummy tokens
    (three runs each from an empty cache, mean), then 128 single-token decode steps; wall-clock around device work."""
    import torch
    cfg = model.config
    print("\n  Forge - Benchmark\n")
    print(f"  Model: {cfg.architecture} ({cfg.num_hidden_layers} layers, {cfg.hidden_size}d)")
    print("  Warming up...")
    ctx = model.create_context()
    ctx.forward([0] * 8, 0)
    ctx.reset_kv()
    print("  Warmup done\n")
    limit = model.runner.plan.max_positions
    for ps in (32, 128, 512):
        if ps + 130 > limit or ps > model.runner.num_pages * model.runner.page_size:
            continue
        runner = model.runner
        from .engine import StepEntry
        runner.admit("bench"); runner.step([StepEntry("bench", [0] * ps, [ps - 1])]); runner.release("bench")   # kernels for this size
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(3):
            runner.admit("bench")
            runner.step([StepEntry("bench", [0] * ps, [ps - 1])])
            runner.release("bench")
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / 3
        print(f"  Prefill {ps:4d} tokens: {ms:7.2f} ms  ({ps / ms * 1e3:8.1f} tok/s)")
    steps = 128
    out = model.generate([0], max_new_tokens=8, do_sample=False)                     # captures the decode graph
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = model.generate([0], max_new_tokens=steps + 1, do_sample=False)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3
    print(f"  Decode  {out['num_generated_tokens'] - 1:4d} tokens: {ms:7.2f} ms  ({(out['num_generated_tokens'] - 1) / ms * 1e3:8.1f} tok/s)")
    print("\n  Benchmark complete")


def main(argv=None):
    a = build_parser().parse_args(argv)
    for k, v in vars(a).items():
        if k.startswith("unsupported_") and v is not None:
            raise SystemExit(f"Error: option --{k[12:].replace('_', '-')} selects a feature this engine does not have")
    if a.interactive:
        raise SystemExit("Error: interactive chat is not part of this engine; give a prompt with -p")
    from . import Logger, Model, load_config, write_random_model
    if a.verbose:
        Logger.set_level(3)
    from .config import config_from_dict
    model_dir = a.model
    if a.random_weights:
        with open(a.random_weights) as f:
            cfg = config_from_dict(json.load(f))
        model_dir = tempfile.mkdtemp(prefix="forge_random_")
        write_random_model(cfg, model_dir, seed=a.seed)
    if not model_dir:
        raise SystemExit("Error: -m/--model is required")
    if a.info:
        cfg = load_config(model_dir)
        for k, v in cfg.to_dict().items():
            print(f"  {k}: {v}")
        return 0
    if a.kv_pages is not None and a.kv_pages < 1:
        raise SystemExit("Error: --kv-pages must be at least 1")
    cache_tokens = a.kv_pages * a.page_size if a.kv_pages else None
    if a.bench:
        model = Model(model_dir, dtype=a.dtype, block_size=a.page_size, max_num_seqs=1, max_tokens_per_step=a.max_tokens_per_step,
                      cache_tokens=cache_tokens)
        run_benchmark(model, a.verbose)
        return 0
    if a.prompt is None and a.prompt_file is None:
        raise SystemExit("Error: no prompt (-p); interactive mode is not part of this engine")
    prompt = parse_ids(a.prompt if a.prompt is not None else open(a.prompt_file).read())
    n_predict = 256 if a.n_predict == -1 else a.n_predict
    model = Model(model_dir, dtype=a.dtype, block_size=a.page_size, max_num_seqs=1,
                  max_tokens_per_step=a.max_tokens_per_step, cache_tokens=cache_tokens)
    times = []
    if a.verbose:                      # per-kernel timing table at the end (decode steps are launched one by one meanwhile)
        from . import kernels
        kernels.profiler_enable()

    def on_token(tok, step):
        times.append(time.perf_counter())
        if not a.no_stream:
            print(tok, end=" ", flush=True)

    t0 = time.perf_counter()
    out = model.generate(prompt, max_new_tokens=n_predict, temperature=a.temp, top_k=a.top_k, top_p=a.top_p,
                         repeat_penalty=a.repeat_penalty, do_sample=a.temp != 0.0, seed=a.seed,
                         eos_token_id=model.config.eos_token_id if model.config.eos_token_id is not None else -1,
                         callback=on_token)
    t1 = time.perf_counter()
    if a.no_stream:
        print(" ".join(map(str, out["token_ids"])), end="")
    prompt_ms = (times[0] - t0) * 1e3 if times else 0.0
    total_ms = (t1 - t0) * 1e3
    print(f"\n\n  [{len(prompt)} prompt, {prompt_ms:.1f} ms, {len(prompt) / max(prompt_ms, 1e-9) * 1e3:.1f} tok/s | "
          f"{out['num_generated_tokens']} generated, {total_ms:.1f} ms, "
          f"{out['num_generated_tokens'] / max(total_ms, 1e-9) * 1e3:.1f} tok/s]")
    if a.verbose:
        print(f"  finish_reason: {out['finish_reason']}", file=sys.stderr)
        kernels.profiler_print(sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Command line, in the manner of the reference's ``fastgguf <command> <model> [ctx] [options]``
(fastgguf.c:10-17, :7067-7101), for model folders and token ids instead of GGUF files and text:

    python -m fastgguf_b200 generate MODEL_DIR [ctx] --prompt 1,2,3 [--prompt ...] [options]
    python -m fastgguf_b200 inspect  MODEL_DIR           config, sizes, tensor table
    python -m fastgguf_b200 dump     MODEL_DIR           every key of config.json
    python -m fastgguf_b200 random   CONFIG.json OUT_DIR [--seed N] [--dtype bfloat16|float32]
    python -m fastgguf_b200 selftest                     every kernel against a plain computation

Options of ``generate`` are the reference's chat options with the same names, meanings and
defaults (fastgguf.c:6957-6982): positional ``ctx`` (2048, at least 64); ``--temp 1.0`` (0 =
greedy); ``--top-k 64`` (0 = off); ``--top-p 0.95``; ``--repeat-penalty 1.0`` (1 = off);
``--repeat-last-n 64``; ``--max-tokens 512`` (0 = until stop); ``--seed N``.  An unknown option
or a missing value prints a message and exits 1; a model that cannot be loaded exits 2
(fastgguf.c:5224-5228).
"""
from __future__ import annotations

import json
import sys
import time
from typing import List

USAGE = __doc__

CHAT_OPTIONS_HELP = (
    "generate options: --temp 1.0 (0 = greedy)  --top-k 64 (0 = off)  --top-p 0.95\n"
    "                  --repeat-penalty 1.0 (1 = off)  --repeat-last-n 64\n"
    "                  --max-tokens 512 (0 = until stop)  --seed N\n"
    "                  --prompt ID,ID,...  (repeat for a batch)  --prompts-file FILE (one prompt a line)\n"
    "                  --stop-id ID (repeat; added to the model's own stop tokens)\n"
    "                  --dtype bfloat16|float32  --batch N  --ignore-eos  --json\n"
    "                  --stream  (print \"request token\" lines to the standard error as tokens are made)\n"
    "                  --profile (device time per kernel launcher; runs the kernels one after another)\n")


class UsageError(Exception):
    pass


def parse_generate_args(argv: List[str]) -> dict:
    """Positional [ctx], then --option value pairs (fastgguf.c:6957-6974)."""
    o = dict(ctx=2048, temp=1.0, top_k=64, top_p=0.95, repeat_penalty=1.0, repeat_last_n=64, max_tokens=512,
             seed=0, prompts=[], stop_ids=[], dtype="bfloat16", batch=None, ignore_eos=False, json=False, stream=False,
             profile=False)
    flags = {"--ignore-eos": "ignore_eos", "--json": "json", "--stream": "stream", "--profile": "profile"}
    valued = {"--temp": ("temp", float), "--top-k": ("top_k", int), "--top-p": ("top_p", float),
              "--repeat-penalty": ("repeat_penalty", float), "--repeat-last-n": ("repeat_last_n", int),
              "--max-tokens": ("max_tokens", int), "--seed": ("seed", int), "--dtype": ("dtype", str),
              "--batch": ("batch", int)}
    i = 0
    while i < len(argv):
        a = argv[i]
        if not a.startswith("-"):
            try:
                o["ctx"] = int(a)
            except ValueError:
                raise UsageError(f"unknown argument {a}") from None
            i += 1
            continue
        if a in flags:
            o[flags[a]] = True
            i += 1
            continue
        if i + 1 >= len(argv):
            raise UsageError(f"missing value for {a}")
        v = argv[i + 1]
        i += 2
        try:
            if a in valued:
                key, typ = valued[a]
                o[key] = typ(v)
            elif a == "--prompt":
                o["prompts"].append([int(t) for t in v.replace(",", " ").split()])
            elif a == "--stop-id":
                o["stop_ids"].append(int(v))
            elif a == "--prompts-file":
                with open(v) as f:
                    o["prompts"].extend([int(t) for t in line.replace(",", " ").split()] for line in f if line.strip())
            else:
                raise UsageError(f"unknown option {a}")
        except ValueError:
            raise UsageError(f"bad value for {a}: {v}") from None
    o["ctx"] = max(64, o["ctx"])
    return o


def cmd_generate(model_dir: str, argv: List[str]) -> int:
    o = parse_generate_args(argv)
    if not o["prompts"]:
        raise UsageError("generate needs at least one --prompt ID,ID,... (token ids) or --prompts-file FILE")
    from .capi import EngineError
    from .engine.api import Engine
    n = len(o["prompts"])
    batch = o["batch"] or min(n, 64)

    def say(*args, **kw):
        # with --json the standard output is one JSON document; the summary lines go to the standard error
        print(*args, file=sys.stderr if o["json"] else sys.stdout, **kw)

    try:
        engine = Engine.from_dir(model_dir, dtype=o["dtype"], max_tokens=batch * ((o["ctx"] + 63) // 64 * 64),
                                 max_batch=batch, max_seq_len=o["ctx"])
    except (EngineError, ValueError, OSError) as e:
        print(e)
        return 2
    info = engine.info()
    # the reference's load-time summary (fastgguf.c:4561-4565), with the cache's size
    say(f"[Config] {engine.config.architecture}: layers={info['layers']} embd={info['hidden_size']} "
        f"ctx={info['max_seq_len']} dtype={o['dtype']}")
    say(f"[Model] {info['tensors']} tensors, {info['weight_bytes'] / 2 ** 20:.1f} MiB, vocab={info['vocab_size']}")
    say(f"[cache] slots={info['slots']} pages={info['pages']} page={info['page_size']} "
        f"bytes/token={info['bytes_per_token']} bytes={info['cache_bytes']} ({info['cache_bytes'] / 2 ** 20:.1f} MiB)")
    if o["temp"] <= 0:
        say("[Sampler] greedy", end="")
    else:
        say(f"[Sampler] temp={o['temp']:.2f} top_k={o['top_k']} top_p={o['top_p']:.2f}", end="")
    say(f" repeat_penalty={o['repeat_penalty']:.2f} (last {o['repeat_last_n']}) max_tokens={o['max_tokens']} "
        f"seed={o['seed']}")
    if o["profile"]:
        engine.profile(True)
    t0 = time.time()
    try:
        out = engine.generate(o["prompts"], temp=o["temp"], top_k=o["top_k"], top_p=o["top_p"],
                              repeat_penalty=o["repeat_penalty"], repeat_last_n=o["repeat_last_n"],
                              max_tokens=o["max_tokens"], seed=o["seed"], ignore_eos=o["ignore_eos"], batch_size=batch,
                              stop_ids=(list(info["stop_token_ids"]) + o["stop_ids"]) if o["stop_ids"] else None,
                              on_token=(lambda r, t: print(r, t, file=sys.stderr, flush=True)) if o["stream"] else None)
    except (EngineError, ValueError) as e:
        print(e)
        return 1
    dt = time.time() - t0
    n_gen = sum(len(c.tokens) for c in out)
    if o["json"]:
        print(json.dumps([{"tokens": c.tokens, "finish_reason": c.finish_reason} for c in out]))
    else:
        for i, c in enumerate(out):
            print(f"[{i}] {' '.join(str(t) for t in c.tokens)}  ({c.finish_reason})")
    say(f"[gen: {n_gen} tok in {dt:.2f}s @ {n_gen / max(dt, 1e-9):.2f} tok/s, prompts included]")
    if o["profile"]:
        # device time per kernel launcher, kernels run one after another (no graphs, no overlap of dependent launches)
        rows = engine.profile_report()
        total = sum(r["ms"] for r in rows) or 1.0
        say(f"[profile] {sum(r['calls'] for r in rows)} launches, {total:.3f} ms on the device")
        for r in rows[:24]:
            say(f"[profile] {r['ms']:10.3f} ms {100 * r['ms'] / total:5.1f} %  {r['calls']:6d} x  {r['name']}")
    return 0


def cmd_inspect(model_dir: str, as_json: bool = False) -> int:
    """What ``fastgguf inspect`` prints for a GGUF file (fastgguf.c:5319-5360), for a model folder: the
    architecture, every configuration field (marked where the file did not give it) and derived size, memory
    per token and for the parameters, a dtype histogram and the tensors."""
    from .capi import EngineError
    from .registry import config_from_dir
    from .weights import folder_tensors
    try:
        cfg = config_from_dir(model_dir)
        tensors = folder_tensors(model_dir)
    except (EngineError, OSError) as e:
        print(e)
        return 2
    desc = cfg.describe()
    if as_json:
        print(json.dumps({"architecture": cfg.architecture, "config": desc, "tensors": tensors}))
        return 0
    defaulted = set(desc.get("defaulted", []))
    print(f"architecture: {cfg.architecture}")
    for k, v in desc.items():
        if k in ("architecture", "defaulted"):
            continue
        print(f"  {k} = {v}" + ("   (default)" if k in defaulted else ""))
    hist, nbytes = {}, {}
    sizes = {"float32": 4, "bfloat16": 2, "float16": 2, "int32": 4, "int64": 8}
    for t in tensors:
        n = 1
        for s in t["shape"]:
            n *= s
        hist[t["dtype"]] = hist.get(t["dtype"], 0) + 1
        nbytes[t["dtype"]] = nbytes.get(t["dtype"], 0) + n * sizes.get(t["dtype"], 0)
    print(f"tensors: {len(tensors)}  (" + ", ".join(f"{k}: {v} ({nbytes[k] / 2 ** 20:.1f} MiB)" for k, v in sorted(hist.items())) + ")")
    for t in tensors[:15]:
        print(f"  {t['name']:<48} {t['dtype']:<9} {t['shape']}")
    if len(tensors) > 15:
        print(f"  ... {len(tensors) - 15} more")
    return 0


def cmd_dump(model_dir: str) -> int:
    """Every key of config.json (the reference's ``dump`` prints every metadata key, fastgguf.c:5362-5375)."""
    from .config.base import ConfigError, read_config_json
    try:
        d = read_config_json(model_dir)
    except ConfigError as e:
        print(e)
        return 2
    for k, v in d.items():
        print(f"{k} = {json.dumps(v)}")
    return 0


def cmd_random(argv: List[str]) -> int:
    if len(argv) < 2:
        raise UsageError("random needs CONFIG.json and OUT_DIR")
    seed, dtype = 0, "bfloat16"
    i = 2
    while i < len(argv):
        if i + 1 >= len(argv):
            raise UsageError(f"missing value for {argv[i]}")
        if argv[i] == "--seed":
            seed = int(argv[i + 1])
        elif argv[i] == "--dtype":
            dtype = argv[i + 1]
        else:
            raise UsageError(f"unknown option {argv[i]}")
        i += 2
    from .capi import EngineError
    from .registry import config_from_dict
    from .weights import write_random_model
    try:
        with open(argv[0]) as f:
            cfg = config_from_dict(json.load(f))
        out = write_random_model(cfg, seed, argv[1], dtype)
    except (EngineError, ValueError, OSError) as e:
        print(e)
        return 2
    print(f"wrote {out}/config.json and {out}/model.safetensors (seed {seed}, {dtype})")
    return 0


def main(argv: List[str] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(USAGE)
        print(CHAT_OPTIONS_HELP)
        return 0 if argv else 1
    cmd, rest = argv[0], argv[1:]
    try:
        if cmd == "selftest":
            from .selftest import run_selftest
            return run_selftest(quick="--quick" in rest)
        if cmd == "random":
            return cmd_random(rest)
        if cmd in ("generate", "chat", "inspect", "dump"):
            if not rest:
                raise UsageError(f"{cmd} needs a model folder")
            if cmd == "inspect":
                return cmd_inspect(rest[0], "--json" in rest[1:])
            if cmd == "dump":
                return cmd_dump(rest[0])
            return cmd_generate(rest[0], rest[1:])
        raise UsageError(f"unknown command {cmd}")
    except UsageError as e:
        print(e)
        print(CHAT_OPTIONS_HELP)
        return 1


if __name__ == "__main__":
    sys.exit(main())

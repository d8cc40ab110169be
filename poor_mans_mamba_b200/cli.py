"""Command line in the manner of the reference's ``app`` (src/main.cpp:112-129):

    python -m poor_mans_mamba_b200 [model_dir] [max_seq] [CPU|GPU] [n_workers] [n_prompts] [max_new_tokens]

with the same positional meanings and defaults (max_seq 2048, n_workers 1, n_prompts 4,
max_new_tokens 16).  ``max_seq`` is what it is there: the longest context of one request; a
request that reaches it ends with what it has.  This engine runs on one GPU: ``CPU`` and
``n_workers`` other than 1 are refused.  The reference sizes one cache slot of max_seq tokens
per request; here the cache is a pool of pages, sized by default for n_prompts requests of
max_seq tokens: ``--max-tokens`` (or ``--num-pages``), ``--page-size``, ``--max-seqs`` and
``--max-seq-len`` set the pool's capacity in tokens, the page size, the number of live requests
and the per-request limit on their own.  The reference encodes fixed demo prompts with the model's tokenizer; here a
``tokenizer.json`` in the model folder is used the same way when the ``tokenizers``
package is importable, otherwise (or with --prompt-len / --prompt-ids) prompts are token
ids: the bos token repeated, as the reference's generate harness does
(benchmarks/generate_bench.cpp:109-111).  ``--random CONFIG.json`` first writes a
random-weights model folder for that configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from typing import List, Optional


def _tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="poor_mans_mamba_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model_dir", nargs="?", default="models/falcon-h1-0.5b-base")
    ap.add_argument("max_seq", nargs="?", type=int, default=2048)
    ap.add_argument("device", nargs="?", default="GPU", choices=["CPU", "GPU"])
    ap.add_argument("n_workers", nargs="?", type=int, default=1)
    ap.add_argument("n_prompts", nargs="?", type=int, default=4)
    ap.add_argument("max_new_tokens", nargs="?", type=int, default=16)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prompt-ids", action="append", help="comma-separated token ids (repeatable)")
    ap.add_argument("--prompt-len", type=int, default=0, help="bos-filled prompts of this length")
    ap.add_argument("--random", metavar="CONFIG_JSON", help="write a random-weights model for this config first")
    ap.add_argument("--max-batched-tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--max-tokens", type=int, default=None,
                    help="capacity of the key/value pool in tokens (default: max_seq x n_prompts)")
    ap.add_argument("--num-pages", type=int, default=None, help="the same capacity given in pages")
    ap.add_argument("--max-seqs", type=int, default=None, help="most requests alive at a time (default: n_prompts)")
    ap.add_argument("--max-seq-len", type=int, default=None,
                    help="longest context of one request (default: the positional max_seq)")
    args = ap.parse_args(argv)

    if args.device == "CPU":
        print("this engine has no CPU path; use GPU", file=sys.stderr)
        return 1
    if args.n_workers != 1:
        print("n_workers must be 1: this engine serves from one GPU", file=sys.stderr)
        return 1
    if args.n_prompts <= 0 or args.max_new_tokens <= 0 or args.max_seq <= 0:
        print("n_prompts, max_new_tokens and max_seq must be > 0", file=sys.stderr)
        return 1
    if args.max_tokens is not None and args.num_pages is not None:
        print("give --max-tokens or --num-pages, not both", file=sys.stderr)
        return 1
    for name in ("page_size", "max_tokens", "num_pages", "max_seqs", "max_seq_len", "max_batched_tokens"):
        if getattr(args, name) is not None and getattr(args, name) <= 0:
            print(f"--{name.replace('_', '-')} must be > 0", file=sys.stderr)
            return 1
    max_seq_len = args.max_seq_len if args.max_seq_len is not None else args.max_seq
    if args.num_pages is not None:
        max_tokens = args.num_pages * args.page_size
    elif args.max_tokens is not None:
        max_tokens = args.max_tokens
    else:
        max_tokens = -(-max_seq_len // args.page_size) * args.page_size * args.n_prompts

    from .entry import Engine
    from .weights import write_random_model

    model_dir = args.model_dir
    tmp = None
    if args.random:
        with open(args.random, "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
        tmp = tempfile.TemporaryDirectory()
        model_dir = write_random_model(cfg, args.seed, tmp.name)
    try:
        eng = Engine(model_dir, dtype=args.dtype, max_tokens=max_tokens, page_size=args.page_size,
                     max_seqs=args.max_seqs if args.max_seqs is not None else args.n_prompts,
                     max_batched_tokens=args.max_batched_tokens, max_seq_len=max_seq_len)
        tok = None if (args.prompt_ids or args.prompt_len) else _tokenizer(model_dir)
        prompts: List[List[int]] = []
        texts: List[Optional[str]] = []
        for i in range(args.n_prompts):
            if args.prompt_ids:
                prompts.append([int(x) for x in args.prompt_ids[i % len(args.prompt_ids)].split(",")])
                texts.append(None)
            elif tok is not None:
                text = f"Hi How are you? ({i})"
                prompts.append(tok.encode(text).ids)
                texts.append(text)
            else:
                n = args.prompt_len or 8
                prompts.append([eng.model.spec.bos_token_id] * n)
                texts.append(None)
        t0 = time.time()
        ids = []
        for p, text in zip(prompts, texts):
            from .engine.scheduler import SamplingParams
            rid = eng.submit(p, SamplingParams(max_new_tokens=args.max_new_tokens,
                                               eos_id=eng.model.spec.eos_token_id,
                                               temperature=args.temperature, seed=args.seed + len(ids)))
            ids.append(rid)
            shown = f'prompt="{text}"' if text is not None else f"prompt_ids={p[:16]}{'...' if len(p) > 16 else ''}"
            print(f"submitted req_id={rid} {shown}")
        while eng.has_work():
            eng.step()
        dt = time.time() - t0
        for rid in ids:
            r = eng.poll(rid)
            if tok is not None:
                print(f'req_id={rid} gen_tokens={len(r.tokens)} text="{tok.decode(r.tokens)}"')
            else:
                print(f"req_id={rid} gen_tokens={len(r.tokens)} status={r.status} tokens={r.tokens}")
        n_gen = sum(len(eng.poll(r).tokens) for r in ids)
        print(f"generated {n_gen} tokens in {dt:.3f}s", file=sys.stderr)
    finally:
        if tmp is not None:
            tmp.cleanup()
    return 0

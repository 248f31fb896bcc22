"""run_gemma2: generate from a model folder on one GPU.

Options are named as in wlejon/brolm's text tools
(tools/run_mistral_text.cpp:63-82): --max-new, --temp (<= 0: greedy, the
default), --top-k, --top-p, --seed, --no-bos.  A model comes from --model DIR
(config.json + safetensors) or from --random with the sizes of a config.json
given by --config.  Prompts are token ids (--ids or --ids-file, one request
per line) or text (--prompt TEXT, may be repeated) with the family's
tokenizer: --tok tokenizer.json, by default the tokenizer.json in the model
folder (brolm src/gemma_tokenizer.cpp; --chat wraps the text in Gemma's turn
markers as brolm's tools wrap theirs in the family's chat template).  With a
tokenizer the completions are printed as text as well.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
import time


def parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="run_gemma2", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="folder with config.json and *.safetensors")
    ap.add_argument("--random", action="store_true", help="random weights for the sizes in --config")
    ap.add_argument("--config", help="config.json for --random (default: gemma-2-2b sizes)")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--ids", action="append", help="prompt token ids, e.g. 2,651,6037 (may be repeated)")
    ap.add_argument("--ids-file", help="file with one prompt per line, ids separated by spaces or commas")
    ap.add_argument("--prompt", action="append", help="prompt text (needs a tokenizer; may be repeated)")
    ap.add_argument("--tok", help="tokenizer.json (default: the one in the --model folder)")
    ap.add_argument("--chat", action="store_true", help="wrap --prompt in Gemma's <start_of_turn> chat markers")
    ap.add_argument("--max-new", type=int, default=48, help="max new tokens (default 48)")
    ap.add_argument("--temp", type=float, default=0.0, help="sampling temperature, <=0 => greedy (default 0)")
    ap.add_argument("--top-k", type=int, default=0, help="top-k cutoff, 0 = off")
    ap.add_argument("--top-p", type=float, default=1.0, help="nucleus top-p, >=1 = off")
    ap.add_argument("--seed", type=int, default=0, help="RNG seed for sampling")
    ap.add_argument("--no-bos", action="store_true", help="do not prepend BOS to the prompts")
    ap.add_argument("--no-eos", action="store_true", help="do not stop at EOS")
    ap.add_argument("--stop-id", type=int, action="append", default=[], help="further stop token (may be repeated)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--batch", type=int, default=0, help="most requests run together (default: as the cache allows)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    if bool(args.model) == bool(args.random):
        print("error: pass exactly one of --model DIR and --random", file=sys.stderr)
        return 2
    tokenizer = None
    tok_path = args.tok or (os.path.join(args.model, "tokenizer.json") if args.model else None)
    if args.prompt or args.tok:
        if not tok_path or not os.path.exists(tok_path):
            print(f"error: tokenizer not found at {tok_path} (pass --tok tokenizer.json, or token ids with --ids)",
                  file=sys.stderr)
            return 2
        from .tokenizer import GemmaTokenizer, TokenizerError
        try:
            tokenizer = GemmaTokenizer.load(tok_path)
        except TokenizerError as e:
            print(f"error: {e}", file=sys.stderr)
            return 2
    prompts = [parse_ids(t) for t in (args.ids or [])]
    if args.ids_file:
        with open(args.ids_file) as fh:
            prompts += [parse_ids(line) for line in fh if line.strip()]
    for text in args.prompt or []:
        if args.chat:
            text = f"<start_of_turn>user\n{text}<end_of_turn>\n<start_of_turn>model\n"
        prompts.append(tokenizer.tokenize(text))            # <bos> is put in front below, unless --no-bos
    if not prompts:
        print("error: no prompt; pass --prompt, --ids or --ids-file", file=sys.stderr)
        return 2

    import brolm_b200 as bb
    try:
        t0 = time.time()
        if args.model:
            print(f"[load] model: {args.model}")
            model = bb.load_model(args.model, dtype=args.dtype, device=args.device)
        else:
            cfg = bb.load_config(args.config) if args.config else bb.Gemma2Config()
            print(f"[load] random weights, seed {args.weights_seed}")
            model = bb.Model(cfg, dtype=args.dtype, device=args.device).init_random(args.weights_seed, on_device=True)
        cfg = model.config
        print(f"[info] hidden={cfg.hidden_size} layers={cfg.num_hidden_layers} q={cfg.num_attention_heads} "
              f"kv={cfg.num_key_value_heads} vocab={cfg.vocab_size} dtype={args.dtype}")
        print(f"[info] weights loaded in {time.time() - t0:.1f} s")
        if not args.no_bos:
            prompts = [[cfg.bos_token_id] + p for p in prompts]
        batch = args.batch or len(prompts)
        need = sum(sorted(((len(p) + args.max_new + 63) // 64 * 64 for p in prompts), reverse=True)[:batch])
        engine = bb.Engine(model, max_tokens=max(need, 64), max_slots=batch)
        opts = bb.GenerateOptions(
            max_new_tokens=args.max_new,
            sampling=bb.SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p, seed=args.seed),
            stop_on_eos=not args.no_eos, stop_ids=tuple(args.stop_id))
        t0 = time.time()
        outs = bb.generate(engine, prompts, eos_id=cfg.eos_token_id, opts=opts, batch_size=batch)
        dt = time.time() - t0
        for p, o in zip(prompts, outs):
            print(f"[info] prompt tokens: {len(p)}")
            print("--- prompt ---")
            print(" ".join(map(str, p)))
            print("--- completion ---")
            print(" ".join(map(str, o)))
            if tokenizer is not None:
                print("--- text ---")
                print(tokenizer.decode(o))
            print(f"[info] generated {len(o)} tokens")
        total = sum(len(o) for o in outs)
        print(f"[info] {total} tokens in {dt:.2f} s ({total / max(dt, 1e-9):.1f} tokens/s, first call includes "
              f"kernel and graph set-up)")
    except Exception as e:  # noqa: BLE001 - the tool reports and exits, as the reference's tools do
        print(f"fatal: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""The command line, in the reference's manner (apps/oracle_cli.cpp:27-85):

    oracle -m <model_dir> -p <prompt> [options]
    oracle -m <model_dir> --tokens 1,2,3 [--tokens 4,5 ...] [options]

Options with the reference's names, defaults and meanings:
    -m <dir>        model folder (config.json + safetensors); required
    -p <text>       prompt (needs tokenizer.json in the folder)
    -n <N>          tokens to generate                      (default 256)
    --temp <f>      temperature; <= 0 is greedy             (default 0.7)
    --top-p <f>     nucleus top-p                           (default 0.9)
    --no-stream     print each answer in one block
    -h, --help
This library's own:
    --tokens a,b,c  a prompt as token ids (repeatable: a batch); prints token ids
    --top-k <N>     (default 40, the value the reference's engine fixes)   --seed <N> (default 0)
    --repeat-penalty <f> (default 1.15)   --repeat-last-n <N> (default 64)
    --stop-id <N>   extra stop id (repeatable)   --ignore-eos
    --dtype bfloat16|float32 (default bfloat16)   --max-tokens <N> cache size in tokens
    --batch <N>     requests per batch (default: all at once)
    --step-tokens <N>  most prompt tokens per step (longer prompts go through in portions)
    --profile       device time per kind of kernel, on standard error (runs without CUDA graphs)
    --random-weights <seed> --config <config.json>   run a configuration with seeded random weights
Unknown option or missing -m / prompt: usage, exit 2.  Model cannot be loaded: exit 1.
The reference's --system and --draft (chat template, speculative decoding) are not part of
this library.
"""
from __future__ import annotations

import json
import sys

USAGE = """Usage: {exe} -m <model_dir> (-p <prompt> | --tokens <ids>) [options]
  -n <N>          tokens to generate      (default 256)
  --temp <f>      temperature             (default 0.7)
  --top-p <f>     nucleus top-p           (default 0.9)
  --top-k <N>     top-k                   (default 40)
  --tokens a,b,c  prompt as token ids (repeatable)
  --seed <N>  --repeat-penalty <f>  --repeat-last-n <N>  --stop-id <N>  --ignore-eos
  --dtype bfloat16|float32  --max-tokens <N>  --batch <N>  --step-tokens <N>  --profile
  --random-weights <seed> --config <config.json>
  --no-stream     print the answer in one block
"""


def main(argv=None) -> int:
    argv = list(sys.argv if argv is None else argv)
    exe, args = argv[0], argv[1:]
    from ..sampling.params import GenParams
    params = GenParams()
    opt = {"model": "", "prompt": "", "tokens": [], "stream": True, "dtype": "bfloat16", "max_tokens": 0,
           "batch": None, "stop": [], "random": None, "config": "", "step_tokens": None, "profile": False}
    i = 0

    def val(name):
        nonlocal i
        if i + 1 >= len(args):
            sys.stderr.write(f"missing value after {name}\n")
            raise SystemExit(2)
        i += 1
        return args[i]

    try:
        while i < len(args):
            k = args[i]
            if k == "-m":
                opt["model"] = val(k)
            elif k == "-p":
                opt["prompt"] = val(k)
            elif k == "-n":
                params.n_predict = int(val(k))
            elif k == "--temp":
                params.temperature = float(val(k))
            elif k == "--top-p":
                params.top_p = float(val(k))
            elif k == "--top-k":
                params.top_k = int(val(k))
            elif k == "--seed":
                params.seed = int(val(k))
            elif k == "--repeat-penalty":
                params.repeat_penalty = float(val(k))
            elif k == "--repeat-last-n":
                params.repeat_last_n = int(val(k))
            elif k == "--tokens":
                opt["tokens"].append([int(t) for t in val(k).replace(" ", "").split(",") if t])
            elif k == "--stop-id":
                opt["stop"].append(int(val(k)))
            elif k == "--ignore-eos":
                params.ignore_eos = True
            elif k == "--dtype":
                opt["dtype"] = val(k)
            elif k == "--max-tokens":
                opt["max_tokens"] = int(val(k))
            elif k == "--batch":
                opt["batch"] = int(val(k))
            elif k == "--step-tokens":
                opt["step_tokens"] = int(val(k))
            elif k == "--profile":
                opt["profile"] = True
            elif k == "--random-weights":
                opt["random"] = int(val(k))
            elif k == "--config":
                opt["config"] = val(k)
            elif k == "--no-stream":
                opt["stream"] = False
            elif k in ("-h", "--help"):
                sys.stderr.write(USAGE.format(exe=exe))
                return 0
            else:
                sys.stderr.write(f"unknown option: {k}\n")
                sys.stderr.write(USAGE.format(exe=exe))
                return 2
            i += 1
    except ValueError as e:
        sys.stderr.write(f"bad value: {e}\n")
        return 2
    have_model = bool(opt["model"]) or (opt["random"] is not None and opt["config"])
    if not have_model or (not opt["prompt"] and not opt["tokens"]):
        sys.stderr.write(USAGE.format(exe=exe))
        return 2

    from ..tokenizer.bpe import Tokenizer
    try:
        from .engine import Engine
        need = sum(len(t) for t in opt["tokens"]) + 4096 + (len(opt["tokens"]) + 1) * (params.n_predict + 64)
        max_tokens = opt["max_tokens"] or need
        if opt["random"] is not None:
            from ..config.base import architecture_name, get_architecture
            raw = json.loads(open(opt["config"]).read())
            config = get_architecture(architecture_name(raw)).config_cls.from_dict(raw)
            engine = Engine.from_config(config, seed=opt["random"], dtype=opt["dtype"], max_tokens=max_tokens,
                                        use_graphs=not opt["profile"])
            tok = None
        else:
            engine = Engine.from_pretrained(opt["model"], dtype=opt["dtype"], max_tokens=max_tokens,
                                            use_graphs=not opt["profile"])
            tok = Tokenizer.from_folder(opt["model"], engine.spec.bos_id)
    except Exception as e:                                   # noqa: BLE001 - reported, exit code 1 as the reference
        sys.stderr.write(f"error: failed to load model '{opt['model'] or opt['config']}': {e}\n")
        return 1

    prompts = list(opt["tokens"])
    text_mode = bool(opt["prompt"])
    if text_mode:
        if tok is None:
            sys.stderr.write("error: -p needs a tokenizer.json in the model folder; use --tokens for token ids\n")
            return 1
        prompts.append(tok.encode(opt["prompt"], add_bos=True))
    if opt["stop"]:
        params.stop_ids = tuple(engine.spec.stop_ids) + tuple(opt["stop"])

    single = len(prompts) == 1
    pending = b""

    def on_token(index, token):
        nonlocal pending
        if not (opt["stream"] and single):
            return
        if text_mode:
            pending += tok.decode_bytes(token)
            try:
                piece, pending = pending.decode("utf-8"), b""
            except UnicodeDecodeError:
                return
            sys.stdout.write(piece)
        else:
            sys.stdout.write(f"{token} ")
        sys.stdout.flush()

    try:
        if opt["profile"]:
            from .profile import KernelProfile
            with KernelProfile() as prof:
                outs = engine.generate(prompts, params, batch_size=opt["batch"], on_token=on_token,
                                       max_step_tokens=opt["step_tokens"])
            prof.report(sys.stderr)
        else:
            outs = engine.generate(prompts, params, batch_size=opt["batch"], on_token=on_token,
                                   max_step_tokens=opt["step_tokens"])
    except Exception as e:                                   # noqa: BLE001 - a kernel's error flag included
        sys.stderr.write(f"error: {e}\n")
        return 1
    if opt["stream"] and single:
        sys.stdout.write("\n")
    else:
        for out in outs:
            sys.stdout.write((tok.decode(out) if text_mode and single else " ".join(map(str, out))) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())

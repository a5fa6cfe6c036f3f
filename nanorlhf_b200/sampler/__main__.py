"""Generate from a checkpoint folder with the in-process rollout engine of its model family.

    python -m nanorlhf_b200.sampler --model DIR --prompt-ids 5,17,3 [--prompt-ids ...] [--n 1] [--max-tokens 32]
                                    [--temperature 0] [--top-p 1.0] [--seed 0] [--dtype bfloat16|float32] [--eos -1]

The model class and its engine (whole-prompt paged-KV engine or the step engine of hybrid decoders) are chosen by
``config.json``.  Prints one JSON line per sample: {"prompt": i, "sample": j, "tokens": [...]}.
"""
import argparse
import json
import sys


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for more prompts")
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--eos", type=int, default=-1, help="stop token id (-1: none)")
    ap.add_argument("--pad", type=int, default=0)
    a = ap.parse_args()
    import torch
    from ..csrc.build import build
    build(verbose=False)
    from ..models.registry import load_model, sampler_kind
    from .engine import generate

    class _Tok:                                   # the engine only needs the two special ids
        pad_token_id, eos_token_id = a.pad, (a.eos if a.eos >= 0 else None)

    dev = torch.device("cuda:0")
    model = load_model(a.model, torch.float32 if a.dtype == "float32" else torch.bfloat16, dev)
    prompts = [[int(t) for t in p.split(",")] for p in a.prompt_ids]
    kw = {"rollout_dtype": a.dtype} if sampler_kind(model) == "hybrid" else {}
    out = generate(a.n, model, _Tok, prompts, a.temperature, a.max_tokens, top_p=a.top_p, seed=a.seed, backend="native",
                   eos_token_id=a.eos, **kw).tolist()
    for i in range(len(prompts)):
        for j in range(a.n):
            print(json.dumps({"prompt": i, "sample": j, "tokens": out[i * a.n + j]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())

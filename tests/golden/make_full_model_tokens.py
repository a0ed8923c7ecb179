"""Generates the full-model greedy-decode fixtures from the CPU oracle.

    python tests/golden/make_full_model_tokens.py            full_model_tokens.json
    python tests/golden/make_full_model_tokens.py --batch8   full_model_tokens_batch8.json

full_model_tokens.json: the oracle's greedy decode of the full synthetic decoder (36 layers,
4096 / 12288, 32 x 8 x 128, vocab 151936, seed 0) after the 512-token seeded prompt, 64 steps.
full_model_tokens_batch8.json: eight independent sequences of the same model, prompts of 64
tokens drawn from Philox keys (seed, 1000 + b), 32 greedy steps each (the shorter prompt keeps
the generation within half an hour of CPU time; the weights are the same 36 layers).

Per step the files hold the oracle's token, its runner-up and the logit margin between the
two, so that a teacher-forced replay (feed the oracle's token at every step, compare the
argmax of every step) can tell a tie that any fp32 summation order may break from a wrong
token.  About half an hour each on 8 cores."""
import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from smelt_b200 import package  # noqa: E402

SEED = 0


def prompt_tokens(vocab: int, n: int, b: int = 0) -> np.ndarray:
    return np.random.Generator(np.random.Philox(key=[SEED, 1000 + b])).integers(0, vocab, size=n).astype(np.int32)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch8", action="store_true")
    args = ap.parse_args()
    cfg = package.FULL_MODEL
    pkg = package.SyntheticPackage(cfg, SEED)
    n_prompt, n_decode, batch = (64, 32, 8) if args.batch8 else (512, 64, 1)
    t0 = time.time()
    model = oracle.model_from_package(pkg, n_prompt + n_decode + 8)
    print("model ready in %.0f s" % (time.time() - t0), flush=True)
    rows = []
    for b in range(batch):
        t0 = time.time()
        rows.append(model.greedy_top2(prompt_tokens(cfg.vocab, n_prompt, b), n_decode))
        print("sequence %d generated in %.0f s: %s" % (b, time.time() - t0, rows[-1][0]), flush=True)
    out = {"seed": SEED, "prompt_len": n_prompt, "n_decode": n_decode, "config": cfg.as_dict(),
           "prompt_rng": "numpy Philox(key=[seed, 1000 + b]).integers(0, vocab, prompt_len), b = sequence index"}
    if args.batch8:
        out.update(batch=batch, tokens=[r[0] for r in rows], runner_up=[r[1] for r in rows], top2_margin=[r[2] for r in rows])
        name = "full_model_tokens_batch8.json"
    else:
        out.update(tokens=rows[0][0], runner_up=rows[0][1], top2_margin=rows[0][2])
        name = "full_model_tokens.json"
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), name), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()

"""Generates full_model_tokens.json: the CPU oracle's greedy decode of the full synthetic
decoder (36 layers, 4096 / 12288, 32 x 8 x 128, vocab 151936, seed 0) after the 512-token seeded
prompt, 64 steps, with the oracle's top-2 logit margin per step.

    python tests/golden/make_full_model_tokens.py        (about half an hour on 8 cores)

The GPU parity test replays the same prompt through the dispatch-record runtime and compares
token ids."""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from smelt_b200 import package  # noqa: E402

SEED, PROMPT_LEN, N_DECODE = 0, 512, 64


def prompt_tokens(vocab: int) -> np.ndarray:
    return np.random.Generator(np.random.Philox(key=[SEED, 1000])).integers(0, vocab, size=PROMPT_LEN).astype(np.int32)


def main():
    cfg = package.FULL_MODEL
    pkg = package.SyntheticPackage(cfg, SEED)
    t0 = time.time()
    model = package.oracle_model(oracle, pkg, PROMPT_LEN + N_DECODE + 8)
    print("model ready in %.0f s" % (time.time() - t0), flush=True)
    t0 = time.time()
    toks, margins = model.generate(prompt_tokens(cfg.vocab), N_DECODE)
    print("generated in %.0f s" % (time.time() - t0), flush=True)
    out = {"seed": SEED, "prompt_len": PROMPT_LEN, "n_decode": N_DECODE, "config": cfg.as_dict(),
           "prompt_rng": "numpy Philox(key=[seed, 1000]).integers(0, vocab, 512)",
           "tokens": [int(t) for t in toks], "top2_margin": [float(m) for m in margins]}
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "full_model_tokens.json"), "w") as f:
        json.dump(out, f, indent=1)
    print(out["tokens"])


if __name__ == "__main__":
    main()

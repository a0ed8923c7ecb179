"""Benchmark configuration 4 end to end: the full 36-layer synthetic decoder on one GPU against
the CPU oracle's greedy tokens (tests/golden/full_model_tokens*.json, written by
tests/golden/make_full_model_tokens.py).

The comparison is teacher-forced: the oracle's token is fed at every step whatever the GPU
chose, and the GPU's argmax of EVERY step is compared.  A differing id is accepted only where
the oracle's own top-2 logits are within two fp16 ulps (margin < 0.02) and the GPU picked the
oracle's runner-up; the count of identical steps is printed."""
import json
import os

import numpy as np
import pytest

from smelt_b200 import capi, package

pytestmark = pytest.mark.gpu

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    with open(os.path.join(GOLDEN_DIR, name)) as f:
        gold = json.load(f)
    assert gold["config"] == package.FULL_MODEL.as_dict()
    return gold


def prompts_of(gold, batch):
    return np.stack([np.random.Generator(np.random.Philox(key=[gold["seed"], 1000 + b])).integers(0, package.FULL_MODEL.vocab, size=gold["prompt_len"])
                     for b in range(batch)]).astype(np.int32)


def run(gold, batch, fuse):
    cfg = package.FULL_MODEL
    n_prompt, n_dec = gold["prompt_len"], gold["n_decode"]
    tokens = np.array(gold["tokens"], np.int32).reshape(batch, n_dec)
    ctx = capi.Context(0)
    try:
        pkg = package.SyntheticPackage(cfg, gold["seed"])
        image, desc, layers = package.build_image(pkg)
        dec = package.Decoder(ctx, image, desc, layers, n_prompt + n_dec + 8, batch, fuse_residual=fuse)
        del image
        got = dec.teacher_forced(prompts_of(gold, batch), tokens.T, use_graph=True)
        assert ctx.device_error() == 0
    finally:
        ctx.close()
    runner, margins = np.array(gold["runner_up"]).reshape(batch, n_dec), np.array(gold["top2_margin"]).reshape(batch, n_dec)
    return [package.compare_greedy(got[:, b], tokens[b], runner[b], margins[b]) for b in range(batch)]


@pytest.mark.parametrize("fuse", [3, 0])
def test_full_model_greedy_tokens_match_the_oracle(fuse):
    """Batch 1: 64 steps after the 512-token prompt, fused and reference-shaped tables."""
    gold = load("full_model_tokens.json")
    (v,) = run(gold, 1, fuse)
    print("full model, batch 1, fuse=%d: %d of %d steps identical, %d tie breaks, first mismatch %s (margin %s)" %
          (fuse, v["identical"], v["checked"], v["tie_breaks"], v["first_mismatch"], v["margin"]))
    assert v["checked"] == 64 and not v["wrong"], v
    near_ties = int(np.sum(np.array(gold["top2_margin"]) < 0.02))
    assert v["identical"] >= 64 - near_ties


def test_full_model_batch8_greedy_tokens_match_the_oracle():
    """Batch 8: eight independent sequences (64-token prompts, 32 steps each; the shorter prompt
    keeps the oracle's generation of the fixture within half an hour)."""
    gold = load("full_model_tokens_batch8.json")
    assert gold["batch"] == 8
    outcomes = run(gold, 8, 3)
    for b, v in enumerate(outcomes):
        print("full model, batch 8, sequence %d: %d of %d steps identical, %d tie breaks" % (b, v["identical"], v["checked"], v["tie_breaks"]))
        assert v["checked"] == gold["n_decode"] and not v["wrong"], (b, v)


def test_full_model_prefill_then_greedy_tokens_match_the_oracle():
    """The 512-token prompt through smelt_cuda_prefill (chunks of 128 positions: tensor-memory QMM,
    batched RoPE / KV write, chunked causal attention), then the 64 teacher-forced steps."""
    gold = load("full_model_tokens.json")
    cfg = package.FULL_MODEL
    n_prompt, n_dec = gold["prompt_len"], gold["n_decode"]
    tokens = np.array(gold["tokens"], np.int32)
    ctx = capi.Context(0)
    try:
        pkg = package.SyntheticPackage(cfg, gold["seed"])
        image, desc, layers = package.build_image(pkg)
        dec = package.Decoder(ctx, image, desc, layers, n_prompt + n_dec + 8, 1, fuse_residual=3)
        del image
        first = dec.prefill(prompts_of(gold, 1)[0], 0, 128)
        dec.build_graph()
        got = [first]
        for i in range(n_dec - 1):
            dec.graph_seed(tokens[i:i + 1], n_prompt + i)
            got.append(int(dec.graph_decode(1, read=True)[0, 0]))
        assert ctx.device_error() == 0
    finally:
        ctx.close()
    v = package.compare_greedy(np.array(got), tokens, np.array(gold["runner_up"]), np.array(gold["top2_margin"]))
    print("full model, prefill + decode: %d of %d steps identical, %d tie breaks, first mismatch %s" % (v["identical"], v["checked"], v["tie_breaks"], v["first_mismatch"]))
    assert v["checked"] == 64 and not v["wrong"], v

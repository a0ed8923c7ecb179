"""A hybrid decoder (DeltaNet layers between attention layers, Sources/SmeltCompiler/DeltaNetPlugin.swift:60-420)
through the table smelt_cuda_build_hybrid_decoder writes: teacher-forced tokens against the oracle's hybrid model,
eagerly and from the captured graph, and a prompt-state snapshot that carries the recurrent state."""
import numpy as np
import pytest

from smelt_b200 import capi, package

pytestmark = pytest.mark.gpu

# three linear-attention layers to one attention layer, as the published hybrid models interleave them
GENERIC = package.DecoderConfig(layers=4, hidden=512, inter=1024, n_q=4, n_kv=2, head_dim=64, vocab=1024, delta_layers=(0, 1, 2),
                                delta_value_heads=8, delta_qk_heads=4, delta_head_dim=64)
D128 = package.DecoderConfig(layers=4, hidden=1024, inter=3072, n_q=8, n_kv=2, head_dim=128, vocab=2048, delta_layers=(0, 2, 3),
                             delta_value_heads=16, delta_qk_heads=16, delta_head_dim=128)


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("cfg,fuse", [(GENERIC, 0), (GENERIC, 3), (D128, 3)])
def test_hybrid_decoder_decodes_the_oracle_tokens(ctx, oracle, cfg, fuse):
    cap, n_dec = 96, 40
    pkg = package.SyntheticPackage(cfg, 31)
    image, desc, layers, hy = package.build_hybrid_image(pkg, keep_for_oracle=True)
    dec = package.Decoder(ctx, image, desc, layers, cap, 1, fuse_residual=fuse, hybrid=hy)
    ref = oracle.model_from_package(pkg, cap)
    prompt = np.array([7, 99, 500, 3, 42, 17], np.int32)
    want, runner, margins = ref.greedy_top2(prompt, n_dec)
    feed = list(prompt) + list(want[:-1])
    got = []
    for pos, tok in enumerate(feed):
        out = int(dec.decode_step([tok], pos)[0])
        if pos >= len(prompt) - 1:
            got.append(out)
    v = package.compare_greedy(np.array(got), want, runner, margins)
    print("hybrid: %d of %d identical, %d tie breaks" % (v["identical"], v["checked"], v["tie_breaks"]))
    assert v["checked"] == n_dec and not v["wrong"], v
    # the captured graph replays the same table from zeroed state: seed one token, replay one step
    dec.reset_cache()
    dec.build_graph()
    got_graph = []
    for pos, tok in enumerate(feed):
        dec.graph_seed([tok], pos)
        out = int(dec.graph_decode(1, read=True)[0, 0])
        if pos >= len(prompt) - 1:
            got_graph.append(out)
    assert got_graph == got
    assert ctx.device_error() == 0


def test_hybrid_snapshot_carries_the_recurrent_state(ctx, oracle):
    cfg, cap = GENERIC, 64
    pkg = package.SyntheticPackage(cfg, 37)
    image, desc, layers, hy = package.build_hybrid_image(pkg, keep_for_oracle=True)
    dec = package.Decoder(ctx, image, desc, layers, cap, 1, fuse_residual=3, hybrid=hy)
    prompt = [11, 5, 900, 64, 2, 77, 300, 8]
    tok = None
    for pos, t in enumerate(prompt):
        tok = int(dec.decode_step([t], pos)[0])
    snap = dec.capture_snapshot(len(prompt), len(prompt), tok)
    cont = []
    cur = tok
    for i in range(10):
        cur = int(dec.decode_step([cur], len(prompt) + i)[0])
        cont.append(cur)
    # wipe everything, restore, and the continuation repeats bit for bit
    dec.reset_cache()
    dec.restore_snapshot(snap)
    again, cur = [], tok
    for i in range(10):
        cur = int(dec.decode_step([cur], len(prompt) + i)[0])
        again.append(cur)
    assert again == cont
    # a recurrent state has no positions to rewind to: a shorter restore is refused
    with pytest.raises(capi.SmeltError):
        dec.restore_snapshot(snap, len(prompt) - 2)
    snap.close()


@pytest.mark.parametrize("cfg,chunk", [(GENERIC, 16), (GENERIC, 24), (D128, 20), (D128, 80)])
def test_hybrid_prefill_table_matches_the_oracles_chunked_prefill(ctx, oracle, cfg, chunk):
    """The prompt of a hybrid decoder through its prompt-chunk table (batched projections, conv1d_update_silu_prefill,
    deltanet_recurrence_mlx_prefill, the gated norm per position and head) against the oracle running the same chunks
    layer by layer; then the oracle's continuation from the state the table left.  The recurrent rows stay in fp32
    across a chunk in both, so the two must chunk alike."""
    n_prompt, n_dec = 90, 16
    cap = n_prompt + n_dec + 8
    pkg = package.SyntheticPackage(cfg, 41)
    image, desc, layers, hy = package.build_hybrid_image(pkg, keep_for_oracle=True)
    dec = package.Decoder(ctx, image, desc, layers, cap, 1, fuse_residual=3, hybrid=hy)
    dec.build_prefill_table(chunk)
    ref = oracle.model_from_package(pkg, cap)
    prompt = np.random.default_rng(41).integers(0, cfg.vocab, size=n_prompt).astype(np.int32)
    ref.reset()
    want0, want_logits = ref.prefill(prompt, 0, chunk, want_logits=True)
    got0 = dec.prefill_by_table(prompt)
    got_logits = dec.logits()[0].astype(np.float32)
    wl = want_logits.astype(np.float32)
    err = float(np.max(np.abs(got_logits - wl)) / np.sqrt(np.mean(wl * wl)))
    assert err < 1e-2, err
    best, second, margin = oracle.top2(want_logits)
    assert got0 == best or (margin < 0.02 and got0 == second), (got0, best, second, margin)
    # teacher-forced continuation: the oracle continues from its own prefill state, the library from the table's
    tok = want0
    for i in range(n_dec):
        w, wlog = ref.decode_step(int(tok), n_prompt + i, want_logits=True)
        g = int(dec.decode_step([int(tok)], n_prompt + i)[0])
        b, s2, mg = oracle.top2(wlog)
        assert g == b or (mg < 0.02 and g == s2), (i, g, b, s2, mg)
        tok = w
    assert ctx.device_error() == 0

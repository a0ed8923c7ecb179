"""The .smeltpkg reader: host-side validation (no GPU) of manifest.json / weights.bin /
dispatches.bin as SmeltRuntime.init applies it (Sources/SmeltRuntime/SmeltRuntime.swift:668-998,
:6322-6350), and, on a GPU, a package read from disk decoding the oracle's tokens."""
import json
import os

import numpy as np
import pytest

from smelt_b200 import capi, package, synth

CFG = package.DecoderConfig(layers=2, hidden=1024, inter=3072, n_q=8, n_kv=2, head_dim=128, vocab=2048)


@pytest.fixture(scope="module")
def pkg_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("pkg") / "model.smeltpkg")
    pkg = package.SyntheticPackage(CFG, 5)
    image, desc, layers = package.build_image(pkg)
    package.write_package(d, CFG, image, desc, layers, 48, fuse_residual=0)
    return d


def _copy(src, dst, patch=None, drop=()):
    os.makedirs(dst)
    for name in os.listdir(src):
        if name in drop:
            continue
        data = open(os.path.join(src, name), "rb").read()
        if name == "manifest.json" and patch:
            m = json.loads(data)
            patch(m)
            data = json.dumps(m).encode()
        open(os.path.join(dst, name), "wb").write(data)
    return dst


def test_inspect_reports_the_package(pkg_dir):
    st, info, err = package.inspect_package(pkg_dir)
    assert st == capi.OK, err
    assert info.vocab_size == CFG.vocab and info.hidden_size == CFG.hidden and info.num_layers == CFG.layers
    assert (info.token_id_slot, info.position_slot, info.weights_slot, info.argmax_slot, info.logits_slot) == (33, 34, 30, 17, 16)
    assert info.n_records == os.path.getsize(os.path.join(pkg_dir, "dispatches.bin")) // 360
    assert info.n_pipelines_used == info.n_pipelines > 5
    assert info.n_weight_entries == 7 * CFG.layers + 2 * CFG.layers + 3
    assert info.weights_bytes == os.path.getsize(os.path.join(pkg_dir, "weights.bin"))


def test_inspect_rejects_broken_packages(pkg_dir, tmp_path):
    # dispatches.bin must be a whole number of 360-byte records (SmeltRuntime.swift:6332-6338)
    d = _copy(pkg_dir, str(tmp_path / "stride"))
    with open(os.path.join(d, "dispatches.bin"), "ab") as f:
        f.write(b"\0" * 7)
    st, _, err = package.inspect_package(d)
    assert st == capi.BAD_ARGUMENT and "not a multiple of dispatch stride 360" in err
    # a kernel outside the implemented set, used by the table: no silent default
    def rename(m):
        m["pipelines"][m["pipelines"].index("embedding_gather")] = "fused_lut_matvec"
    st, _, err = package.inspect_package(_copy(pkg_dir, str(tmp_path / "unknown"), rename))
    assert st == capi.UNKNOWN_PIPELINE and "fused_lut_matvec" in err
    # ... but an unknown kernel the decode table never dispatches is fine (prefill kernels live in the same list)
    st, info, err = package.inspect_package(_copy(pkg_dir, str(tmp_path / "unused"), lambda m: m["pipelines"].append("prefill_attention_causal")))
    assert st == capi.OK and info.n_pipelines == info.n_pipelines_used + 1
    # a record naming a pipeline index the manifest does not list
    st, _, err = package.inspect_package(_copy(pkg_dir, str(tmp_path / "short"), lambda m: m["pipelines"].pop()))
    assert st == capi.UNKNOWN_PIPELINE and "names pipeline" in err
    # a weight entry that runs past weights.bin
    def grow(m):
        m["weights"]["entries"][3]["scales_offset"] = m["weights"]["total_bytes"] - 8
    st, _, err = package.inspect_package(_copy(pkg_dir, str(tmp_path / "weights"), grow))
    assert st == capi.OUT_OF_RANGE and "outside weights.bin" in err
    # weights.bin shorter than the manifest says
    d = _copy(pkg_dir, str(tmp_path / "truncated"))
    size = os.path.getsize(os.path.join(d, "weights.bin"))
    with open(os.path.join(d, "weights.bin"), "r+b") as f:
        f.truncate(size - 4096)
    st, _, err = package.inspect_package(d)
    assert st == capi.OUT_OF_RANGE and "manifest declares" in err
    # missing pieces
    for name, patch in (("noslots", lambda m: m.pop("buffers")), ("nolayout", lambda m: m["slotLayout"].pop("tokenIdSlot")),
                        ("novocab", lambda m: m["config"].pop("vocabSize"))):
        st, _, err = package.inspect_package(_copy(pkg_dir, str(tmp_path / name), patch))
        assert st == capi.BAD_ARGUMENT and "missing" in err
    st, _, err = package.inspect_package(_copy(pkg_dir, str(tmp_path / "notable"), drop=("dispatches.bin",)))
    assert st == capi.BAD_ARGUMENT and "dispatches.bin" in err
    os.makedirs(str(tmp_path / "junk"))
    open(str(tmp_path / "junk" / "manifest.json"), "w").write('{"pipelines": [1, 2')
    st, _, err = package.inspect_package(str(tmp_path / "junk"))
    assert st == capi.BAD_ARGUMENT and "manifest.json" in err


def test_manifest_keys_follow_the_reference_schema(pkg_dir):
    """Top-level and slotLayout keys camelCase, weight entries and buffer slots snake_case
    (SmeltManifest.swift:26-98, :806-817, :1710-1724, :1764-1767)."""
    m = json.load(open(os.path.join(pkg_dir, "manifest.json")))
    assert {"version", "modelName", "config", "checksums", "device", "weights", "buffers", "pipelines", "slotLayout"} <= set(m)
    assert {"keyCacheBaseSlot", "valCacheBaseSlot", "tokenIdSlot", "positionSlot", "weightsSlot", "ropeTablePairs"} <= set(m["slotLayout"])
    e = m["weights"]["entries"][0]
    assert {"name", "offset", "size_bytes", "shape", "dtype", "group_size", "scales_offset", "biases_offset"} <= set(e) and e["dtype"] == "affine_u4"
    s = m["buffers"]["slots"][0]
    assert set(s) == {"index", "name", "size_bytes", "dtype", "shape", "category"}
    assert any(x["name"] == "keyCache_0" and x["shape"] == [CFG.n_kv, 48, CFG.head_dim] for x in m["buffers"]["slots"])


@pytest.mark.gpu
@pytest.mark.parametrize("fuse", [0, 3])
def test_package_from_disk_decodes_the_oracle_tokens(tmp_path, oracle, fuse):
    """write -> smelt_cuda_open_package -> decode_step / captured graph, with the KV caches grown
    from the compiled 48 positions to 80 at load: the oracle's tokens at every teacher-forced step."""
    d = str(tmp_path / "m.smeltpkg")
    pkg = package.SyntheticPackage(CFG, 5)
    image, desc, layers = package.build_image(pkg, keep_for_oracle=True)
    package.write_package(d, CFG, image, desc, layers, 48, fuse_residual=fuse)
    ref = oracle.model_from_package(pkg, 80)
    prompt = np.array([7, 99, 1500, 3, 42], np.int32)
    want, runner, margins = ref.greedy_top2(prompt, 60)  # runs past the compiled 48 positions
    ctx = capi.Context(0)
    try:
        ses = package.PackageSession(ctx, d, context_capacity=80)
        assert ses.info.cache_seq_capacity == 80 and ses.info.n_records == ses.n_records
        feed = list(prompt) + list(want[:-1])
        got = []
        for pos, tok in enumerate(feed):
            out = ses.decode_step(int(tok), pos)
            if pos >= len(prompt) - 1:
                got.append(out)
        v = package.compare_greedy(np.array(got), want, runner, margins)
        assert not v["wrong"], v
        # the captured graph replays the same table
        ses.build_graph()
        for l in range(2 * CFG.layers):
            ctx.call("zero_slot", package.KV_BASE_SLOT + l)
        got_graph = []
        for pos, tok in enumerate(feed):
            out = ses.graph_step(int(tok), pos)
            if pos >= len(prompt) - 1:
                got_graph.append(out)
        assert got_graph == got
        assert ctx.device_error() == 0
        st = ctx.lib.smelt_cuda_decode_step(ctx.h, ses.table, ses.n_records, np.array([1], np.int32).ctypes.data_as(capi.C.c_void_p), 80, None)
        assert st == capi.OUT_OF_RANGE  # past the context the package was opened for
    finally:
        ctx.close()


def test_inspect_counts_the_prefill_table(tmp_path):
    d = str(tmp_path / "p.smeltpkg")
    pkg = package.SyntheticPackage(CFG, 6)
    image, desc, layers = package.build_image(pkg)
    package.write_package(d, CFG, image, desc, layers, 48, prefill_chunk=16)
    st, info, err = package.inspect_package(d)
    assert st == 0, err
    assert info.n_prefill_records == 5 + 9 * CFG.layers  # gather + nine records per layer + final norm, LM head, two argmax
    # a prefill table that names a kernel this library does not bind leaves the package openable for decoding
    m = json.load(open(os.path.join(d, "manifest.json")))
    m["pipelines"][-1] = "fused_lut_matmul"
    json.dump(m, open(os.path.join(d, "manifest.json"), "w"))
    st, info, err = package.inspect_package(d)
    assert st == 0 and info.n_prefill_records == 0 and info.n_records > 0


@pytest.mark.gpu
def test_package_prefill_table_then_decode(tmp_path, oracle):
    """A package with prefill_dispatches.bin: the prompt in chunks through its own prompt-chunk table, then the
    oracle's tokens from its decode table."""
    d = str(tmp_path / "p.smeltpkg")
    pkg = package.SyntheticPackage(CFG, 7)
    image, desc, layers = package.build_image(pkg, keep_for_oracle=True)
    package.write_package(d, CFG, image, desc, layers, 64, fuse_residual=3, prefill_chunk=16)
    ref = oracle.model_from_package(pkg, 64)
    prompt = synth.rng_for(7, "package prompt").integers(0, CFG.vocab, size=37).astype(np.int32)
    want, runner, margins = ref.greedy_top2(prompt, 20)
    ctx = capi.Context(0)
    try:
        ses = package.PackageSession(ctx, d)
        assert ses.info.n_prefill_records > 0
        got = [ses.prefill(prompt, 0, 16)]
        for i in range(19):
            got.append(ses.decode_step(int(want[i]), len(prompt) + i))
        v = package.compare_greedy(np.array(got), want, runner, margins)
        assert v["checked"] == 20 and not v["wrong"], v
        assert ctx.device_error() == 0
    finally:
        ctx.close()

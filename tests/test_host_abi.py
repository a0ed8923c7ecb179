"""CPU-side checks of the C ABI: the library loads and exports every declared symbol, the
record layout is the reference's, pipeline names resolve like the reference's kernel table,
and the decoder table builder emits the reference's per-token record sequence."""
import ctypes as C

import numpy as np
import pytest

from smelt_b200 import capi, package


@pytest.fixture(scope="module")
def lib():
    return capi.load()


def test_library_exports_every_declared_symbol(lib):
    names = capi.declared_symbols()
    assert len(names) >= 55
    for n in names:
        assert hasattr(lib, n), n


def test_no_device_means_loud_failure_not_a_cpu_path(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.smelt_cuda_create(0, C.byref(h)) != 0 and not h.value
    with pytest.raises(capi.SmeltError):
        capi.Context(0)


# Tests/SmeltCompilerTests/DispatchTableTests.swift:12-30 pins strides 16 / 8 / 360.
def test_dispatch_record_layout():
    assert C.sizeof(capi.BufferRecord) == 16 and C.sizeof(capi.ConstantRecord) == 8 and C.sizeof(capi.DispatchRecord) == 360
    D = capi.DispatchRecord
    assert (D.pipeline.offset, D.style.offset, D.buffer_count.offset, D.constant_count.offset) == (2, 4, 5, 6)
    assert (D.min_seq_len.offset, D.grid.offset, D.threadgroup.offset, D.buf.offset, D.con.offset) == (8, 12, 24, 40, 296)
    assert (capi.BufferRecord.binding_index.offset, capi.BufferRecord.offset_kind.offset, capi.BufferRecord.offset.offset) == (2, 3, 8)


@pytest.mark.parametrize("name,ok", [
    ("affine_matvec:4096:64", True), ("affine_matvec", True), ("affine_matvec_c1024_r4096_g64", True),
    ("affine_matvec_c2048_r6144_g64_batched_full", True), ("affine_matvec_c2560_r10240_g128_batched_ext_b5", True),
    ("fused_affine_matvec_add_c6144_r2048_g64", True), ("fused_affine_gate_up_swiglu_c2048_r6144_g64_batched", True),
    ("fused_dual_affine_matvec_c2048_r16_g64", True), ("fp16_matvec", True), ("embedding_gather", True),
    ("affine_embedding_gather", True), ("argmax_fp16_partials", True), ("argmax_key_reduce", True),
    ("signed_binary_matvec_g128_rows8", True), ("signed_ternary_matvec_g128_rows8", True),
    ("signed_binary_gate_up_swiglu_g128_rows8_batched_b4", True), ("signed_ternary_affine_matvec_g128_rows8", True),
    ("kv_cache_update", True), ("apply_rope", True), ("rope_kv_cache_update", True), ("attention_decode", True),
    ("attention_decode_d256_h16_kv4", True), ("attention_decode_d128_h16_kv2_sdpa", True), ("attention_decode_mlx_vector_d256", True),
    ("rms_norm_1pw", True), ("per_head_rms_norm", True), ("elementwise_add", True), ("swiglu_fused", True),
    # outside the hot path: no silent default (MatvecKernelTable.swift:258-270)
    ("smelt_rmsnorm_affine_qkv:4096:64", True), ("smelt_rmsnorm_affine_gate_up_swiglu:4096:64", True), ("smelt_rope_qkv_append", True), ("smelt_rope_attention_decode", True),
    ("smelt_rmsnorm_affine_qkv:4096:32", False), ("smelt_rmsnorm_affine_qkv:512:64", False),
    ("fused_lut_matvec", False), ("tqh_matvec", False), ("attention_decode_softcap", False), ("affine_matvec:4096:48", False),
    ("attention_decode_mlx_vector_2pass_1_d256_b128", True), ("attention_decode_mlx_vector_2pass_2_d256_b128", True),
    ("attention_decode_mlx_vector_2pass_1_d128_b128", False), ("recurrence_step", False), ("", False),
])
def test_pipeline_names(lib, name, ok):
    assert bool(lib.smelt_cuda_pipeline_supported(name.encode())) == ok


def _table(cfg, batch, tp=1, fuse=False):
    lib = capi.load()
    desc = capi.DecoderDesc(layers=cfg.layers, hidden=cfg.hidden, inter=cfg.inter // tp, n_q=cfg.n_q // tp, n_kv=cfg.n_kv // tp,
                            head_dim=cfg.head_dim, vocab=cfg.vocab, group=64, eps=1e-6, rope_theta=1e6, embedding=0, lm_head=128,
                            final_norm=256, tp_world=tp, tp_rank=0, fuse_residual=int(fuse))
    layers = (capi.LayerRef * cfg.layers)()
    n = C.c_size_t(0)
    assert lib.smelt_cuda_build_decoder(None, C.byref(desc), layers, 128, batch, None, C.byref(n)) == 0
    table = (capi.DispatchRecord * n.value)()
    assert lib.smelt_cuda_build_decoder(None, C.byref(desc), layers, 128, batch, table, C.byref(n)) == 0
    need = C.c_size_t(0)
    assert lib.smelt_cuda_decoder_pipelines(C.byref(desc), batch, None, 0, C.byref(need)) == 0
    buf = C.create_string_buffer(need.value)
    assert lib.smelt_cuda_decoder_pipelines(C.byref(desc), batch, buf, need.value, C.byref(need)) == 0
    names = buf.value.decode().split("\n")[:-1]
    return table, names


def test_decoder_table_follows_the_reference_emitter():
    cfg = package.DecoderConfig(layers=2, hidden=4096, inter=12288, n_q=32, n_kv=8, head_dim=128, vocab=151936)
    table, names = _table(cfg, 1)
    seq = [names[r.pipeline] if r.op_kind == 0 else "<swap>" for r in table]
    layer = ["rms_norm_1pw", "affine_matvec:4096:64", "fused_dual_affine_matvec:4096:64", "apply_rope", "rope_kv_cache_update",
             "kv_cache_update", "attention_decode", "affine_matvec:4096:64", "elementwise_add", "<swap>", "rms_norm_1pw",
             "fused_affine_gate_up_swiglu:4096:64", "affine_matvec:12288:64", "elementwise_add", "<swap>"]
    assert seq == ["embedding_gather"] + layer * 2 + ["rms_norm_1pw", "fp16_matvec", "argmax_fp16_partials", "argmax_key_reduce"]
    # every name the builder emits is a registered kernel, bindings stay within the record's limits
    for n in names:
        assert capi.load().smelt_cuda_pipeline_supported(n.encode())
    attn = next(r for r in table if r.op_kind == 0 and names[r.pipeline] == "attention_decode")
    assert attn.grid[0] == 32 and attn.buffer_count == 5 and attn.constant_count == 6
    kinds = {attn.con[i].binding_index: attn.con[i].kind for i in range(attn.constant_count)}
    assert kinds[7] == capi.CONST_POSITION_PLUS1 and kinds[6] == capi.CONST_CACHE_SEQ_CAPACITY
    gate = next(r for r in table if r.op_kind == 0 and names[r.pipeline].startswith("fused_affine_gate_up"))
    assert [gate.buf[i].binding_index for i in range(gate.buffer_count)] == [0, 1, 2, 3, 4, 5, 6, 7]
    assert gate.con[0].binding_index == 8 and gate.con[0].value == 12288


def test_decoder_table_variants():
    cfg = package.DecoderConfig(layers=1, hidden=2048, inter=6144, n_q=16, n_kv=4, head_dim=128, vocab=1000)
    _, names_b = _table(cfg, 8)
    assert "affine_matvec_c2048_r2048_g64_batched" in names_b and "fused_affine_gate_up_swiglu_c2048_r6144_g64_batched" in names_b
    table_f, names_f = _table(cfg, 1, fuse=True)
    assert "fused_affine_matvec_add:2048:64" in names_f and "elementwise_add" not in names_f
    table_x, names_x = _table(cfg, 1, fuse=3)
    assert [names_x[r.pipeline] if r.op_kind == 0 else "<swap>" for r in table_x][1:8] == [
        "smelt_rmsnorm_affine_qkv:2048:64", "smelt_rope_attention_decode", "fused_affine_matvec_add:2048:64", "<swap>",
        "smelt_rmsnorm_affine_gate_up_swiglu:2048:64", "fused_affine_matvec_add:6144:64", "<swap>"]
    att = table_x[2]
    assert att.buffer_count == 6 and att.constant_count == 8  # every constant slot of a record is in use
    qkv = table_x[1]
    assert qkv.buffer_count == 14 and qkv.constant_count == 4
    small = package.DecoderConfig(layers=1, hidden=512, inter=1536, n_q=8, n_kv=2, head_dim=64, vocab=1000)
    assert not any(n.startswith("smelt_rmsnorm") for n in _table(small, 1, fuse=3)[1])  # hidden % 1024: reference-shaped records
    table_pm, names_pm = _table(cfg, 1, tp=2, fuse=6)
    seq_pm = [names_pm[r.pipeline] for r in table_pm if r.op_kind == 0]
    assert seq_pm.count("smelt_tp_reduce_add") == 2 and "smelt_tp_all_reduce" not in seq_pm and "elementwise_add" not in seq_pm
    table_vp, names_vp = _table(package.DecoderConfig(layers=1, hidden=2048, inter=6144, n_q=16, n_kv=4, head_dim=128, vocab=1000), 1, tp=2, fuse=14)
    seq_vp = [names_vp[r.pipeline] for r in table_vp if r.op_kind == 0]
    assert seq_vp[-3:] == ["fp16_matvec", "argmax_fp16_partials", "smelt_tp_argmax"]
    head = next(r for r in table_vp if r.op_kind == 0 and names_vp[r.pipeline] == "fp16_matvec")
    assert head.grid[0] == 500  # this rank's half of the vocabulary
    table_tp, names_tp = _table(cfg, 1, tp=2)
    seq = [names_tp[r.pipeline] for r in table_tp if r.op_kind == 0]
    assert seq.count("smelt_tp_all_reduce") == 2  # after O and after down
    i = seq.index("smelt_tp_all_reduce")
    assert seq[i - 1].startswith("affine_matvec") and seq[i + 1] == "elementwise_add"


def test_weights_image_layout():
    """Tensors start 128-byte aligned, packed -> scales -> biases, no overlap (WeightPackerTests.swift:43-97)."""
    img = package.WeightsImage()
    w = np.arange(10 * 32, dtype=np.uint8).reshape(10, 32)
    s = np.ones((10, 1), np.float16)
    b = np.full((10, 1), 2, np.float16)
    ref = img.add_affine(w, s, b)
    off = img.add(np.arange(5, dtype=np.float16))
    assert ref.packed % 128 == 0 and ref.scales % 128 == 0 and ref.biases % 128 == 0 and off % 128 == 0
    assert ref.packed + w.nbytes <= ref.scales and ref.scales + s.nbytes <= ref.biases and ref.biases + b.nbytes <= off
    raw = img.tobytes()
    assert np.array_equal(raw[ref.packed:ref.packed + 320], w.reshape(-1))
    assert raw.size % 128 == 0

"""Which of the reference's Metal kernels the library binds by name.  tests/golden/kernel_names.txt lists every
`kernel void` of the reference's shaders (written by tests/golden/make_kernel_names.py); the library's own
name table is asked, without a GPU, through smelt_cuda_pipeline_supported.  The shader files of the decode
path must be covered completely or up to the exceptions spelled out here, so that a change that drops a name
fails, and a package that names a kernel outside this list fails when it is opened, not in the middle of a token."""
import collections
import ctypes as C
import os

from smelt_b200 import capi

HERE = os.path.dirname(os.path.abspath(__file__))

# file -> the names NOT bound (everything else in the file must be)
EXPECTED_GAPS = {
    "signed_quant.metal": set(),
    "activations.metal": set(),
    "activations_precise.metal": set(),
    "attention_fused.metal": set(),
    "norms_gated_precise.metal": set(),
    "norms.metal": set(),
    "conv1d.metal": set(),
    "prefill_recurrence.metal": set(),
    "recurrence.metal": set(),
    "signed_quant_precise.metal": set(),
}


def supported_by_file():
    lib = C.CDLL(capi.LIB_PATH)
    lib.smelt_cuda_pipeline_supported.argtypes = [C.c_char_p]
    lib.smelt_cuda_pipeline_supported.restype = C.c_int
    by = collections.defaultdict(dict)
    for line in open(os.path.join(HERE, "golden", "kernel_names.txt")):
        f, name = line.split()
        by[f][name] = bool(lib.smelt_cuda_pipeline_supported(name.encode()))
    return by


def test_decode_path_shaders_are_bound_by_name():
    by = supported_by_file()
    for f, gaps in EXPECTED_GAPS.items():
        missing = {n for n, ok in by[f].items() if not ok}
        assert missing == gaps, (f, sorted(missing ^ gaps))


def test_affine_and_attention_families_do_not_shrink():
    by = supported_by_file()
    families = ("affine_matvec", "fused_affine_matvec_add", "fused_affine_gate_up_swiglu", "fused_dual_affine_matvec", "affine_embedding_gather")
    affine = [n for n in by["lut_matvec.metal"] if n.startswith(families) and "argmax" not in n and not n.endswith("_reference")]
    bound = [n for n in affine if by["lut_matvec.metal"][n]]
    assert len(bound) == len(affine), sorted(set(affine) - set(bound))
    assert sum(by["attention.metal"].values()) >= 16
    assert sum(sum(d.values()) for d in by.values()) >= 376


def test_committed_token_fixtures_describe_the_current_full_model():
    """bench.py and the full-model GPU test replay tests/golden/full_model_tokens*.json only when the fixture's
    configuration equals the model's own description: a new configuration field must not silently switch that off."""
    import json

    from smelt_b200 import package
    for name in ("full_model_tokens.json", "full_model_tokens_batch8.json"):
        with open(os.path.join(HERE, "golden", name)) as f:
            gold = json.load(f)
        assert gold["config"] == package.FULL_MODEL.as_dict(), name

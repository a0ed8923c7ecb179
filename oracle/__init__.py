"""ctypes front end of the CPU oracle (``smelt_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the CPU-baseline
and reference legs of ``bench.py``; never by the ``smelt_b200`` package.  Every function takes
and returns numpy arrays; fp16 data travels as ``np.float16`` (viewed as uint16 at the ABI).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsmelt_oracle.so")


def build(force: bool = False) -> str:
    """Compile ``smelt_oracle.c`` into ``libsmelt_oracle.so`` (gcc, OpenMP, no FMA contraction)."""
    src = os.path.join(_HERE, "smelt_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.so_model_create.restype = C.c_void_p
        _lib.so_argmax_f16.restype = C.c_int32
    return _lib


class OracleError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"oracle {what} failed with code {code}")
        self.code = code


GEOMETRY, INVALID_CODE = -1, -2
BINARY1, TERNARY2 = 1, 2


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _h(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8, a.dtype
    return a


def _check(rc: int, what: str):
    if rc != 0:
        raise OracleError(rc, what)


def num_threads() -> int:
    return lib().so_num_threads()


def set_num_threads(n: int) -> None:
    lib().so_set_num_threads(int(n))


# ── affine u4 ────────────────────────────────────────────────────────────────
def affine_quantize(values: np.ndarray, group: int):
    values = np.ascontiguousarray(values, dtype=np.float32)
    rows, cols = values.shape
    groups = (cols + group - 1) // group
    packed = np.zeros((rows, (cols + 1) // 2), np.uint8)
    scales = np.zeros((rows, groups), np.float16)
    biases = np.zeros((rows, groups), np.float16)
    for r in range(rows):
        _check(lib().so_affine_u4_quantize_row(_p(values[r]), cols, group, _p(packed[r]), _p(scales[r]), _p(biases[r])),
               "affine_u4_quantize_row")
    return packed, scales, biases


def affine_dequantize(packed, scales, biases, cols: int, group: int) -> np.ndarray:
    packed, scales, biases = _u8(packed), _h(scales), _h(biases)
    rows = packed.shape[0]
    out = np.zeros((rows, cols), np.float32)
    for r in range(rows):
        _check(lib().so_affine_u4_dequantize_row(_p(packed[r]), _p(scales[r]), _p(biases[r]), cols, group, _p(out[r])),
               "affine_u4_dequantize_row")
    return out


def affine_dequantize_f16(packed, scales, biases, rows: int, cols: int, group: int) -> np.ndarray:
    out = np.zeros((rows, cols), np.float16)
    _check(lib().so_affine_u4_dequantize_rows_f16(_p(_u8(packed)), _p(_h(scales)), _p(_h(biases)), rows, cols, group, _p(out)),
           "affine_u4_dequantize_rows_f16")
    return out


def _xb(x, cols):
    x = _h(x)
    x2 = x.reshape(-1, cols)
    return x2, x2.shape[0]


def affine_matvec(w, s, b, x, rows: int, cols: int, group: int, f32: bool = False) -> np.ndarray:
    x2, batch = _xb(x, cols)
    y = np.zeros((batch, rows), np.float32 if f32 else np.float16)
    fn = lib().so_affine_matvec_f32 if f32 else lib().so_affine_matvec
    _check(fn(_p(_u8(w)), _p(_h(s)), _p(_h(b)), _p(x2), rows, cols, group, batch, _p(y)), "affine_matvec")
    return y


def affine_matvec_add(w, s, b, x, residual, rows, cols, group) -> np.ndarray:
    x2, batch = _xb(x, cols)
    y = np.zeros((batch, rows), np.float16)
    _check(lib().so_affine_matvec_add(_p(_u8(w)), _p(_h(s)), _p(_h(b)), _p(x2), _p(_h(residual)), rows, cols, group, batch, _p(y)),
           "affine_matvec_add")
    return y


def affine_gate_up_swiglu(gw, gs, gb, uw, us, ub, x, rows, cols, group, round_gate_up: bool = False) -> np.ndarray:
    x2, batch = _xb(x, cols)
    y = np.zeros((batch, rows), np.float16)
    _check(lib().so_affine_gate_up_swiglu(_p(_u8(gw)), _p(_h(gs)), _p(_h(gb)), _p(_u8(uw)), _p(_h(us)), _p(_h(ub)), _p(x2),
                                          rows, cols, group, batch, int(round_gate_up), _p(y)), "affine_gate_up_swiglu")
    return y


def fp16_matvec(w, x, rows, cols) -> np.ndarray:
    x2, batch = _xb(x, cols)
    y = np.zeros((batch, rows), np.float16)
    _check(lib().so_fp16_matvec(_p(_h(w)), _p(x2), rows, cols, batch, _p(y)), "fp16_matvec")
    return y


# ── binary / ternary ─────────────────────────────────────────────────────────
def signed_packed_byte_count(n: int, fmt: int) -> int:
    out = C.c_int64()
    _check(lib().so_signed_packed_byte_count(C.c_int64(n), fmt, C.byref(out)), "signed_packed_byte_count")
    return out.value


def signed_groups_per_row(padded_cols: int, group: int) -> int:
    out = C.c_int()
    _check(lib().so_signed_groups_per_row(padded_cols, group, C.byref(out)), "signed_groups_per_row")
    return out.value


def signed_validate_codes(codes, logical_count: int, fmt: int):
    codes = _u8(codes)
    bad = C.c_int64(-1)
    rc = lib().so_signed_validate_codes(_p(codes), C.c_int64(codes.size), C.c_int64(logical_count), fmt, C.byref(bad))
    return rc, bad.value


def signed_dequantize_row(fmt, codes, scales, cols, padded_cols, group) -> np.ndarray:
    codes, scales = _u8(codes), _h(scales)
    out = np.zeros(cols, np.float32)
    _check(lib().so_signed_dequantize_row(fmt, _p(codes), C.c_int64(codes.size), _p(scales), C.c_int64(scales.size * 2),
                                          cols, padded_cols, group, _p(out)), "signed_dequantize_row")
    return out


def signed_matvec(fmt, codes, scales, x, rows, cols, group=128, f32: bool = False) -> np.ndarray:
    x2, batch = _xb(x, cols)
    y = np.zeros((batch, rows), np.float32 if f32 else np.float16)
    fn = lib().so_signed_matvec_f32 if f32 else lib().so_signed_matvec
    _check(fn(fmt, _p(_u8(codes)), _p(_h(scales)), _p(x2), rows, cols, group, batch, _p(y)), "signed_matvec")
    return y


def signed_matvec_add(fmt, codes, scales, x, residual, rows, cols, group=128) -> np.ndarray:
    x2, batch = _xb(x, cols)
    y = np.zeros((batch, rows), np.float16)
    _check(lib().so_signed_matvec_add(fmt, _p(_u8(codes)), _p(_h(scales)), _p(x2), _p(_h(residual)), rows, cols, group, batch, _p(y)),
           "signed_matvec_add")
    return y


def signed_gate_up_swiglu(fmt, gc, gs, uc, us, x, rows, cols, group=128, staged: bool = True) -> np.ndarray:
    x2, batch = _xb(x, cols)
    y = np.zeros((batch, rows), np.float16)
    _check(lib().so_signed_gate_up_swiglu(fmt, _p(_u8(gc)), _p(_h(gs)), _p(_u8(uc)), _p(_h(us)), _p(x2), rows, cols, group,
                                          batch, int(staged), _p(y)), "signed_gate_up_swiglu")
    return y


def swiglu_staged(gate, up) -> np.ndarray:
    gate, up = _h(gate), _h(up)
    y = np.zeros(gate.shape, np.float16)
    lib().so_swiglu_staged(_p(gate), _p(up), C.c_int64(gate.size), _p(y))
    return y


# ── glue ─────────────────────────────────────────────────────────────────────
def rms_norm_1pw(x, w, eps: float, two_stage: bool = True) -> np.ndarray:
    x, w = _h(x), _h(w)
    y = np.zeros(x.shape, np.float16)
    _check(lib().so_rms_norm_1pw(_p(x), _p(w), x.size, C.c_float(eps), int(two_stage), _p(y)), "rms_norm_1pw")
    return y


HEAD_NORM_DIRECT, HEAD_NORM_1PW, HEAD_NORM_NOSCALE = 0, 1, 2
EW_SILU, EW_SIGMOID, EW_SOFTPLUS, EW_COPY, EW_SCALAR_MUL, EW_LOGIT_CAP, EW_MUL, EW_SIGMOID_MUL, EW_GEGLU, EW_BIAS_ADD = range(10)


def head_norm(mode: int, x, w, heads: int, head_dim: int, eps: float, tgs: int = 32) -> np.ndarray:
    """The per-head norms of attention_fused.metal with their reduction topologies (w unused for HEAD_NORM_NOSCALE)."""
    y = np.zeros((heads, head_dim), np.float16)
    wv = _h(w) if w is not None else np.zeros(head_dim, np.float16)
    _check(lib().so_head_norm(mode, _p(_h(x)), _p(wv), heads, head_dim, C.c_float(eps), tgs, _p(y)), "head_norm")
    return y


def row_norm(x, w=None, *, topology: int, value: int, tgs: int = 256, eps: float = 1e-6, scale: int = 0, pre=None, residual=None, scalar=None):
    """The row norms of norms.metal with their reduction topologies (see so_row_norm).  Returns (y or None, scales [rows])."""
    x = _h(x)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    rows, dim = x2.shape
    y = np.zeros_like(x2) if (value or pre is not None) else None
    sc = np.zeros(rows, np.float32)
    opt = lambda a: _p(_h(a)) if a is not None else None
    _check(lib().so_row_norm(_p(x2), opt(pre), opt(w), opt(residual), opt(scalar), _p(y) if y is not None else None, _p(sc), rows, dim, C.c_float(eps),
                             topology, tgs, value, scale), "row_norm")
    return (y.reshape(x.shape) if y is not None else None), sc


def gate_split(x, heads: int, head_dim: int):
    q, g = np.zeros((heads, head_dim), np.float16), np.zeros((heads, head_dim), np.float16)
    lib().so_gate_split(_p(_h(x)), heads, head_dim, _p(q), _p(g))
    return q, g


def elementwise(op: int, a, b=None, scalar: float = 0.0, b_stride: int = 0) -> np.ndarray:
    """a [batch, count] (or [count]); b per op (see so_elementwise)."""
    a = _h(a)
    a2 = a.reshape(1, -1) if a.ndim == 1 else a
    y = np.zeros_like(a2)
    _check(lib().so_elementwise(op, _p(a2), _p(_h(b)) if b is not None else None, _p(y), a2.shape[1], a2.shape[0], b_stride or a2.shape[1], C.c_float(scalar)),
           "elementwise")
    return y.reshape(a.shape)


def per_head_rms_norm(x, w, heads, head_dim, eps) -> np.ndarray:
    x, w = _h(x), _h(w)
    y = np.zeros(x.shape, np.float16)
    _check(lib().so_per_head_rms_norm(_p(x), _p(w), heads, head_dim, C.c_float(eps), _p(y)), "per_head_rms_norm")
    return y


def elementwise_add(a, b) -> np.ndarray:
    a, b = _h(a), _h(b)
    y = np.zeros(a.shape, np.float16)
    lib().so_elementwise_add(_p(a), _p(b), C.c_int64(a.size), _p(y))
    return y


def argmax_f16(logits) -> int:
    logits = _h(logits)
    return int(lib().so_argmax_f16(_p(logits), C.c_int64(logits.size)))


def apply_rope(qk, head_dim, rope_dim, heads, layout, position, base_log2=0.0, math_mode=1, cos=None, sin=None) -> np.ndarray:
    out = _h(qk).copy()
    cp = _p(_h(cos)) if cos is not None else None
    sp = _p(_h(sin)) if sin is not None else None
    _check(lib().so_apply_rope(_p(out), cp, sp, head_dim, rope_dim, heads, layout, C.c_uint32(position), C.c_float(base_log2),
                               math_mode), "apply_rope")
    return out


def kv_cache_update(cache, new_kv, capacity, head_dim, pos, heads) -> np.ndarray:
    out = _h(cache).copy()
    _check(lib().so_kv_cache_update(_p(out), _p(_h(new_kv)), capacity, head_dim, pos, heads), "kv_cache_update")
    return out


def rope_kv_cache_update(cache, new_kv, capacity, head_dim, pos, heads, rope_dim, layout, base_log2=0.0, math_mode=1,
                         cos=None, sin=None) -> np.ndarray:
    out = _h(cache).copy()
    cp = _p(_h(cos)) if cos is not None else None
    sp = _p(_h(sin)) if sin is not None else None
    _check(lib().so_rope_kv_cache_update(_p(out), _p(_h(new_kv)), cp, sp, capacity, head_dim, pos, heads, rope_dim, layout,
                                         C.c_float(base_log2), math_mode), "rope_kv_cache_update")
    return out


def attention_decode(q, k_cache, v_cache, n_q, n_kv, head_dim, capacity, seq_len, scale=None, sliding_window=0) -> np.ndarray:
    q, k_cache, v_cache = _h(q), _h(k_cache), _h(v_cache)
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(head_dim))
    out = np.zeros((n_q, head_dim), np.float16)
    _check(lib().so_attention_decode(_p(q), _p(k_cache), _p(v_cache), n_q, n_kv, head_dim, capacity, seq_len,
                                     C.c_float(scale), sliding_window, _p(out)), "attention_decode")
    return out


def attention_decode_mlx_2pass(q, k_cache, v_cache, n_q, n_kv, capacity, seq_len) -> np.ndarray:
    """The reference's D256 split-K record pair (interleaved key blocks, fp16 partials)."""
    q, k_cache, v_cache = _h(q), _h(k_cache), _h(v_cache)
    partials = np.zeros((n_q, 128, 256), np.float16)
    stats = np.zeros((2, n_q, 128), np.float32)
    out = np.zeros((n_q, 256), np.float16)
    _check(lib().so_attention_decode_mlx_2pass(_p(q), _p(k_cache), _p(v_cache), n_q, n_kv, capacity, seq_len, _p(partials), _p(stats),
                                               _p(out)), "attention_decode_mlx_2pass")
    return out


# ── whole decoder ────────────────────────────────────────────────────────────
class Model:
    """Greedy decoder over packed weights held in numpy arrays (kept alive by this object)."""

    WHICH = {"q": 0, "k": 1, "v": 2, "o": 3, "gate": 4, "up": 5, "down": 6}

    def __init__(self, cfg: dict, capacity: int):
        self.cfg = dict(cfg)
        self.capacity = capacity
        self._keep = []
        self._m = C.c_void_p(lib().so_model_create(
            cfg["layers"], cfg["hidden"], cfg["inter"], cfg["n_q"], cfg["n_kv"], cfg["head_dim"], cfg["vocab"],
            cfg.get("group", 64), capacity, C.c_float(cfg.get("eps", 1e-6)), C.c_float(cfg.get("rope_theta", 1e6))))
        if not self._m:
            raise MemoryError("so_model_create")

    def close(self):
        if self._m:
            lib().so_model_destroy(self._m)
            self._m = None

    def __del__(self):
        self.close()

    def set_globals(self, embedding, lm_head, final_norm):
        arrs = [_h(embedding), _h(lm_head), _h(final_norm)]
        self._keep += arrs
        lib().so_model_set_globals(self._m, *[_p(a) for a in arrs])

    def set_layer(self, layer: int, tensors: dict, input_norm, post_norm):
        for name, idx in self.WHICH.items():
            w, s, b = tensors[name]
            arrs = [_u8(w), _h(s), _h(b)]
            self._keep += arrs
            _check(lib().so_model_set_affine(self._m, layer, idx, *[_p(a) for a in arrs]), "model_set_affine")
        arrs = [_h(input_norm), _h(post_norm)]
        self._keep += arrs
        _check(lib().so_model_set_norms(self._m, layer, *[_p(a) for a in arrs]), "model_set_norms")

    DELTA_WHICH = {"dqkv": 0, "dz": 1, "da": 2, "db": 3, "dout": 4}

    def set_delta_geometry(self, value_heads: int, qk_heads: int, head_dim: int, conv_kernel: int):
        _check(lib().so_model_set_delta_geometry(self._m, value_heads, qk_heads, head_dim, conv_kernel), "model_set_delta_geometry")

    def set_delta_layer(self, layer: int, tensors: dict, conv_w, a_log, dt_bias, norm_w):
        """Turns `layer` into a DeltaNet layer: its five projections (dqkv, dz, da, db, dout) and four small tensors."""
        for name, idx in self.DELTA_WHICH.items():
            w, s, b = tensors[name]
            arrs = [_u8(w), _h(s), _h(b)]
            self._keep += arrs
            _check(lib().so_model_set_delta_affine(self._m, layer, idx, *[_p(a) for a in arrs]), "model_set_delta_affine")
        arrs = [_h(conv_w), _h(a_log), _h(dt_bias), _h(norm_w)]
        self._keep += arrs
        _check(lib().so_model_set_delta_params(self._m, layer, *[_p(a) for a in arrs]), "model_set_delta_params")

    def reset(self):
        lib().so_model_reset_cache(self._m)

    def fill_kv(self, layer: int, k, v):
        """Load positions [0, n) of one layer's caches from [n_kv, n, head_dim] fp16 arrays."""
        k, v = _h(k), _h(v)
        _check(lib().so_model_fill_kv(self._m, layer, _p(k), _p(v), k.shape[1]), "model_fill_kv")

    def decode_step(self, token: int, position: int, want_logits: bool = False):
        logits = np.zeros(self.cfg["vocab"], np.float16) if want_logits else None
        out = C.c_int32(-1)
        _check(lib().so_model_decode_step(self._m, C.c_int32(token), position, _p(logits) if want_logits else None,
                                          C.byref(out)), "model_decode_step")
        return (out.value, logits) if want_logits else out.value

    def prefill(self, tokens, start_pos: int = 0, chunk: int = 512, want_logits: bool = False):
        """The prompt `chunk` positions at a time, layer by layer over each chunk (so_model_prefill).  Returns the
        greedy token after the last position (and its logits)."""
        toks = np.ascontiguousarray(np.asarray(tokens).reshape(-1), np.int32)
        logits = np.zeros(self.cfg["vocab"], np.float16) if want_logits else None
        out = C.c_int32(-1)
        _check(lib().so_model_prefill(self._m, _p(toks), len(toks), int(start_pos), int(chunk), _p(logits) if want_logits else None, C.byref(out)),
               "model_prefill")
        return (out.value, logits) if want_logits else out.value

    def greedy_top2(self, prompt, n_decode: int):
        """Greedy decode of one sequence from an empty cache; per step the token, the runner-up
        and the logit margin between the two (lists of n_decode entries).  A teacher-forced replay
        of these tokens can then tell a tie that any fp32 summation order may break from a
        wrong token."""
        self.reset()
        logits = None
        for i, t in enumerate(prompt):
            last = i + 1 == len(prompt)
            r = self.decode_step(int(t), i, want_logits=last)
            if last:
                logits = r[1]
        toks, second, margin = [], [], []
        pos = len(prompt)
        for i in range(n_decode):
            a, b, m = top2(logits)
            toks.append(a); second.append(b); margin.append(m)
            if i + 1 < n_decode:
                _, logits = self.decode_step(a, pos, want_logits=True)
                pos += 1
        return toks, second, margin

    def generate(self, prompt, n_decode: int):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        toks = np.zeros(n_decode, np.int32)
        margins = np.zeros(n_decode, np.float32)
        _check(lib().so_model_generate(self._m, _p(prompt), prompt.size, n_decode, _p(toks), _p(margins)), "model_generate")
        return toks, margins


def model_from_package(pkg, capacity: int) -> Model:
    """The decoder above over the tensors of a synthetic package (any object with ``cfg``,
    ``tensors``, ``layer_tensor``, ``norm_delta``, ``embedding`` and ``lm_head``, such as
    ``smelt_b200.package.SyntheticPackage``).  Lives here so that the product package holds no
    oracle adapter."""
    c = pkg.cfg
    m = Model(c.as_dict(), capacity)
    emb, head, fin = pkg.tensors.get("globals") or (pkg.embedding(), pkg.lm_head(), pkg.norm_delta("final_norm"))
    m.set_globals(emb, head, fin)
    delta_layers = tuple(getattr(c, "delta_layers", ()) or ())
    if delta_layers:
        m.set_delta_geometry(c.delta_value_heads, c.delta_qk_heads, c.delta_head_dim, c.conv_kernel)
    for l in range(c.layers):
        t = {name: pkg.tensors.get((l, name)) or pkg.layer_tensor(l, name) for name in Model.WHICH}
        norms = pkg.tensors.get((l, "norms")) or (pkg.norm_delta(f"layer{l}.input_norm"), pkg.norm_delta(f"layer{l}.post_norm"))
        m.set_layer(l, t, *norms)
        if l in delta_layers:
            dt = {name: pkg.tensors.get((l, name)) or pkg.delta_tensor(l, name) for name in Model.DELTA_WHICH}
            small = pkg.tensors.get((l, "delta_small")) or pkg.delta_small(l)
            m.set_delta_layer(l, dt, *small)
    return m


def top2(logits) -> tuple[int, int, float]:
    """(best id, runner-up id, margin) of fp16 logits under the argmax ordering: larger value
    first, lower index on ties, -0 == +0."""
    v = np.asarray(logits, np.float32)
    best = int(np.argmax(v))
    w = v.copy()
    w[best] = -np.inf
    second = int(np.argmax(w))
    return best, second, float(v[best] - v[second])


# ── DeltaNet decode step (conv1d.metal, norms.metal, recurrence.metal) ──
def conv1d_update_silu(state, new_val, weight, channels: int, kernel_size: int):
    """Returns (state after the shift, activated output)."""
    st = _h(state).copy()
    out = np.zeros(channels, np.float16)
    _check(lib().so_conv1d_update_silu(_p(st), _p(_h(new_val)), _p(_h(weight)), _p(out), channels, kernel_size), "conv1d_update_silu")
    return st, out


def rms_scale_qk(qkv, head_dim: int, eps: float, qkv_dim: int, qk_heads: int, batch: int = 1) -> np.ndarray:
    out = _h(qkv).copy()
    _check(lib().so_rms_scale_qk(_p(out), head_dim, C.c_float(eps), qkv_dim, qk_heads, batch), "rms_scale_qk")
    return out


def deltanet_recurrence_decode(state, qkv, b_proj, a_proj, a_log, dt_bias, head_dim: int, value_heads: int, qk_heads: int):
    """Returns (state after the step, output [value_heads, head_dim])."""
    st = _h(state).copy()
    out = np.zeros((value_heads, head_dim), np.float16)
    _check(lib().so_deltanet_recurrence_decode(_p(st), _p(_h(qkv)), _p(_h(b_proj)), _p(_h(a_proj)), _p(_h(a_log)), _p(_h(dt_bias)), _p(out),
                                               head_dim, value_heads, qk_heads), "deltanet_recurrence_decode")
    return st, out


def conv1d_update_silu_prefill(state, qkv, weight, seq_len: int, channels: int, kernel_size: int, history: bool = False):
    """Returns (state after the chunk, activated qkv [seq_len, channels], history [seq_len + 1, channels, kernel_size] or None)."""
    st = _h(state).copy()
    x = _h(qkv).copy()
    hist = np.zeros((seq_len + 1, channels, kernel_size), np.float16) if history else None
    _check(lib().so_conv1d_update_silu_prefill(_p(st), _p(x), _p(_h(weight)), seq_len, channels, kernel_size, _p(hist) if history else None),
           "conv1d_update_silu_prefill")
    return st, x.reshape(seq_len, channels), hist


def deltanet_recurrence_prefill(state, qkv, b_proj, a_proj, a_log, dt_bias, head_dim: int, value_heads: int, qk_heads: int, seq_len: int,
                                history: bool = False):
    """Returns (state after the chunk, output [seq_len, value_heads, head_dim], history
    [seq_len + 1, value_heads, head_dim, head_dim] or None)."""
    st = _h(state).copy()
    out = np.zeros((seq_len, value_heads, head_dim), np.float16)
    hist = np.zeros((seq_len + 1, value_heads, head_dim, head_dim), np.float16) if history else None
    _check(lib().so_deltanet_recurrence_prefill(_p(st), _p(_h(qkv)), _p(_h(b_proj)), _p(_h(a_proj)), _p(_h(a_log)), _p(_h(dt_bias)), _p(out),
                                                head_dim, value_heads, qk_heads, seq_len, _p(hist) if history else None),
           "deltanet_recurrence_prefill")
    return st, out, hist


def dn_compute_gates(b_proj, a_proj, a_log, dt_bias, heads: int):
    """compute_gates: (beta [heads], g [heads]) as fp16."""
    beta, g = np.zeros(heads, np.float16), np.zeros(heads, np.float16)
    _check(lib().so_dn_compute_gates(_p(_h(b_proj)), _p(_h(a_proj)), _p(_h(a_log)), _p(_h(dt_bias)), _p(beta), _p(g), heads), "dn_compute_gates")
    return beta, g


def dn_state_decay(state, g_val, head_dim: int, heads: int) -> np.ndarray:
    st = _h(state).copy()
    _check(lib().so_dn_state_decay(_p(st), _p(_h(g_val)), head_dim, heads), "dn_state_decay")
    return st


def dn_kv_mem_readout(state, key, head_dim: int, heads: int) -> np.ndarray:
    out = np.zeros((heads, head_dim), np.float32)
    _check(lib().so_dn_kv_mem_readout(_p(_h(state)), _p(_h(key)), _p(out), head_dim, heads), "dn_kv_mem_readout")
    return out


def dn_compute_delta(value, kv_mem, beta, head_dim: int, heads: int) -> np.ndarray:
    out = np.zeros((heads, head_dim), np.float32)
    _check(lib().so_dn_compute_delta(_p(_h(value)), _p(np.ascontiguousarray(kv_mem, np.float32)), _p(_h(beta)), _p(out), head_dim, heads), "dn_compute_delta")
    return out


def dn_outer_product_update(state, key, delta, head_dim: int, heads: int, g_val=None) -> np.ndarray:
    """outer_product_update, or state_decay_update when g_val is given."""
    st = _h(state).copy()
    _check(lib().so_dn_outer_product_update(_p(st), _p(_h(g_val)) if g_val is not None else None, _p(_h(key)),
                                            _p(np.ascontiguousarray(delta, np.float32)), head_dim, heads), "dn_outer_product_update")
    return st


def dn_kv_readout_delta(state, key, value, g_val, beta, head_dim: int, heads: int) -> np.ndarray:
    out = np.zeros((heads, head_dim), np.float32)
    _check(lib().so_dn_kv_readout_delta(_p(_h(state)), _p(_h(key)), _p(_h(value)), _p(_h(g_val)), _p(_h(beta)), None, None, None, None,
                                        _p(out), None, head_dim, heads), "dn_kv_readout_delta")
    return out


def dn_gates_kv_readout_delta(state, key, value, b_proj, a_proj, a_log, dt_bias, head_dim: int, heads: int):
    """Returns (delta [heads, head_dim] fp32, g [heads] fp16)."""
    out, g = np.zeros((heads, head_dim), np.float32), np.zeros(heads, np.float16)
    _check(lib().so_dn_kv_readout_delta(_p(_h(state)), _p(_h(key)), _p(_h(value)), None, None, _p(_h(b_proj)), _p(_h(a_proj)), _p(_h(a_log)),
                                        _p(_h(dt_bias)), _p(out), _p(g), head_dim, heads), "dn_gates_kv_readout_delta")
    return out, g


def dn_query_readout(state, query, head_dim: int, scale: float, heads: int) -> np.ndarray:
    out = np.zeros((heads, head_dim), np.float16)
    _check(lib().so_dn_query_readout(_p(_h(state)), _p(_h(query)), _p(out), head_dim, C.c_float(scale), heads), "dn_query_readout")
    return out


def deltanet_recurrence_fused(state, qkv, b_proj, a_proj, a_log, dt_bias, conv_state, conv_weight, z_proj, norm_weight, head_dim: int,
                              head_scale: float, qkv_dim: int, conv_k: int, heads: int, rms_eps: float, tgs: int = 256):
    """deltanet_recurrence_fused: returns (state, conv state, out [heads, head_dim])."""
    st, cs = _h(state).copy(), _h(conv_state).copy()
    out = np.zeros((heads, head_dim), np.float16)
    _check(lib().so_deltanet_recurrence_fused(_p(st), _p(_h(qkv)), _p(_h(b_proj)), _p(_h(a_proj)), _p(_h(a_log)), _p(_h(dt_bias)), _p(out), _p(cs),
                                              _p(_h(conv_weight)), _p(_h(z_proj)), _p(_h(norm_weight)), head_dim, C.c_float(head_scale), qkv_dim,
                                              conv_k, heads, C.c_float(rms_eps), tgs), "deltanet_recurrence_fused")
    return st, cs, out


def deltanet_recurrence_prefill_fused(state, conv_state, qkv, conv_weight, a_log, dt_bias, b_buf, a_buf, head_dim: int, heads: int, seq_len: int,
                                      qkv_dim: int, conv_k: int, head_scale: float, l2_eps: float, tgs: int = 0):
    """deltanet_recurrence_prefill (the fused per-head kernel): returns (state, conv state, qkv after conv and
    norms [seq_len, qkv_dim], out [seq_len, heads, head_dim])."""
    st, cs, x = _h(state).copy(), _h(conv_state).copy(), _h(qkv).copy()
    out = np.zeros((seq_len, heads, head_dim), np.float16)
    _check(lib().so_deltanet_recurrence_prefill_fused(_p(st), _p(cs), _p(x), _p(_h(conv_weight)), _p(_h(a_log)), _p(_h(dt_bias)), _p(_h(b_buf)),
                                                      _p(_h(a_buf)), _p(out), head_dim, heads, seq_len, qkv_dim, conv_k, C.c_float(head_scale),
                                                      C.c_float(l2_eps), tgs or max(32, (head_dim + 31) // 32 * 32)), "deltanet_recurrence_prefill_fused")
    return st, cs, x.reshape(seq_len, qkv_dim), out


def rms_norm_gated(x, gate, weight, head_dim: int, eps: float, heads: int) -> np.ndarray:
    out = np.zeros((heads, head_dim), np.float16)
    _check(lib().so_rms_norm_gated(_p(_h(x)), _p(_h(gate)), _p(_h(weight)), _p(out), head_dim, C.c_float(eps), heads), "rms_norm_gated")
    return out


def rms_norm_gated_tg(x, gate, weight, head_dim: int, eps: float, heads: int, tgs: int) -> np.ndarray:
    """rms_norm_gated as a threadgroup of `tgs` threads sums it."""
    out = np.zeros((heads, head_dim), np.float16)
    _check(lib().so_rms_norm_gated_tg(_p(_h(x)), _p(_h(gate)), _p(_h(weight)), _p(out), head_dim, C.c_float(eps), heads, tgs), "rms_norm_gated_tg")
    return out


def rms_norm_gated_d128(x, gate, weight, heads: int) -> np.ndarray:
    out = np.zeros((heads, 128), np.float16)
    _check(lib().so_rms_norm_gated_d128(_p(_h(x)), _p(_h(gate)), _p(_h(weight)), _p(out), heads), "rms_norm_gated_d128")
    return out


def signed_embedding_gather(fmt: int, codes, scales, token_ids, hidden: int) -> np.ndarray:
    ids = np.ascontiguousarray(token_ids, np.int32)
    out = np.zeros((len(ids), hidden), np.float16)
    _check(lib().so_signed_embedding_gather(fmt, _p(_u8(codes)), _p(_h(scales)), _p(ids), _p(out), hidden, len(ids)), "signed_embedding_gather")
    return out


# ── signed activation bit-planes (signed_quant.metal:751-2101) ──
def signed_activation_bitplanes(x, cols: int, planes: int):
    """Returns (planes uint32 [groups, planes, 4], scales fp16 [groups])."""
    groups = cols // 128
    out = np.zeros((groups, planes, 4), np.uint32)
    sc = np.zeros(groups, np.float16)
    _check(lib().so_signed_activation_bitplanes(_p(_h(x)), cols, planes, _p(out), _p(sc)), "signed_activation_bitplanes")
    return out, sc


def swiglu_signed_activation_bitplanes_i5(gate, up, cols: int):
    groups = cols // 128
    out = np.zeros((groups, 5, 4), np.uint32)
    sc = np.zeros(groups, np.float16)
    _check(lib().so_swiglu_signed_activation_bitplanes_i5(_p(_h(gate)), _p(_h(up)), cols, _p(out), _p(sc)), "swiglu_signed_activation_bitplanes_i5")
    return out, sc


def sigmoid_mul_signed_activation_bitplanes_i6(a, b, cols: int):
    groups = cols // 128
    out, sc = np.zeros((groups, 6, 4), np.uint32), np.zeros(groups, np.float16)
    _check(lib().so_sigmoid_mul_signed_activation_bitplanes_i6(_p(_h(a)), _p(_h(b)), cols, _p(out), _p(sc)), "sigmoid_mul_signed_activation_bitplanes_i6")
    return out, sc


def norm_scale_signed_activation_bitplanes(norm_scale: float, x, norm_weight, cols: int, planes: int):
    groups = cols // 128
    out, sc = np.zeros((groups, planes, 4), np.uint32), np.zeros(groups, np.float16)
    rs = np.array([norm_scale], np.float32)
    _check(lib().so_norm_scale_signed_activation_bitplanes(_p(rs), _p(_h(x)), _p(_h(norm_weight)), cols, planes, _p(out), _p(sc)),
           "norm_scale_signed_activation_bitplanes")
    return out, sc


def rms_norm_gated_d128_signed_activation_bitplanes_i6(x, gate, weight, heads: int, eps: float, tgs: int):
    out, sc = np.zeros((heads, 6, 4), np.uint32), np.zeros(heads, np.float16)
    _check(lib().so_rms_norm_gated_d128_signed_activation_bitplanes_i6(_p(_h(x)), _p(_h(gate)), _p(_h(weight)), heads, C.c_float(eps), tgs, _p(out), _p(sc)),
           "rms_norm_gated_d128_signed_activation_bitplanes_i6")
    return out, sc


def signed_bitplane_matvec(fmt: int, codes, weight_scales, planes_arr, act_scales, rows: int, cols: int, planes: int, residual=None) -> np.ndarray:
    out = np.zeros(rows, np.float16)
    pl = np.ascontiguousarray(planes_arr, dtype=np.uint32)
    _check(lib().so_signed_bitplane_matvec(fmt, _p(_u8(codes)), _p(_h(weight_scales)), _p(pl), _p(_h(act_scales)),
                                           _p(_h(residual)) if residual is not None else None, rows, cols, planes, _p(out)), "signed_bitplane_matvec")
    return out


def signed_bitplane_gate_up_swiglu(fmt: int, gc, gs, uc, us, planes_arr, act_scales, rows: int, cols: int, planes: int) -> np.ndarray:
    out = np.zeros(rows, np.float16)
    pl = np.ascontiguousarray(planes_arr, dtype=np.uint32)
    _check(lib().so_signed_bitplane_gate_up_swiglu(fmt, _p(_u8(gc)), _p(_h(gs)), _p(_u8(uc)), _p(_h(us)), _p(pl), _p(_h(act_scales)), rows, cols, planes,
                                                   _p(out)), "signed_bitplane_gate_up_swiglu")
    return out

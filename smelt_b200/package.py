"""Host-side mirror of the pieces of a ``.smeltpkg`` the decode path touches: the ``weights.bin``
image layout, a synthetic decoder package, and a ``Decoder`` that drives ``libsmelt_cuda``
through dispatch records the way ``SmeltRuntime.decodeStep`` does.

Tensor placement follows the reference packer: each tensor starts 128-byte aligned and is laid
out ``[packed] -> align128 -> [scales] -> align128 -> [biases]``
(Sources/SmeltCompiler/SmeltWeightPacker.swift:807-810); norm weights are stored as ``w - 1``
because the text path always runs ``rms_norm_1pw`` (Sources/SmeltCompiler/SmeltCompiler.swift:1974-2005).
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass, field

import numpy as np

from . import capi, synth

WEIGHTS_SLOT = 30  # SmeltFixedSlot.weights (Sources/SmeltCompiler/SmeltBufferPlan.swift:129-198)
LOGITS_SLOT, ARGMAX_SLOT = 16, 17
KV_BASE_SLOT = 40


def align128(n: int) -> int:
    return (n + 127) & ~127


class WeightsImage:
    """An in-memory ``weights.bin``."""

    def __init__(self):
        self.chunks: list[tuple[int, np.ndarray]] = []
        self.size = 0

    def _put(self, arr: np.ndarray) -> int:
        arr = np.ascontiguousarray(arr)
        off = align128(self.size)
        self.chunks.append((off, arr.view(np.uint8).reshape(-1)))
        self.size = off + arr.nbytes
        return off

    def add_affine(self, packed, scales, biases) -> capi.AffineRef:
        return capi.AffineRef(self._put(packed), self._put(scales), self._put(biases))

    def add(self, arr) -> int:
        return self._put(arr)

    def tobytes(self) -> np.ndarray:
        out = np.zeros(align128(self.size), np.uint8)
        for off, a in self.chunks:
            out[off:off + a.size] = a
        return out


@dataclass
class DecoderConfig:
    layers: int
    hidden: int
    inter: int
    n_q: int
    n_kv: int
    head_dim: int
    vocab: int
    group: int = 64
    eps: float = 1e-6
    rope_theta: float = 1e6
    # hybrid decoders: the layers whose token mixer is a DeltaNet block, and that block's geometry
    delta_layers: tuple = ()
    delta_value_heads: int = 0
    delta_qk_heads: int = 0
    delta_head_dim: int = 0
    conv_kernel: int = 4

    def as_dict(self):
        d = dict(self.__dict__)
        if not self.delta_layers:  # a plain decoder describes itself as before the hybrid fields existed (committed fixtures compare it)
            for k in ("delta_layers", "delta_value_heads", "delta_qk_heads", "delta_head_dim", "conv_kernel"):
                d.pop(k)
        else:
            d["delta_layers"] = list(self.delta_layers)
        return d


# BASELINE config 4: the full random-init decoder.
FULL_MODEL = DecoderConfig(layers=36, hidden=4096, inter=12288, n_q=32, n_kv=8, head_dim=128, vocab=151936)


@dataclass
class SyntheticPackage:
    cfg: DecoderConfig
    seed: int
    tensors: dict = field(default_factory=dict)  # name -> arrays (kept for the oracle)

    def layer_tensor(self, layer: int, name: str):
        """(packed, scales, biases) of one projection, regenerated from its own stream."""
        c = self.cfg
        shapes = {"q": (c.n_q * c.head_dim, c.hidden), "k": (c.n_kv * c.head_dim, c.hidden), "v": (c.n_kv * c.head_dim, c.hidden),
                  "o": (c.hidden, c.n_q * c.head_dim), "gate": (c.inter, c.hidden), "up": (c.inter, c.hidden),
                  "down": (c.hidden, c.inter)}
        rows, cols = shapes[name]
        return synth.affine_u4_model(self.seed, f"layer{layer}.{name}", rows, cols, c.group)

    def delta_tensor(self, layer: int, name: str):
        """(packed, scales, biases) of one DeltaNet projection: dqkv, dz, da, db, dout."""
        c = self.cfg
        dq, dv = (2 * c.delta_qk_heads + c.delta_value_heads) * c.delta_head_dim, c.delta_value_heads * c.delta_head_dim
        shapes = {"dqkv": (dq, c.hidden), "dz": (dv, c.hidden), "da": (c.delta_value_heads, c.hidden), "db": (c.delta_value_heads, c.hidden),
                  "dout": (c.hidden, dv)}
        rows, cols = shapes[name]
        return synth.affine_u4_model(self.seed, f"layer{layer}.{name}", rows, cols, c.group)

    def delta_small(self, layer: int):
        """(conv weight [qkv_dim, K], A_log [Hv], dt_bias [Hv], gated-norm weight [D]) of a DeltaNet layer."""
        c = self.cfg
        g = synth.rng_for(self.seed, f"layer{layer}.delta_small")
        dq = (2 * c.delta_qk_heads + c.delta_value_heads) * c.delta_head_dim
        conv_w = (g.standard_normal((dq, c.conv_kernel)) * 0.5).astype(np.float16)
        a_log = g.uniform(-2.0, 0.5, c.delta_value_heads).astype(np.float16)
        dt_bias = g.uniform(-0.5, 0.5, c.delta_value_heads).astype(np.float16)
        norm_w = (1.0 + 0.1 * g.standard_normal(c.delta_head_dim)).astype(np.float16)
        return conv_w, a_log, dt_bias, norm_w

    def norm_delta(self, name: str) -> np.ndarray:
        """Stored norm weight (w - 1): weight == 1 plus small seeded noise, so the stored tensor is near zero."""
        g = synth.rng_for(self.seed, name)
        return (g.uniform(-0.05, 0.05, size=self.cfg.hidden).astype(np.float32)).astype(np.float16)

    def embedding(self) -> np.ndarray:
        return synth.normal_f16(self.seed, "embedding", (self.cfg.vocab, self.cfg.hidden), 0.02)

    def lm_head(self) -> np.ndarray:
        return synth.normal_f16(self.seed, "lm_head", (self.cfg.vocab, self.cfg.hidden), 0.02)


def shard_rows(t, rank: int, world: int):
    """Column-parallel shard: a contiguous row range of packed / scales / biases."""
    packed, scales, biases = t
    n = packed.shape[0] // world
    sl = slice(rank * n, (rank + 1) * n)
    return packed[sl], scales[sl], biases[sl]


def shard_cols(t, rank: int, world: int, group: int):
    """Row-parallel shard: a column range aligned to quantisation groups, repacked densely."""
    packed, scales, biases = t
    cols = packed.shape[1] * 2
    n = cols // world
    assert n % group == 0, "K-shards must align to quantisation groups"
    cs = slice(rank * n // 2, (rank + 1) * n // 2)
    gs = slice(rank * n // group, (rank + 1) * n // group)
    return np.ascontiguousarray(packed[:, cs]), np.ascontiguousarray(scales[:, gs]), np.ascontiguousarray(biases[:, gs])


def build_image(pkg: SyntheticPackage, tp_rank: int = 0, tp_world: int = 1, keep_for_oracle: bool = False,
                vocab_parallel: bool = False):
    """Lay the (optionally tensor-parallel-sharded) synthetic decoder out as a weights image.

    Returns (image bytes, DecoderDesc, LayerRef array).  Column-parallel: Q by query head,
    K/V by KV head, gate/up by rows; row-parallel: O and down by group-aligned column ranges.
    vocab_parallel (tp_world > 1): the image holds only this rank's vocab / tp_world rows of the
    LM head (pair it with bit 3 of the decoder's fuse flags).
    """
    c = pkg.cfg
    assert c.n_kv % tp_world == 0 and c.inter % (tp_world * c.group) == 0
    img = WeightsImage()
    layers = (capi.LayerRef * c.layers)()
    keep = pkg.tensors if keep_for_oracle else None
    for l in range(c.layers):
        ref = layers[l]
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            t = pkg.layer_tensor(l, name)
            if keep is not None:
                keep[(l, name)] = t
            if tp_world > 1:
                t = shard_cols(t, tp_rank, tp_world, c.group) if name in ("o", "down") else shard_rows(t, tp_rank, tp_world)
            setattr(ref, name, img.add_affine(*t))
        n_in, n_post = pkg.norm_delta(f"layer{l}.input_norm"), pkg.norm_delta(f"layer{l}.post_norm")
        if keep is not None:
            keep[(l, "norms")] = (n_in, n_post)
        ref.input_norm, ref.post_norm = img.add(n_in), img.add(n_post)
    emb, head, fin = pkg.embedding(), pkg.lm_head(), pkg.norm_delta("final_norm")
    if keep is not None:
        keep["globals"] = (emb, head, fin)
    if vocab_parallel and tp_world > 1:
        assert c.vocab % tp_world == 0
        rows = c.vocab // tp_world
        head = np.ascontiguousarray(head[tp_rank * rows:(tp_rank + 1) * rows])
    desc = capi.DecoderDesc(layers=c.layers, hidden=c.hidden, inter=c.inter // tp_world, n_q=c.n_q // tp_world,
                            n_kv=c.n_kv // tp_world, head_dim=c.head_dim, vocab=c.vocab, group=c.group, eps=c.eps,
                            rope_theta=c.rope_theta, embedding=img.add(emb), lm_head=img.add(head),
                            final_norm=img.add(fin), tp_world=tp_world, tp_rank=tp_rank, fuse_residual=0)
    return img.tobytes(), desc, layers


@dataclass
class HybridRefs:
    """What ``smelt_cuda_build_hybrid_decoder`` needs beside the plain decoder's description."""
    desc: "capi.DeltaDesc"
    refs: object     # (capi.DeltaRef * layers)
    kinds: object    # (c_uint8 * layers): 1 = DeltaNet layer


def build_hybrid_image(pkg: SyntheticPackage, keep_for_oracle: bool = False):
    """``build_image`` for a hybrid decoder: every layer's norms and feed-forward tensors, attention tensors for the
    attention layers, the DeltaNet mixer's tensors for ``cfg.delta_layers``.  Returns (image, desc, layers, HybridRefs)."""
    c = pkg.cfg
    img = WeightsImage()
    layers = (capi.LayerRef * c.layers)()
    refs = (capi.DeltaRef * c.layers)()
    kinds = (C.c_uint8 * c.layers)()
    keep = pkg.tensors if keep_for_oracle else None
    for l in range(c.layers):
        ref = layers[l]
        is_delta = l in c.delta_layers
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            t = pkg.layer_tensor(l, name)
            if keep is not None:
                keep[(l, name)] = t
            if is_delta and name in ("q", "k", "v", "o"):
                continue  # the mixer of this layer is the DeltaNet block
            setattr(ref, name, img.add_affine(*t))
        n_in, n_post = pkg.norm_delta(f"layer{l}.input_norm"), pkg.norm_delta(f"layer{l}.post_norm")
        if keep is not None:
            keep[(l, "norms")] = (n_in, n_post)
        ref.input_norm, ref.post_norm = img.add(n_in), img.add(n_post)
        if is_delta:
            kinds[l] = 1
            for name, field_ in (("dqkv", "qkv"), ("dz", "z"), ("da", "a"), ("db", "b"), ("dout", "out")):
                t = pkg.delta_tensor(l, name)
                if keep is not None:
                    keep[(l, name)] = t
                setattr(refs[l], field_, img.add_affine(*t))
            small = pkg.delta_small(l)
            if keep is not None:
                keep[(l, "delta_small")] = small
            refs[l].conv_weight, refs[l].a_log, refs[l].dt_bias, refs[l].norm_weight = (img.add(a) for a in small)
    emb, head, fin = pkg.embedding(), pkg.lm_head(), pkg.norm_delta("final_norm")
    if keep is not None:
        keep["globals"] = (emb, head, fin)
    desc = capi.DecoderDesc(layers=c.layers, hidden=c.hidden, inter=c.inter, n_q=c.n_q, n_kv=c.n_kv, head_dim=c.head_dim, vocab=c.vocab,
                            group=c.group, eps=c.eps, rope_theta=c.rope_theta, embedding=img.add(emb), lm_head=img.add(head),
                            final_norm=img.add(fin), tp_world=1, tp_rank=0, fuse_residual=0)
    ddesc = capi.DeltaDesc(c.delta_value_heads, c.delta_qk_heads, c.delta_head_dim, c.conv_kernel)
    return img.tobytes(), desc, layers, HybridRefs(ddesc, refs, kinds)


class Decoder:
    """Drives the C ABI the way ``SmeltRuntime`` does: upload weights, build the record table,
    then ``decode_step`` per token or replay a captured graph."""

    def __init__(self, ctx: capi.Context, image: np.ndarray, desc: capi.DecoderDesc, layers, capacity: int, batch: int = 1,
                 fuse_residual: int = 0, hybrid: "HybridRefs | None" = None):
        self.ctx, self.desc, self.layers, self.capacity, self.batch = ctx, desc, layers, capacity, batch
        self.hybrid = hybrid
        desc.fuse_residual = int(fuse_residual)
        ctx.call("upload_weights", WEIGHTS_SLOT, image, C.c_size_t(image.nbytes))
        n = C.c_size_t(0)
        if hybrid is not None:
            build = lambda h, table: ctx.lib.smelt_cuda_build_hybrid_decoder(h, C.byref(desc), layers, C.byref(hybrid.desc), hybrid.refs, hybrid.kinds,
                                                                             capacity, table, C.byref(n))
        else:
            build = lambda h, table: ctx.lib.smelt_cuda_build_decoder(h, C.byref(desc), layers, capacity, batch, table, C.byref(n))
        st = build(None, None)
        if st != 0:
            raise capi.SmeltError(st, "build_decoder (count) failed")
        self.table = (capi.DispatchRecord * n.value)()
        ctx._check(build(ctx.h, self.table))
        self.n_records = n.value
        self.graph_ready = False

    def decode_step(self, tokens, position: int) -> np.ndarray:
        tokens = np.ascontiguousarray(np.atleast_1d(tokens), dtype=np.int32)
        out = np.zeros(self.batch, np.int32)
        self.ctx._check(self.ctx.lib.smelt_cuda_decode_step(self.ctx.h, self.table, self.n_records, tokens.ctypes.data_as(C.c_void_p),
                                                           int(position), out.ctypes.data_as(C.c_void_p)))
        return out

    def logits(self) -> np.ndarray:
        out = np.empty((self.batch, self.desc.vocab), np.float16)
        self.ctx._check(self.ctx.lib.smelt_cuda_read_slot(self.ctx.h, LOGITS_SLOT, 0, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def build_graph(self):
        self.ctx._check(self.ctx.lib.smelt_cuda_graph_build(self.ctx.h, self.table, self.n_records))
        self.graph_ready = True

    def graph_seed(self, tokens, position: int):
        tokens = np.ascontiguousarray(np.atleast_1d(tokens), dtype=np.int32)
        self.ctx._check(self.ctx.lib.smelt_cuda_graph_seed(self.ctx.h, tokens.ctypes.data_as(C.c_void_p), int(position)))

    def graph_decode(self, n_steps: int, read: bool = True):
        out = np.zeros((n_steps, self.batch), np.int32) if read else None
        self.ctx._check(self.ctx.lib.smelt_cuda_graph_decode(self.ctx.h, n_steps, out.ctypes.data_as(C.c_void_p) if read else None))
        return out

    def prefill(self, tokens, start_pos: int = 0, chunk: int = 0) -> int:
        """Prompt tokens through ``smelt_cuda_prefill`` (batch 1): fills the KV caches for positions
        ``start_pos ...`` and returns the argmax after the last token."""
        tokens = np.ascontiguousarray(np.asarray(tokens).reshape(-1), dtype=np.int32)
        out = C.c_int32(0)
        self.ctx._check(self.ctx.lib.smelt_cuda_prefill(self.ctx.h, C.byref(self.desc), self.layers, tokens.ctypes.data_as(C.c_void_p), len(tokens),
                                                        int(start_pos), int(chunk), C.byref(out)))
        return int(out.value)

    def build_prefill_table(self, max_chunk: int = 512):
        """The prompt-chunk dispatch table of this decoder in the reference's prefill record shapes
        (``smelt_cuda_build_prefill_table``); call it before ``build_graph``."""
        n = C.c_size_t(0)
        lib, hy = self.ctx.lib, self.hybrid
        if hy is not None:
            build = lambda h, table: lib.smelt_cuda_build_hybrid_prefill_table(h, C.byref(self.desc), self.layers, C.byref(hy.desc), hy.refs, hy.kinds,
                                                                               int(max_chunk), table, C.byref(n))
        else:
            build = lambda h, table: lib.smelt_cuda_build_prefill_table(h, C.byref(self.desc), self.layers, int(max_chunk), table, C.byref(n))
        self.ctx._check(build(None, None))
        self.prefill_records = (capi.DispatchRecord * n.value)()
        self.ctx._check(build(self.ctx.h, self.prefill_records))
        self.prefill_chunk = int(max_chunk)
        return self.prefill_records

    def prefill_by_table(self, tokens, start_pos: int = 0) -> int:
        """Prompt tokens through the prefill table, a chunk at a time (``smelt_cuda_enqueue_prefill``): the
        record-interpreted twin of ``prefill``.  Returns the argmax after the last token."""
        tokens = np.ascontiguousarray(np.asarray(tokens).reshape(-1), dtype=np.int32)
        if not hasattr(self, "prefill_records"):
            self.build_prefill_table()
        for t0 in range(0, len(tokens), self.prefill_chunk):
            part = np.ascontiguousarray(tokens[t0:t0 + self.prefill_chunk])
            self.ctx._check(self.ctx.lib.smelt_cuda_enqueue_prefill(self.ctx.h, self.prefill_records, len(self.prefill_records), part.ctypes.data_as(C.c_void_p),
                                                                    len(part), int(start_pos) + t0))
        out = np.zeros(1, np.int32)
        self.ctx._check(self.ctx.lib.smelt_cuda_read_slot(self.ctx.h, ARGMAX_SLOT, 0, out.ctypes.data_as(C.c_void_p), 4))
        return int(out[0])

    def reset_cache(self):
        L = self.desc.layers
        for l in range(2 * L):
            if self.hybrid is None or not self.hybrid.kinds[l % L]:
                self.ctx.call("zero_slot", KV_BASE_SLOT + l)
        if self.hybrid is not None:  # the DeltaNet layers' convolution taps and recurrent matrices
            for l in range(L):
                if self.hybrid.kinds[l]:
                    self.ctx.call("zero_slot", KV_BASE_SLOT + 2 * L + l)
                    self.ctx.call("zero_slot", KV_BASE_SLOT + 3 * L + l)

    # ── prompt-state snapshots (SmeltRuntime.captureDevicePromptSnapshot / restore…, SmeltRuntime.swift:1385-1553) ──
    def kv_slots(self):
        """The K and V cache slots of every layer as ``smelt_cuda_kv_slot`` records."""
        rows = (self.desc.n_kv // max(1, self.desc.tp_world)) * self.batch
        L = self.desc.layers
        which = [l for l in range(2 * L) if self.hybrid is None or not self.hybrid.kinds[l % L]]
        arr = (capi.KvSlot * len(which))()
        for i, l in enumerate(which):
            arr[i] = capi.KvSlot(KV_BASE_SLOT + l, rows, self.desc.head_dim)
        return arr

    def state_slots(self):
        """The convolution-tap and recurrent-matrix slots of a hybrid decoder's DeltaNet layers (copied whole by a snapshot)."""
        if self.hybrid is None:
            return []
        L = self.desc.layers
        return [KV_BASE_SLOT + 2 * L + l for l in range(L) if self.hybrid.kinds[l]] + [KV_BASE_SLOT + 3 * L + l for l in range(L) if self.hybrid.kinds[l]]

    def capture_snapshot(self, captured_length: int, prompt_length: int = 0, next_token: int = 0) -> "Snapshot":
        kv = self.kv_slots()
        st = np.array(self.state_slots(), np.int32)
        h = C.c_void_p()
        self.ctx._check(self.ctx.lib.smelt_cuda_snapshot_capture(self.ctx.h, kv, len(kv), st.ctypes.data_as(C.c_void_p) if len(st) else None, len(st),
                                                                 int(captured_length), int(prompt_length), int(next_token), C.byref(h)))
        return Snapshot(self.ctx, h)

    def restore_snapshot(self, snap: "Snapshot", length: int | None = None):
        self.ctx._check(self.ctx.lib.smelt_cuda_snapshot_restore(self.ctx.h, snap.h, snap.info().captured_length if length is None else int(length)))

    def teacher_forced(self, prompt, teacher, use_graph: bool = True) -> np.ndarray:
        """Scores a given continuation: feeds the prompt, then ``teacher[i - 1]`` at decode step i
        whatever the model itself chose, and returns the argmax of every step, shape
        ``[len(teacher), batch]``.  prompt ``[batch, n_prompt]``, teacher ``[n_steps, batch]``
        (the last teacher row is only compared, never fed)."""
        prompt = np.asarray(prompt, dtype=np.int32).reshape(self.batch, -1)
        teacher = np.asarray(teacher, dtype=np.int32).reshape(-1, self.batch)
        n_prompt = prompt.shape[1]
        if use_graph and not self.graph_ready:
            self.build_graph()

        def step(tokens, pos):
            if not use_graph:
                return self.decode_step(tokens, pos)
            self.graph_seed(tokens, pos)
            return self.graph_decode(1, read=True)[0]

        cur = None
        for i in range(n_prompt):
            if use_graph and i + 1 < n_prompt:
                self.graph_seed(prompt[:, i], i)
                self.graph_decode(1, read=False)
            else:
                cur = step(prompt[:, i], i)
        out = np.zeros((teacher.shape[0], self.batch), np.int32)
        for i in range(teacher.shape[0]):
            out[i] = cur
            if i + 1 < teacher.shape[0]:
                cur = step(teacher[i], n_prompt + i)
        return out

    def generate(self, prompt, n_decode: int, use_graph: bool = True) -> np.ndarray:
        """Feed the prompt token by token (the reference does the same without a prefill table,
        Sources/SmeltRuntime/SmeltModel.swift:619-631), then n_decode greedy steps."""
        prompt = np.asarray(prompt, dtype=np.int32).reshape(self.batch, -1)
        n_prompt = prompt.shape[1]
        out = np.zeros((n_decode, self.batch), np.int32)
        if use_graph:
            if not self.graph_ready:
                self.build_graph()
            # teacher-forced prompt: seed each position, replay one step
            for i in range(n_prompt - 1):
                self.graph_seed(prompt[:, i], i)
                self.graph_decode(1, read=False)
            self.graph_seed(prompt[:, n_prompt - 1], n_prompt - 1)
            return self.graph_decode(n_decode, read=True)
        cur = None
        for i in range(n_prompt):
            cur = self.decode_step(prompt[:, i], i)
        for i in range(n_decode):
            out[i] = cur
            if i + 1 < n_decode:
                cur = self.decode_step(cur, n_prompt + i)
        return out


class Snapshot:
    """Owner of one ``smelt_cuda_snapshot``."""

    def __init__(self, ctx: capi.Context, handle):
        self.ctx, self.h = ctx, handle

    def info(self) -> capi.SnapshotInfo:
        out = capi.SnapshotInfo()
        self.ctx._check(self.ctx.lib.smelt_cuda_snapshot_info(self.h, C.byref(out)))
        return out

    def export(self) -> np.ndarray:
        blob = np.zeros(self.info().blob_bytes, np.uint8)
        self.ctx._check(self.ctx.lib.smelt_cuda_snapshot_export(self.ctx.h, self.h, blob.ctypes.data_as(C.c_void_p), C.c_size_t(blob.nbytes)))
        return blob

    @classmethod
    def from_blob(cls, ctx: capi.Context, blob: np.ndarray) -> "Snapshot":
        blob = np.ascontiguousarray(blob, dtype=np.uint8)
        h = C.c_void_p()
        ctx._check(ctx.lib.smelt_cuda_snapshot_import(ctx.h, blob.ctypes.data_as(C.c_void_p), C.c_size_t(blob.nbytes), C.byref(h)))
        return cls(ctx, h)

    def close(self):
        if self.h:
            self.ctx.lib.smelt_cuda_snapshot_destroy(self.h)
            self.h = None


def write_package(path: str, cfg: DecoderConfig, image: np.ndarray, desc: capi.DecoderDesc, layers, capacity: int,
                  fuse_residual: int = 0, prefill_chunk: int = 0) -> None:
    """Writes a ``.smeltpkg`` directory for a synthetic decoder in the reference's wire formats:
    ``manifest.json`` (top-level and slotLayout keys camelCase, weight entries and buffer slots
    snake_case, Sources/SmeltSchema/SmeltManifest.swift:26-98, :806-817, :1710-1768),
    ``weights.bin`` (the image) and ``dispatches.bin`` (the decode table as raw 360-byte records,
    Sources/SmeltRuntime/SmeltRuntime.swift:6322-6350) and, with ``prefill_chunk`` > 0,
    ``prefill_dispatches.bin`` (the prompt-chunk table for chunks of up to that many positions, its
    pipelines appended to the manifest's and its activation slots to the buffer plan).  Stands in
    for the build-time compiler."""
    lib = capi.load()
    os.makedirs(path, exist_ok=True)
    desc.fuse_residual = int(fuse_residual)
    n = C.c_size_t(0)
    if lib.smelt_cuda_build_decoder(None, C.byref(desc), layers, capacity, 1, None, C.byref(n)) != 0:
        raise capi.SmeltError(1, "build_decoder (count) failed")
    table = (capi.DispatchRecord * n.value)()
    if lib.smelt_cuda_build_decoder(None, C.byref(desc), layers, capacity, 1, table, C.byref(n)) != 0:
        raise capi.SmeltError(1, "build_decoder (dry run) failed")
    need = C.c_size_t(0)
    lib.smelt_cuda_decoder_pipelines(C.byref(desc), 1, None, C.c_size_t(0), C.byref(need))
    buf = C.create_string_buffer(need.value)
    lib.smelt_cuda_decoder_pipelines(C.byref(desc), 1, buf, C.c_size_t(need.value), C.byref(need))
    pipelines = [p for p in buf.value.decode().split("\n") if p]
    H, I, D = cfg.hidden, desc.inter, cfg.head_dim
    qd, kvd = desc.n_q * D, desc.n_kv * D
    parts = (cfg.vocab + 2047) // 2048
    slots = [(0, "hiddenA", H * 2, "fp16", [H], "activation"), (1, "hiddenB", H * 2, "fp16", [H], "activation"),
             (8, "normOutBuf", H * 2, "fp16", [H], "activation"), (13, "ffnIntBuf", I * 2, "fp16", [I], "activation"),
             (14, "ffnDownBuf", H * 2, "fp16", [H], "activation"), (16, "logits", cfg.vocab * 2, "fp16", [cfg.vocab], "activation"),
             (17, "argmaxResult", 8, "int32", [2], "activation"), (20, "attnQBuf", qd * 2, "fp16", [qd], "activation"),
             (21, "attnKBuf", kvd * 2, "fp16", [kvd], "activation"), (22, "attnVBuf", kvd * 2, "fp16", [kvd], "activation"),
             (23, "attnOutBuf", qd * 2, "fp16", [qd], "activation"), (WEIGHTS_SLOT, "weights", 0, "raw", [], "weight"),
             (33, "tokenId", 4, "int32", [1], "dynamic"), (34, "position", 8, "int32", [2], "dynamic"),
             (35, "argmaxScratch", parts * 8, "raw", [parts * 8], "activation")]
    for l in range(cfg.layers):
        for base, name in ((KV_BASE_SLOT, "keyCache"), (KV_BASE_SLOT + cfg.layers, "valCache")):
            slots.append((base + l, f"{name}_{l}", desc.n_kv * capacity * D * 2, "fp16", [desc.n_kv, capacity, D], "state"))
    entries = []

    def affine_entry(name, ref, rows, cols):
        groups = cols // cfg.group
        entries.append({"name": name, "offset": int(ref.packed), "size_bytes": rows * cols // 2, "shape": [rows, cols], "dtype": "affine_u4",
                        "group_size": cfg.group, "scales_offset": int(ref.scales), "scales_size_bytes": rows * groups * 2,
                        "biases_offset": int(ref.biases), "biases_size_bytes": rows * groups * 2})

    for l in range(cfg.layers):
        L = layers[l]
        for name, rows, cols in (("q", qd, H), ("k", kvd, H), ("v", kvd, H), ("o", H, qd), ("gate", I, H), ("up", I, H), ("down", H, I)):
            affine_entry(f"layers.{l}.{name}", getattr(L, name), rows, cols)
        for name in ("input_norm", "post_norm"):
            entries.append({"name": f"layers.{l}.{name}", "offset": int(getattr(L, name)), "size_bytes": H * 2, "shape": [H], "dtype": "fp16"})
    rows_head = cfg.vocab // desc.tp_world if (fuse_residual & 8) and desc.tp_world > 1 else cfg.vocab
    entries += [{"name": "embedding", "offset": int(desc.embedding), "size_bytes": cfg.vocab * H * 2, "shape": [cfg.vocab, H], "dtype": "fp16"},
                {"name": "lm_head", "offset": int(desc.lm_head), "size_bytes": rows_head * H * 2, "shape": [rows_head, H], "dtype": "fp16"},
                {"name": "final_norm", "offset": int(desc.final_norm), "size_bytes": H * 2, "shape": [H], "dtype": "fp16"}]
    prefill_table = None
    if prefill_chunk > 0:
        T = int(prefill_chunk)
        pn = C.c_size_t(0)
        if lib.smelt_cuda_build_prefill_table(None, C.byref(desc), layers, T, None, C.byref(pn)) != 0:
            raise capi.SmeltError(1, "build_prefill_table (count) failed")
        prefill_table = (capi.DispatchRecord * pn.value)()
        if lib.smelt_cuda_build_prefill_table(None, C.byref(desc), layers, T, prefill_table, C.byref(pn)) != 0:
            raise capi.SmeltError(1, "build_prefill_table (dry run) failed")
        lib.smelt_cuda_prefill_pipelines(C.byref(desc), None, C.c_size_t(0), C.byref(need))
        pbuf = C.create_string_buffer(need.value)
        lib.smelt_cuda_prefill_pipelines(C.byref(desc), pbuf, C.c_size_t(need.value), C.byref(need))
        base = len(pipelines)
        pipelines = pipelines + [p for p in pbuf.value.decode().split("\n") if p]
        for r in prefill_table:  # the dry run numbers its pipelines from 0: they follow the decode table's in the manifest
            if r.op_kind == 0:
                r.pipeline += base
        slots = [s_ if s_[0] != 33 else (33, "tokenId", T * 4, "int32", [T], "dynamic") for s_ in slots]
        slots += [(2, "prefillHiddenA", T * H * 2, "fp16", [T, H], "activation"), (3, "prefillHiddenB", T * H * 2, "fp16", [T, H], "activation"),
                  (4, "prefillNormOut", T * H * 2, "fp16", [T, H], "activation"), (5, "prefillQ", T * qd * 2, "fp16", [T, qd], "activation"),
                  (6, "prefillK", T * kvd * 2, "fp16", [T, kvd], "activation"), (7, "prefillV", T * kvd * 2, "fp16", [T, kvd], "activation"),
                  (9, "prefillAttnOut", T * qd * 2, "fp16", [T, qd], "activation"), (10, "prefillFfn", T * I * 2, "fp16", [T, I], "activation")]
    manifest = {
        "version": 1, "kind": "text-generation", "architecture": "text-generation", "modelName": "synthetic-affine-u4-decoder",
        "config": {"hiddenSize": H, "numLayers": cfg.layers, "vocabSize": cfg.vocab, "staticSeqCapacity": capacity, "ropeDim": D,
                   "numDeltaLayers": 0, "numAttnLayers": cfg.layers, "deltaNumHeads": 0, "deltaQKVDim": 0, "attnQProjDim": qd,
                   "attnKProjDim": kvd, "attnVProjDim": kvd, "attnOutDim": qd, "ffnDim": I, "attentionByRole": {}, "turboQuantHPatterns": []},
        "checksums": {}, "device": {}, "weights": {"total_bytes": int(image.nbytes), "entries": entries},
        "buffers": {"slots": [{"index": i, "name": n_, "size_bytes": int(b), "dtype": dt, "shape": sh, "category": cat} for i, n_, b, dt, sh, cat in slots]},
        "pipelines": pipelines,
        "slotLayout": {"convStateBaseSlot": -1, "recStateBaseSlot": -1, "keyCacheBaseSlot": KV_BASE_SLOT, "valCacheBaseSlot": KV_BASE_SLOT + cfg.layers,
                       "ropeCosSlot": -1, "ropeSinSlot": -1, "ropeTablePairs": [], "tokenIdSlot": 33, "positionSlot": 34, "weightsSlot": WEIGHTS_SLOT},
    }
    with open(os.path.join(path, "manifest.json"), "w") as f:
        json.dump(manifest, f, sort_keys=True)
    np.asarray(image, np.uint8).tofile(os.path.join(path, "weights.bin"))
    with open(os.path.join(path, "dispatches.bin"), "wb") as f:
        f.write(bytes(table))
    if prefill_table is not None:
        with open(os.path.join(path, "prefill_dispatches.bin"), "wb") as f:
            f.write(bytes(prefill_table))


class PackageSession:
    """A ``.smeltpkg`` opened by the library's own reader (``smelt_cuda_open_package``): the
    counterpart of ``SmeltRuntime(packagePath:)`` followed by ``decodeStep``."""

    def __init__(self, ctx: capi.Context, path: str, context_capacity: int = 0):
        self.ctx = ctx
        self.info = capi.PackageInfo()
        opts = capi.PackageOptions(context_capacity=context_capacity, context_limit=0)
        ctx._check(ctx.lib.smelt_cuda_open_package(ctx.h, path.encode(), C.byref(opts), C.byref(self.info)))
        table, n = C.c_void_p(), C.c_size_t(0)
        ctx._check(ctx.lib.smelt_cuda_package_table(ctx.h, C.byref(table), C.byref(n)))
        self.table, self.n_records = table, n.value

    def decode_step(self, token: int, position: int) -> int:
        tok, out = np.array([token], np.int32), np.zeros(1, np.int32)
        self.ctx._check(self.ctx.lib.smelt_cuda_decode_step(self.ctx.h, self.table, self.n_records, tok.ctypes.data_as(C.c_void_p), int(position),
                                                           out.ctypes.data_as(C.c_void_p)))
        return int(out[0])

    def build_graph(self):
        self.ctx._check(self.ctx.lib.smelt_cuda_graph_build(self.ctx.h, self.table, self.n_records))

    def prefill(self, tokens, start_pos: int = 0, chunk: int = 0) -> int:
        """The prompt through the package's own prefill table (``smelt_cuda_package_prefill_table`` +
        ``smelt_cuda_enqueue_prefill``), ``chunk`` positions at a time (0 = all at once); returns the argmax after
        the last token.  Raises when the package has no runnable prefill table."""
        table, n = C.c_void_p(), C.c_size_t(0)
        self.ctx._check(self.ctx.lib.smelt_cuda_package_prefill_table(self.ctx.h, C.byref(table), C.byref(n)))
        tokens = np.ascontiguousarray(np.asarray(tokens).reshape(-1), dtype=np.int32)
        step = int(chunk) if chunk else len(tokens)
        for t0 in range(0, len(tokens), step):
            part = np.ascontiguousarray(tokens[t0:t0 + step])
            self.ctx._check(self.ctx.lib.smelt_cuda_enqueue_prefill(self.ctx.h, table, n.value, part.ctypes.data_as(C.c_void_p), len(part), int(start_pos) + t0))
        out = np.zeros(1, np.int32)
        self.ctx._check(self.ctx.lib.smelt_cuda_read_slot(self.ctx.h, self.info.argmax_slot, 0, out.ctypes.data_as(C.c_void_p), 4))
        return int(out[0])

    def graph_step(self, token: int, position: int) -> int:
        tok, out = np.array([token], np.int32), np.zeros(1, np.int32)
        self.ctx._check(self.ctx.lib.smelt_cuda_graph_step(self.ctx.h, tok.ctypes.data_as(C.c_void_p), int(position), out.ctypes.data_as(C.c_void_p)))
        return int(out[0])


def inspect_package(path: str):
    """(status, PackageInfo, first problem) from the host-only validator."""
    info, err = capi.PackageInfo(), C.create_string_buffer(512)
    st = capi.load().smelt_cuda_inspect_package(path.encode(), C.byref(info), err, C.c_size_t(512))
    return st, info, err.value.decode()


def open_tp_exchange(ctx: capi.Context, dist, world: int) -> None:
    """Every rank publishes the IPC handle of its exchange buffer, gathers the others' through
    ``torch.distributed`` and maps them: enables the fused all-reduce + residual add records."""
    import torch

    handle = np.zeros(capi.TP_HANDLE_BYTES, np.uint8)
    ctx._check(ctx.lib.smelt_cuda_tp_exchange_handle(ctx.h, handle.ctypes.data_as(C.c_void_p)))
    mine = torch.from_numpy(handle).cuda()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    allh = np.ascontiguousarray(torch.stack(gathered).cpu().numpy())
    ctx._check(ctx.lib.smelt_cuda_tp_exchange_open(ctx.h, allh.ctypes.data_as(C.c_void_p)))
    dist.barrier()



def compare_greedy(got, tokens, runner_up, margins, tie: float = 0.02) -> dict:
    """Outcome of a teacher-forced replay against known-good greedy tokens of one sequence.

    A step counts as identical when the ids are equal.  A differing id is a tie break, not an
    error, only when the known-good top-2 logit margin of that step is below ``tie`` (two fp16
    ulps at the magnitude of these logits) AND the id is the known-good runner-up; everything
    else lands in ``wrong``."""
    got, tokens, runner_up, margins = (np.asarray(a).reshape(-1) for a in (got, tokens, runner_up, margins))
    diff = np.nonzero(got != tokens)[0]
    wrong = [int(i) for i in diff if not (margins[i] < tie and got[i] == runner_up[i])]
    first = int(diff[0]) if diff.size else None
    return {"checked": int(tokens.size), "identical": int(tokens.size - diff.size), "tie_breaks": int(diff.size - len(wrong)),
            "wrong": wrong, "first_mismatch": first, "margin": float(margins[first]) if first is not None else None}

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

    def as_dict(self):
        return dict(self.__dict__)


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


class Decoder:
    """Drives the C ABI the way ``SmeltRuntime`` does: upload weights, build the record table,
    then ``decode_step`` per token or replay a captured graph."""

    def __init__(self, ctx: capi.Context, image: np.ndarray, desc: capi.DecoderDesc, layers, capacity: int, batch: int = 1,
                 fuse_residual: int = 0):
        self.ctx, self.desc, self.layers, self.capacity, self.batch = ctx, desc, layers, capacity, batch
        desc.fuse_residual = int(fuse_residual)
        ctx.call("upload_weights", WEIGHTS_SLOT, image, C.c_size_t(image.nbytes))
        n = C.c_size_t(0)
        st = ctx.lib.smelt_cuda_build_decoder(None, C.byref(desc), layers, capacity, batch, None, C.byref(n))
        if st != 0:
            raise capi.SmeltError(st, "build_decoder (count) failed")
        self.table = (capi.DispatchRecord * n.value)()
        ctx._check(ctx.lib.smelt_cuda_build_decoder(ctx.h, C.byref(desc), layers, capacity, batch, self.table, C.byref(n)))
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

    def reset_cache(self):
        for l in range(2 * self.desc.layers):
            self.ctx.call("zero_slot", KV_BASE_SLOT + l)

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
    """Verdict of a teacher-forced replay against known-good greedy tokens of one sequence.

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

"""Data-parallel training of one update plan across the GPUs of a box.

The reference is single-process; this is the multi-GPU form of its step
(runtime/engine/update_engine.cc:736-771). A global step is K *chunks*, each one
execution of the plan's train stream up to the first optimiser instruction
(update_engine.cc:249-261) on the plan's compiled batch. One process per GPU runs
K / world_size consecutive chunks and keeps one packed LoRA-gradient set per chunk.
The sets are summed in ONE fixed binary tree over the chunk index,
((g0+g1)+(g2+g3))+..., scaled by 1/K (a power of two), and every rank then runs the
optimiser instructions on identical bits. The tree is over chunks, not ranks: the
local subtree is reduced on the device, the world_size partial sums are exchanged
with an NCCL all-gather over NVLink and the tree is finished in rank order — so 1,
2, 4 and 8 GPU runs produce bit-identical parameters. Only LoRA gradients and the
scalar loss cross GPUs; frozen weights and adapter state are replicated.

K and world_size must be powers of two with world_size <= K.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from .engine import UpdateEngine
from .formats import Op, parse_plan


def _is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def gradient_spans(train: np.ndarray):
    """(arena offset, float count) of every optimiser instruction's gradient operand,
    plus the loss... in stream order. Reference: in[1] of kSgdStep / kAdamWStep."""
    offs, counts = [], []
    for ins in train:
        if int(ins["opcode"]) in (int(Op.SGD), int(Op.ADAMW)):
            offs.append(int(ins["in"][1]))
            counts.append(int(ins["out"][0]))
    return np.array(offs, np.uint64), np.array(counts, np.uint64)


def tree_sum_host(sets: np.ndarray) -> np.ndarray:
    """The fixed binary tree over axis 0, on the host (the CPU model of the device
    tree; used by the gloo tests)."""
    s = [np.asarray(x, np.float32).copy() for x in sets]
    stride = 1
    while stride < len(s):
        for a in range(0, len(s), 2 * stride):
            if a + stride < len(s):
                s[a] = s[a] + s[a + stride]
        stride *= 2
    return s[0]


class DataParallelTrainer:
    """One rank of a data-parallel job. With world_size == 1 no process group is needed."""

    def __init__(self, plan: bytes, chunks_per_step: int, rank: int = 0, world_size: int = 1,
                 device: int = 0, mode: int = 0, gemm: int = 0, group=None):
        import torch
        if not (_is_pow2(chunks_per_step) and _is_pow2(world_size) and world_size <= chunks_per_step):
            raise ValueError("chunks_per_step and world_size must be powers of two, world_size <= chunks")
        self.torch = torch
        self.K, self.rank, self.world = chunks_per_step, rank, world_size
        self.local = chunks_per_step // world_size
        self.group = group
        self.engine = UpdateEngine(device, mode, gemm)
        self.engine.load_from_memory(plan)
        self.h = self.engine.header
        p = parse_plan(plan)
        self.n_train = len(p.train)
        self.opt_begin = self.engine.opt_begin()
        self.offs, self.counts = gradient_spans(p.train)
        self.fps = int(self.counts.sum()) + 1          # + the chunk loss
        self.dev = torch.device("cuda", device)
        self.ctx = self.engine.ctx()
        self.stream = torch.cuda.ExternalStream(L.lib().seeml_b200_ctx_stream(self.ctx), device=self.dev)
        with torch.cuda.device(self.dev):
            self.sets = torch.zeros((max(self.local, 1), self.fps), dtype=torch.float32, device=self.dev)
            self.gathered = torch.zeros((world_size, self.fps), dtype=torch.float32, device=self.dev)
        # the loss rides the packed set as one more span
        self.pack_offs = np.concatenate([self.offs, np.array([self.h.loss_ref], np.uint64)])
        self.pack_counts = np.concatenate([self.counts, np.array([1], np.uint64)])
        self.step_index = 0
        self.launches = 0
        in_bytes = self.h.input_floats * 4
        self._pin_in = [L.lib().seeml_b200_pinned_alloc(in_bytes) for _ in range(2)]
        self._pin_lab = [L.lib().seeml_b200_pinned_alloc(max(self.h.label_bytes, 4)) for _ in range(2)]
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # -- one global step -----------------------------------------------------------------
    def _pack(self, local_chunk: int):
        lib = L.lib()
        dst = self.sets[local_chunk].data_ptr()
        L.check(lib.seeml_b200_grads_pack(self.ctx, self.pack_offs.ctypes.data, self.pack_counts.ctypes.data,
                                          len(self.pack_offs), C.c_void_p(dst)))

    def _reduce_and_step(self):
        lib, torch = L.lib(), self.torch
        L.check(lib.seeml_b200_tree_sum(self.ctx, C.c_void_p(self.sets.data_ptr()), self.fps, self.local, 1.0))
        if self.world > 1:
            with torch.cuda.stream(self.stream):
                torch.distributed.all_gather_into_tensor(self.gathered, self.sets[0], group=self.group)
            total = self.gathered
        else:
            total = self.sets
        L.check(lib.seeml_b200_tree_sum(self.ctx, C.c_void_p(total.data_ptr()), self.fps,
                                        self.world if self.world > 1 else 1, 1.0 / self.K))
        L.check(lib.seeml_b200_grads_unpack(self.ctx, self.pack_offs.ctypes.data, self.pack_counts.ctypes.data,
                                            len(self.pack_offs), C.c_void_p(total.data_ptr())))
        self.engine.run_train_range(self.opt_begin, self.n_train)
        self.launches += self.engine.last_launches() + 4

    def step(self, tokens: np.ndarray, labels: np.ndarray) -> float:
        """One global step from HOST buffers: `tokens` / `labels` hold this rank's `local`
        chunks back to back ([local, batch] words each). Copies ride pinned staging
        buffers and the copy stream; the mean loss over all K chunks is read back."""
        lib = L.lib()
        self.step_index += 1
        self.engine.set_step(self.step_index)
        self.launches = 0
        in_b, lab_b = self.h.input_floats * 4, self.h.label_bytes
        tok = np.ascontiguousarray(tokens).reshape(self.local, -1).view(np.uint8)
        lab = np.ascontiguousarray(labels).reshape(self.local, -1).view(np.uint8)

        def stage(c):
            s = c & 1
            C.memmove(self._pin_in[s], tok[c].ctypes.data, in_b)
            C.memmove(self._pin_lab[s], lab[c].ctypes.data, lab_b)
            L.check(lib.seeml_b200_stage_h2d(self.ctx, s, self._pin_in[s], in_b, self._pin_lab[s], lab_b))
        stage(0)
        for c in range(self.local):
            s = c & 1
            L.check(lib.seeml_b200_stage_commit(self.ctx, s, self.h.input_ref, self.h.label_ref))
            L.check(lib.seeml_b200_stage_wait(self.ctx, s))
            self.engine.run_train_range(0, self.opt_begin)
            self.launches += self.engine.last_launches() + 2
            if c + 1 < self.local:
                stage(c + 1)            # next chunk's copy overlaps this chunk's compute
            self._pack(c)
        self._reduce_and_step()
        self.h2d_bytes = self.local * (in_b + lab_b)
        self.d2h_bytes = 4
        return self.engine.loss_value()

    def step_resident(self, tokens_dev, labels_dev, read_loss: bool = False):
        """One global step with this rank's chunks already in HBM ([local, batch] i32 / f32
        torch tensors): device-to-device moves into the I/O slots only."""
        lib = L.lib()
        self.step_index += 1
        self.engine.set_step(self.step_index)
        self.launches = 0
        in_b, lab_b = self.h.input_floats * 4, self.h.label_bytes
        for c in range(self.local):
            L.check(lib.seeml_b200_d2d(self.ctx, self.h.input_ref, C.c_void_p(tokens_dev[c].data_ptr()), in_b))
            L.check(lib.seeml_b200_d2d(self.ctx, self.h.label_ref, C.c_void_p(labels_dev[c].data_ptr()), lab_b))
            self.engine.run_train_range(0, self.opt_begin)
            self.launches += self.engine.last_launches() + 2
            self._pack(c)
        self._reduce_and_step()
        return self.engine.loss_value() if read_loss else None

    def persistent(self) -> np.ndarray:
        return self.engine.arena_read(0, self.h.persistent_size)

    def close(self):
        for p in self._pin_in + self._pin_lab:
            L.lib().seeml_b200_pinned_free(p)
        self._pin_in, self._pin_lab = [], []
        self.engine.close()

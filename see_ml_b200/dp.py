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
from .formats import Op


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
    """One rank of a data-parallel job: a thin caller of the C ABI's K-chunk step
    (seeml_b200_engine_dp_configure / dp_step_host / dp_step_device). With world_size == 1
    no communicator is needed. With more ranks the NCCL id made by rank 0 is handed round
    through `group` (a torch.distributed process group, used for that one broadcast only)
    or passed in as `comm_id` (128 bytes) by a host that has its own channel."""

    def __init__(self, plan: bytes, chunks_per_step: int, rank: int = 0, world_size: int = 1,
                 device: int = 0, mode: int = 0, gemm: int = 0, group=None, comm_id: bytes | None = None):
        if not (_is_pow2(chunks_per_step) and _is_pow2(world_size) and world_size <= chunks_per_step):
            raise ValueError("chunks_per_step and world_size must be powers of two, world_size <= chunks")
        lib = L.lib()
        self.K, self.rank, self.world, self.device = chunks_per_step, rank, world_size, device
        self.local = chunks_per_step // world_size
        self.engine = UpdateEngine(device, mode, gemm)
        self.engine.load_from_memory(plan)
        self.h = self.engine.header
        self.ctx = self.engine.ctx()
        self.comm = C.c_void_p()
        if world_size > 1:
            if comm_id is None:
                import torch
                buf = torch.zeros(128, dtype=torch.uint8, device=torch.device("cuda", device))
                if rank == 0:
                    raw = (C.c_uint8 * 128)()
                    L.check(lib.seeml_b200_comm_unique_id(raw))
                    buf.copy_(torch.tensor(list(raw), dtype=torch.uint8))
                torch.distributed.broadcast(buf, src=0, group=group)
                comm_id = bytes(buf.cpu().tolist())
            idbuf = (C.c_uint8 * 128).from_buffer_copy(comm_id)
            L.check(lib.seeml_b200_comm_init(device, idbuf, rank, world_size, C.byref(self.comm)))
        L.check(lib.seeml_b200_engine_dp_configure(self.engine.h, chunks_per_step, rank, world_size, self.comm))
        self.launches = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    @property
    def stream(self):
        """The compute stream as a torch stream (for CUDA-event timing by the caller)."""
        import torch
        return torch.cuda.ExternalStream(L.lib().seeml_b200_ctx_stream(self.ctx),
                                         device=torch.device("cuda", self.device))

    def step(self, tokens: np.ndarray, labels: np.ndarray) -> float:
        """One global step from HOST buffers: `tokens` / `labels` hold this rank's `local`
        chunks back to back ([local, batch] words each). The mean loss over all K chunks is
        read back."""
        tok = np.ascontiguousarray(tokens)
        lab = np.ascontiguousarray(labels)
        loss = C.c_float()
        L.check(L.lib().seeml_b200_engine_dp_step_host(self.engine.h, tok.ctypes.data_as(C.c_void_p),
                                                       lab.ctypes.data_as(C.c_void_p), C.byref(loss)))
        self.launches = self.engine.last_launches()
        self.h2d_bytes = self.local * (self.h.input_floats * 4 + self.h.label_bytes)
        self.d2h_bytes = 4
        return loss.value

    def step_resident(self, tokens_dev, labels_dev, read_loss: bool = False):
        """One global step with this rank's chunks already in HBM ([local, batch] i32 / f32
        torch tensors, contiguous): device-to-device moves into the I/O slots only."""
        loss = C.c_float()
        L.check(L.lib().seeml_b200_engine_dp_step_device(self.engine.h, C.c_void_p(tokens_dev.data_ptr()),
                                                         C.c_void_p(labels_dev.data_ptr()),
                                                         C.byref(loss) if read_loss else None))
        self.launches = self.engine.last_launches()
        return loss.value if read_loss else None

    def persistent(self) -> np.ndarray:
        return self.engine.arena_read(0, self.h.persistent_size)

    def close(self):
        self.engine.close()
        if self.comm:
            L.lib().seeml_b200_comm_destroy(self.comm)
            self.comm = C.c_void_p()

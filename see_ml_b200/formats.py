"""Byte layouts of the SeeML artefacts the backend consumes, kept bit-exact.

* SEEU update plan: 280-byte ``PlanHeader``, 64-byte ``UpdateInstruction``,
  24-byte ``EmitEntry`` (reference: source/plan/schema.h:84-178,
  source/plan/instruction.h:27-151). Little-endian, packed.
* SDS corpus (reference: runtime/feeder/dataset.h:13-26).
* SMF model container, writer only (reference: source/language/model_format.h:45-130,
  tool/export_model.py:74-130) — used to hand the same model to the reference
  compiler in parity tests.
* The plan seal ``PlanSelfHash`` / ``ContentHash64`` (reference:
  source/identity/hash.h:80-161), vectorised with numpy.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field, fields
from enum import IntEnum

import numpy as np

SEEU_MAGIC = 0x55454553
SEEU_VERSION = 7
SEEU_OLDEST_READABLE = 4
RODATA_BIT = 1 << 63
NULL_REF = (1 << 64) - 1
ALIGN = 64
PLAN_HASH_OFFSET = 216


def align_up(v: int, a: int = ALIGN) -> int:
    return (v + a - 1) & ~(a - 1)


class Op(IntEnum):
    """Opcode vocabulary (reference: source/plan/instruction.h:27-104)."""
    NOP = 0
    GEMM_NN = 1
    GEMM_NT = 2
    GEMM_TN = 3
    GEMM_ACC_NN = 4
    ADD = 5
    ADD_BIAS = 6
    RELU_FWD = 7
    RELU_BWD = 8
    SCALE = 9
    REDUCE_ROWS = 10
    XENT_FWD = 11
    XENT_BWD = 12
    MSE_FWD = 13
    MSE_BWD = 14
    KL_FWD = 15
    KL_BWD = 16
    SGD = 17
    ADAMW = 18
    FILL = 19
    COPY = 20
    MUL = 21
    GELU_FWD = 22
    GELU_BWD = 23
    SILU_FWD = 24
    SILU_BWD = 25
    LAYERNORM_FWD = 26
    LAYERNORM_BWD = 27
    CLIP_NORM = 28
    GEMM_NN_Q8 = 29
    GEMM_NT_Q8 = 30
    RMSNORM_FWD = 31
    RMSNORM_BWD = 32
    ROPE_FWD = 33
    ROPE_BWD = 34
    ATTN_FWD = 35
    ATTN_DP = 36
    ATTN_DV = 37
    SOFTMAX_ROWS_BWD = 38
    ATTN_DQ = 39
    ATTN_DK = 40
    EMBED = 41


FLAG_BIAS = 1
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3

INSTR_DTYPE = np.dtype([("opcode", "<u2"), ("flags", "<u2"), ("pad", "<u4"),
                        ("in", "<u8", (4,)), ("out", "<u8", (3,))])
assert INSTR_DTYPE.itemsize == 64
EMIT_DTYPE = np.dtype([("smf_data_offset", "<u8"), ("byte_size", "<u8"),
                       ("arena_offset", "<u8")])
assert EMIT_DTYPE.itemsize == 24

_HEADER_FMT = "<II" + "QQ" + "QQQQ" + "II" + "Q" + "QQQQ" + "QQQQQQ" + "fffff" + "I" + \
    "QQ" + "QQ" + "QQ" + "II" + "Q" + "ff" + "II" + "Q" + "QQ"
assert struct.calcsize(_HEADER_FMT) == 280


def f32_bits(x: float) -> int:
    return int(np.float32(x).view(np.uint32))


def bits_f32(w: int) -> float:
    return float(np.uint32(w & 0xFFFFFFFF).view(np.float32))


def pack32(hi: int, lo: int) -> int:
    assert 0 <= hi <= 0xFFFFFFFF and 0 <= lo <= 0xFFFFFFFF
    return (hi << 32) | lo


@dataclass
class PlanHeader:
    magic: int = SEEU_MAGIC
    version: int = SEEU_VERSION
    arena_size: int = 0
    persistent_size: int = 0
    input_ref: int = NULL_REF
    input_floats: int = 0
    label_ref: int = NULL_REF
    label_bytes: int = 0
    label_kind: int = 0
    optimizer_kind: int = 1
    loss_ref: int = NULL_REF
    train_instr_offset: int = 0
    train_instr_count: int = 0
    merge_instr_offset: int = 0
    merge_instr_count: int = 0
    rodata_offset: int = 0
    rodata_size: int = 0
    persist_init_offset: int = 0
    persist_init_size: int = 0
    emit_table_offset: int = 0
    emit_count: int = 0
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    pad2: int = 0
    batch: int = 0
    default_steps: int = 0
    eval_instr_offset: int = 0
    eval_instr_count: int = 0
    source_model_hash: int = 0
    plan_hash: int = 0
    lr_schedule: int = 0
    pad3: int = 0
    warmup_steps: int = 0
    min_lr_factor: float = 0.0
    clip_norm: float = 0.0
    input_kind: int = 0
    pad4: int = 0
    seq_len: int = 0
    reserved0: int = 0
    reserved1: int = 0

    def pack(self) -> bytes:
        return struct.pack(_HEADER_FMT, *[getattr(self, f.name) for f in fields(self)])

    @classmethod
    def unpack(cls, blob: bytes) -> "PlanHeader":
        return cls(*struct.unpack(_HEADER_FMT, bytes(blob[:280])))


# --- hashes -------------------------------------------------------------------
_FNV_BASIS = np.uint64(0xcbf29ce484222325)
_FNV_PRIME = np.uint64(0x100000001b3)
_GOLDEN = 0x9E3779B97F4A7C15
_M64 = (1 << 64) - 1


def _mix_word(state: int, word: int) -> int:
    for b in range(8):
        state ^= (word >> (8 * b)) & 0xFF
        state = (state * 0x100000001b3) & _M64
    return state


def _striped(chunk: np.ndarray) -> int:
    """8-lane interleaved FNV-1a of one span (reference: hash.h:89-109)."""
    n = int(chunk.size)
    lanes = np.array([(0xcbf29ce484222325 ^ ((_GOLDEN * (l + 1)) & _M64)) for l in range(8)],
                     dtype=np.uint64)
    full = n // 8
    with np.errstate(over="ignore"):
        if full:
            body = chunk[:full * 8].reshape(full, 8).astype(np.uint64)
            # state_k = (state_{k-1} ^ b_k) * p. XOR only touches the low byte, but it
            # does not commute with the multiply, so iterate rows; 8 lanes vectorised.
            for row in body:
                lanes = (lanes ^ row) * _FNV_PRIME
        for l, byte in enumerate(chunk[full * 8:]):
            lanes[l] = (lanes[l] ^ np.uint64(byte)) * _FNV_PRIME
    h = 0xcbf29ce484222325
    for l in range(8):
        h = _mix_word(h, int(lanes[l]))
    return _mix_word(h, n)


def _chunk_grain(n: int, grain: int) -> int:
    cap = (n + 255) // 256
    return max(grain, cap, 1)


def content_hash64(data: bytes | np.ndarray, hash_off: int | None = None) -> int:
    """ContentHash64 / PlanSelfHash. Pure-Python row loop: meant for small blobs
    (tests); the host library carries the fast implementation."""
    buf = np.frombuffer(bytes(data), dtype=np.uint8).copy()
    if hash_off is not None:
        buf[hash_off:hash_off + 8] = 0
    n = int(buf.size)
    g = _chunk_grain(n, 1 << 20)
    h = 0xcbf29ce484222325
    if n == 0:
        h = _mix_word(h, _striped(buf))
    for b in range(0, n, g):
        h = _mix_word(h, _striped(buf[b:min(n, b + g)]))
    return _mix_word(h, n)


# --- plan container -------------------------------------------------------------
@dataclass
class Plan:
    header: PlanHeader
    train: np.ndarray
    merge: np.ndarray
    eval: np.ndarray
    rodata: np.ndarray            # uint8
    persist_init: np.ndarray      # uint8
    emit: np.ndarray
    blob: bytes | None = None


def parse_plan(blob: bytes) -> Plan:
    h = PlanHeader.unpack(blob)
    mv = memoryview(blob)

    def sec(off, count, dt):
        return np.frombuffer(mv, dtype=dt, count=count, offset=off).copy()
    return Plan(
        header=h,
        train=sec(h.train_instr_offset, h.train_instr_count, INSTR_DTYPE),
        merge=sec(h.merge_instr_offset, h.merge_instr_count, INSTR_DTYPE),
        eval=sec(h.eval_instr_offset, h.eval_instr_count, INSTR_DTYPE),
        rodata=np.frombuffer(mv, dtype=np.uint8, count=h.rodata_size, offset=h.rodata_offset),
        persist_init=np.frombuffer(mv, dtype=np.uint8, count=h.persist_init_size,
                                   offset=h.persist_init_offset),
        emit=sec(h.emit_table_offset, h.emit_count, EMIT_DTYPE),
        blob=blob)


def assemble_plan(header: PlanHeader, train: np.ndarray, merge: np.ndarray, eval_: np.ndarray,
                  rodata: np.ndarray, persist_init: np.ndarray, emit: np.ndarray,
                  hasher=None) -> bytes:
    """Section order and alignment of the reference's plan assembly
    (compiler/driver/update_compiler.cc:488-536); seals plan_hash last.
    ``hasher(blob_bytes, hash_off) -> int`` may supply a fast PlanSelfHash."""
    off = align_up(280)
    header.train_instr_offset, header.train_instr_count = off, len(train)
    off += len(train) * 64
    header.merge_instr_offset, header.merge_instr_count = off, len(merge)
    off += len(merge) * 64
    header.eval_instr_offset, header.eval_instr_count = off, len(eval_)
    off += len(eval_) * 64
    off = align_up(off)
    header.rodata_offset, header.rodata_size = off, int(rodata.nbytes)
    off = align_up(off + rodata.nbytes)
    header.persist_init_offset, header.persist_init_size = off, int(persist_init.nbytes)
    off = align_up(off + persist_init.nbytes)
    header.emit_table_offset, header.emit_count = off, len(emit)
    off += len(emit) * 24
    header.plan_hash = 0
    blob = bytearray(off)
    blob[0:280] = header.pack()
    blob[header.train_instr_offset:header.train_instr_offset + train.nbytes] = train.tobytes()
    blob[header.merge_instr_offset:header.merge_instr_offset + merge.nbytes] = merge.tobytes()
    blob[header.eval_instr_offset:header.eval_instr_offset + eval_.nbytes] = eval_.tobytes()
    blob[header.rodata_offset:header.rodata_offset + rodata.nbytes] = rodata.tobytes()
    blob[header.persist_init_offset:header.persist_init_offset + persist_init.nbytes] = \
        persist_init.tobytes()
    blob[header.emit_table_offset:header.emit_table_offset + emit.nbytes] = emit.tobytes()
    hfn = hasher or (lambda b, o: content_hash64(b, o))
    header.plan_hash = hfn(blob, PLAN_HASH_OFFSET)
    blob[PLAN_HASH_OFFSET:PLAN_HASH_OFFSET + 8] = struct.pack("<Q", header.plan_hash)
    return bytes(blob)


# --- SDS corpus -----------------------------------------------------------------
SDS_MAGIC = 0x31534453


def write_sds(path: str, inputs: np.ndarray, labels: np.ndarray | None, label_kind: int = 1):
    """f32 feature rows + (i32 class | dense f32 | no) labels, interleaved per record."""
    x = np.ascontiguousarray(inputs, dtype=np.float32)
    n, d = x.shape
    if labels is None:
        label_kind, label_dim, lab = 0, 0, None
    elif label_kind == 1:
        lab, label_dim = np.asarray(labels, dtype=np.int32).reshape(n, 1), 0
    else:
        lab = np.asarray(labels, dtype=np.float32).reshape(n, -1)
        label_dim = lab.shape[1]
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQIIQ", SDS_MAGIC, 1, n, d, label_kind, 0, label_dim))
        if lab is None:
            f.write(x.tobytes())
        else:
            rec = np.concatenate([x.view(np.uint8).reshape(n, -1),
                                  np.ascontiguousarray(lab).view(np.uint8).reshape(n, -1)], axis=1)
            f.write(rec.tobytes())


def write_token_sds(path: str, records: np.ndarray):
    """[N, S+1] i32 token records; labels are the shifted view, derived at serve time."""
    a = np.ascontiguousarray(records, dtype=np.int32)
    assert a.ndim == 2 and a.shape[1] >= 2 and (a >= 0).all()
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQIIQ", SDS_MAGIC, 2, a.shape[0], a.shape[1] - 1, 1, 1, 0))
        f.write(a.tobytes())


# --- SMF model container (writer) -------------------------------------------------
SMF_MAGIC = 0x31464D53
(SMF_MATMUL, SMF_ADDBIAS, SMF_RELU, SMF_GELU, SMF_SILU, SMF_MUL, SMF_LAYERNORM, SMF_ADD,
 SMF_RMSNORM, SMF_ROPE, SMF_ATTENTION, SMF_EMBEDDING) = range(12)


def _s(name: str) -> bytes:
    b = name.encode()
    return struct.pack("<H", len(b)) + b


@dataclass
class ModelGraph:
    """A frozen model as the SMF container describes it: named constant tensors
    and a topologically ordered op list over the op-kind vocabulary above."""
    input_name: str
    input_dim: int
    seq_len: int = 0
    token_input: bool = False
    tensors: dict = field(default_factory=dict)   # name -> np.ndarray f32 (insertion ordered)
    ops: list = field(default_factory=list)       # (kind, name, [inputs], output, attr0)

    def tensor(self, name: str, arr) -> str:
        self.tensors[name] = np.ascontiguousarray(np.asarray(arr, dtype=np.float32))
        return name

    def op(self, kind: int, name: str, inputs: list, output: str, attr0: int = 0) -> str:
        self.ops.append((kind, name, list(inputs), output, attr0))
        return output

    @property
    def output_name(self) -> str:
        return self.ops[-1][3] if self.ops else self.input_name

    def smf_offsets(self) -> dict:
        """name -> absolute file offset of each constant tensor's f32 blob."""
        return self._layout()[1]

    def _meta(self, offsets: dict) -> bytes:
        version = 4 if self.token_input else 3
        out = struct.pack("<IIII", SMF_MAGIC, version, len(self.tensors) + 1, len(self.ops))
        out += _s(self.input_name) + _s(self.output_name) + struct.pack("<Q", self.seq_len)
        dims = [-1] if self.token_input else [-1, self.input_dim]
        out += _s(self.input_name) + struct.pack("<BB", len(dims), 0)
        for d in dims:
            out += struct.pack("<q", d)
        out += struct.pack("<QQ", 0, 0)
        for name, arr in self.tensors.items():
            out += _s(name) + struct.pack("<BB", arr.ndim, 1)
            for d in arr.shape:
                out += struct.pack("<q", d)
            out += struct.pack("<QQ", offsets.get(name, 0), arr.nbytes)
        for kind, name, inputs, output, attr0 in self.ops:
            out += struct.pack("<B", kind) + _s(name) + struct.pack("<B", len(inputs))
            for i in inputs:
                out += _s(i)
            out += _s(output) + struct.pack("<I", attr0)
        return out

    def _layout(self):
        cursor, offsets = align_up(len(self._meta({}))), {}
        for name, arr in self.tensors.items():
            offsets[name] = cursor
            cursor = align_up(cursor + arr.nbytes)
        return cursor, offsets

    def write_smf(self, path: str):
        total, offsets = self._layout()
        with open(path, "wb") as f:
            meta = self._meta(offsets)
            f.write(meta)
            pos = len(meta)
            for name, arr in self.tensors.items():
                f.write(b"\0" * (offsets[name] - pos))
                f.write(arr.tobytes())
                pos = offsets[name] + arr.nbytes
            f.write(b"\0" * (total - pos))

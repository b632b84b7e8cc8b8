"""Deterministic fuzz arm over the attacker / corruption-facing parsers of the host side:
the SEEU plan admission (`seeml_b200_plan_verify`, what `engine_load_*` runs before any
device work) and the SDS corpus reader (`seeml_b200_dataset_load`). Modelled on the
reference's libFuzzer harness (test/fuzz/binary_formats.cc:1-115, arms [1] and [2]): hostile
bytes may be REJECTED but must never crash, hang or over-read, every refusal must carry a
diagnostic attributable to a registered unit, and - because the integrity hash would stop
nearly every mutation at the first gate - plans are resealed with PlanSelfHash the way the
reference harness reseals them, so the section / instruction / bounds validators underneath
are what gets attacked. Where the reference build is present the verdict (accept / reject)
on every resealed plan must also equal the reference loader's."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

import plancases
from oracle import pyoracle as O
from see_ml_b200 import _lib as L
from see_ml_b200 import formats as F

UNITS = ("UpdateEngine: ", "PlanValidator: ", "Dataset: ", "BatchPipeline: ", "DurableIO: ", "Checkpoint: ")
HASH_AT = 216
EDGE_U64 = [0, 1, 2, 63, 64, 65, 280, (1 << 31) - 1, 1 << 31, (1 << 32) - 1, 1 << 32, 1 << 40, (1 << 63) - 1,
            1 << 63, (1 << 63) + 64, (1 << 64) - 64, (1 << 64) - 1]


def _attributable(msg: str) -> bool:
    return any(msg.startswith(u) and len(msg) > len(u) for u in UNITS)


def _reseal(lib, b: bytearray):
    if len(b) >= 280:
        a = np.frombuffer(bytes(b), np.uint8)
        h = int(lib.seeml_b200_plan_self_hash(a.ctypes.data, a.size, HASH_AT))
        b[HASH_AT:HASH_AT + 8] = struct.pack("<Q", h)
    return b


def _mutate_plan(rng, blob: bytes, plan) -> bytearray:
    b = bytearray(blob)
    h = plan.header
    kind = int(rng.integers(0, 9))
    if kind == 0:                                     # a header u64 field gets an edge value
        off = int(rng.choice([8, 16, 24, 32, 40, 48, 64, 72, 80, 88, 96, 104, 112, 120, 128, 136, 144, 176, 184, 192,
                              200, 232, 256]))
        v = int(rng.choice(len(EDGE_U64) + 3))
        val = EDGE_U64[v] if v < len(EDGE_U64) else [len(b), len(b) + 1, len(b) - 1][v - len(EDGE_U64)]
        b[off:off + 8] = struct.pack("<Q", val & ((1 << 64) - 1))
    elif kind == 1:                                   # a header u32 field
        off = int(rng.choice([4, 56, 60, 224, 248]))
        b[off:off + 4] = struct.pack("<I", int(rng.choice([0, 1, 2, 3, 4, 5, 6, 7, 8, 255, 0xFFFFFFFF])))
    elif kind in (2, 3, 4):                           # one instruction word of one of the three programs
        progs = [(h.train_instr_offset, h.train_instr_count), (h.merge_instr_offset, h.merge_instr_count),
                 (h.eval_instr_offset, h.eval_instr_count)]
        off0, cnt = progs[int(rng.integers(0, 3))]
        if cnt:
            at = off0 + 64 * int(rng.integers(0, cnt))
            what = int(rng.integers(0, 4))
            if what == 0:
                b[at:at + 2] = struct.pack("<H", int(rng.choice([0, 41, 42, 43, 255, 65535, int(rng.integers(0, 42))])))
            elif what == 1:
                b[at + 2:at + 4] = struct.pack("<H", int(rng.choice([1, 2, 4, 6, 7, 8, 0x8000, 0xFFFF])))
            else:
                word = at + 8 + 8 * int(rng.integers(0, 7))
                old = struct.unpack("<Q", b[word:word + 8])[0]
                val = int(rng.choice(len(EDGE_U64) + 5))
                new = EDGE_U64[val] if val < len(EDGE_U64) else [old + 4, old ^ (1 << 63), old * 2 + 64, old + 1,
                                                                h.arena_size - 4][val - len(EDGE_U64)]
                b[word:word + 8] = struct.pack("<Q", new & ((1 << 64) - 1))
    elif kind == 5:                                   # truncate or extend
        n = int(rng.integers(0, len(b) + 1)) if rng.random() < 0.7 else len(b) + int(rng.integers(1, 200))
        b = bytearray(b[:n]) if n <= len(b) else b + bytearray(n - len(b))
    elif kind == 6:                                   # random byte noise anywhere
        for _ in range(int(rng.integers(1, 8))):
            b[int(rng.integers(0, len(b)))] = int(rng.integers(0, 256))
    elif kind == 7:                                   # an emit-table entry
        if h.emit_count:
            at = h.emit_table_offset + 24 * int(rng.integers(0, h.emit_count)) + 8 * int(rng.integers(0, 3))
            b[at:at + 8] = struct.pack("<Q", EDGE_U64[int(rng.integers(0, len(EDGE_U64)))])
    else:                                             # swap two sections' offsets
        offs = [72, 88, 104, 120, 136, 192]
        i, j = rng.choice(len(offs), 2, replace=False)
        a_, b_ = bytes(b[offs[i]:offs[i] + 8]), bytes(b[offs[j]:offs[j] + 8])
        b[offs[i]:offs[i] + 8], b[offs[j]:offs[j] + 8] = b_, a_
    return b


def test_hostile_plans_are_refused_never_crash_and_match_the_reference_verdict(golden_dir, backend_lib):
    lib = backend_lib
    z = np.load(os.path.join(golden_dir, "plans.npz"))
    rng = np.random.default_rng(20240611)
    have_ref = O.have_ref()
    accepted = rejected = compared = 0
    for pc in plancases.plan_cases():
        blob = z[pc.name].tobytes()
        plan = F.parse_plan(blob)
        for it in range(900):
            b = _mutate_plan(rng, blob, plan)
            sealed = it % 8 != 0                      # one in eight stays unsealed: the hash gate itself
            if sealed:
                b = _reseal(lib, b)
            a = np.frombuffer(bytes(b), np.uint8)
            rc = lib.seeml_b200_plan_verify(a.ctypes.data if a.size else None, a.size)
            if rc == 0:
                accepted += 1
            else:
                rejected += 1
                assert _attributable(L.last_error()), (pc.name, it, L.last_error())
            # differential arm: the reference loader on the same bytes (it allocates the arena the
            # header names, so only plans with a modest arena are handed over)
            if have_ref and a.size >= 280 and struct.unpack("<Q", bytes(b[8:16]))[0] <= (1 << 26):
                ref = O.ref()
                e = ref.ref_engine_new()
                err = C.create_string_buffer(512)
                rrc = ref.ref_engine_load_memory(e, a.ctypes.data, a.size, err, 512)
                ref.ref_engine_free(e)
                assert (rrc == 0) == (rc == 0), (pc.name, it, L.last_error(), err.value.decode())
                compared += 1
    assert rejected > 1500 and accepted > 50, (accepted, rejected)
    if have_ref:
        assert compared > 1500


def _sds_seeds(tmp_path):
    rng = np.random.default_rng(5)
    p1, p2, p3 = (str(tmp_path / n) for n in ("a.sds", "b.sds", "c.sds"))
    F.write_sds(p1, rng.standard_normal((9, 5)).astype(np.float32), rng.integers(0, 4, 9).astype(np.int32))
    F.write_sds(p2, rng.standard_normal((7, 3)).astype(np.float32), rng.standard_normal((7, 2)).astype(np.float32),
                label_kind=2)
    F.write_token_sds(p3, rng.integers(0, 50, (6, 9)).astype(np.int32))
    return [open(p, "rb").read() for p in (p1, p2, p3)]


def test_hostile_corpora_are_refused_never_crash(tmp_path, backend_lib):
    lib = backend_lib
    rng = np.random.default_rng(77)
    path = str(tmp_path / "fuzz.sds")
    loaded = refused = 0
    for seed in _sds_seeds(tmp_path):
        for it in range(700):
            b = bytearray(seed)
            kind = int(rng.integers(0, 5))
            if kind == 0:
                off = int(rng.choice([8, 16, 32]))
                b[off:off + 8] = struct.pack("<Q", EDGE_U64[int(rng.integers(0, len(EDGE_U64)))])
            elif kind == 1:
                off = int(rng.choice([0, 4, 24, 28]))
                b[off:off + 4] = struct.pack("<I", int(rng.choice([0, 1, 2, 3, 4, 0x31534453, 0xFFFFFFFF])))
            elif kind == 2:
                b = b[:int(rng.integers(0, len(b) + 1))]
            elif kind == 3:
                for _ in range(int(rng.integers(1, 6))):
                    b[int(rng.integers(0, len(b)))] = int(rng.integers(0, 256))
            else:
                b += bytes(int(rng.integers(1, 64)))
            open(path, "wb").write(bytes(b))
            h = lib.seeml_b200_dataset_load(path.encode())
            if h:
                loaded += 1
                n, d = lib.seeml_b200_dataset_num_samples(h), lib.seeml_b200_dataset_input_dim(h)
                # an accepted corpus must be servable: one small batch into right-sized slots
                if 0 < n and 0 < d <= 64:
                    kind_in = lib.seeml_b200_dataset_input_kind(h)
                    rows = d if kind_in == 1 else 1
                    inp = np.zeros(max(rows * (1 if kind_in == 1 else d), 1) + 8, np.uint32)
                    lab = np.zeros(rows * max(lib.seeml_b200_dataset_label_bytes_per_sample(h), 4) + 64, np.uint8)
                    lib.seeml_b200_dataset_fill_batch(h, rows, inp.ctypes.data, lab.ctypes.data)
                lib.seeml_b200_dataset_free(h)
            else:
                refused += 1
                assert _attributable(L.last_error()), (it, L.last_error())
    assert refused > 500 and loaded > 100, (loaded, refused)


def test_a_missing_corpus_file_is_a_dataset_error(backend_lib, tmp_path):
    assert not backend_lib.seeml_b200_dataset_load(str(tmp_path / "absent.sds").encode())
    assert _attributable(L.last_error())

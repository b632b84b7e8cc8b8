"""Host-side logic of the backend against the golden fixtures (no GPU needed):
the plan synthesiser, the C ABI's hashes / validator / plan admission, and the
feeder's serving order. The library must load and export every declared symbol on
a machine without a GPU, and must refuse device work there instead of falling back."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import plancases
from see_ml_b200 import _lib as L
from see_ml_b200 import formats as F
from see_ml_b200 import plansynth as PS
from see_ml_b200.engine import Dataset


def _hasher(lib):
    return lambda b, o: int(lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o))


def test_abi_exports_every_declared_symbol(backend_lib):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = ""
    for fn in sorted(os.listdir(os.path.join(root, "include"))):
        if fn.endswith(".h"):
            text += open(os.path.join(root, "include", fn)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(seeml_b200_[a-z0-9_]+)\s*\(", text))
    assert len(declared) > 60
    for name in declared:
        assert hasattr(backend_lib, name), f"{name} declared in include/ but not exported"
        assert name in L.SIGNATURES, f"{name} has no ctypes signature"
    assert backend_lib.seeml_b200_abi_version() == 1


def test_no_cpu_fallback(backend_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    out = C.c_void_p()
    rc = backend_lib.seeml_b200_ctx_create(0, 4096, None, 0, None, 0, None, C.byref(out))
    assert rc != 0 and not out.value
    assert "no CUDA device" in L.last_error()
    assert not backend_lib.seeml_b200_engine_create(0, 0, 0)


def test_hashes_match_reference(golden_dir, backend_lib):
    m = json.load(open(os.path.join(golden_dir, "misc.json")))["misc"]["hash"]
    for n_s, want in m.items():
        n = int(n_s)
        buf = np.random.default_rng(n).integers(0, 256, n, dtype=np.uint8)
        p = buf.ctypes.data if n else None
        assert backend_lib.seeml_b200_content_hash64(p, n) == int(want["content"])
        assert backend_lib.seeml_b200_plan_self_hash(p, n, 216) == int(want["self216"])


def test_validator_verdicts_match_reference(golden_dir, backend_lib):
    want = {v["name"]: v for v in json.load(open(os.path.join(golden_dir, "misc.json")))["misc"]["validator"]}
    cases = plancases.validator_cases()
    assert {c["name"] for c in cases} == set(want)
    for c in cases:
        rc = backend_lib.seeml_b200_validate_instruction(c["instr"].ctypes.data, c["arena"], c["rodata"],
                                                         c["version"])
        assert (rc == 0) == bool(want[c["name"]]["accepted"]), c["name"]
        if rc:
            assert L.last_error() == want[c["name"]]["message"], c["name"]


@pytest.mark.parametrize("pc", plancases.plan_cases(), ids=lambda p: p.name)
def test_synthesised_plan_is_byte_identical_to_reference_compiler(golden_dir, backend_lib, pc, tmp_path):
    z = np.load(os.path.join(golden_dir, "plans.npz"))
    smf = str(tmp_path / "m.smf")
    pc.model.write_smf(smf)
    raw = np.fromfile(smf, np.uint8)
    pc.spec.source_model_hash = int(backend_lib.seeml_b200_content_hash64(raw.ctypes.data, raw.size))
    blob, info = PS.synthesize(pc.model, pc.spec, hasher=_hasher(backend_lib))
    assert blob == z[pc.name].tobytes()
    assert backend_lib.seeml_b200_plan_verify(np.frombuffer(blob, np.uint8).ctypes.data, len(blob)) == 0
    assert len(info.params) == 2 * len(info.adapters)


def test_plan_admission_rejects_what_the_reference_rejects(golden_dir, backend_lib):
    """Load hardening (reference: test/runtime/engine/update_engine_test.cc:84-195):
    truncation, bad magic, versions outside the readable window, a flipped byte, a
    section out of bounds, an unknown opcode and an out-of-bounds operand (resealed)."""
    z = np.load(os.path.join(golden_dir, "plans.npz"))
    blob = z["llama_tiny"].tobytes()
    verify = lambda b: backend_lib.seeml_b200_plan_verify(np.frombuffer(b, np.uint8).ctypes.data, len(b))
    assert verify(blob) == 0
    assert verify(blob[:100]) != 0 and "smaller than its header" in L.last_error()
    bad = bytearray(blob); bad[0] ^= 0xFF
    assert verify(bytes(bad)) != 0 and "bad plan magic" in L.last_error()
    bad = bytearray(blob); bad[5000] ^= 0x01
    assert verify(bytes(bad)) != 0 and "plan hash mismatch" in L.last_error()
    assert verify(blob[:-8]) != 0

    def reseal(mutate):
        p = F.parse_plan(blob)
        mutate(p)
        return F.assemble_plan(p.header, p.train, p.merge, p.eval, np.asarray(p.rodata),
                               np.asarray(p.persist_init), p.emit, hasher=_hasher(backend_lib))
    for v in (3, 8):
        b = reseal(lambda p: setattr(p.header, "version", v))
        assert verify(b) != 0 and "unsupported plan version" in L.last_error()

    def unknown_op(p): p.train["opcode"][3] = 99
    assert verify(reseal(unknown_op)) != 0 and "unknown opcode 99" in L.last_error()

    def oob(p):
        i = int(np.nonzero(p.train["opcode"] == int(F.Op.GEMM_NN))[0][0])
        p.train["in"][i, 2] = p.header.arena_size - 4
    assert verify(reseal(oob)) != 0 and "out of bounds" in L.last_error()

    def labels_elsewhere(p):
        i = int(np.nonzero(p.train["opcode"] == int(F.Op.XENT_FWD))[0][0])
        p.train["in"][i, 1] = p.header.input_ref
    assert verify(reseal(labels_elsewhere)) != 0 and "staged label slot" in L.last_error()

    def tokens_elsewhere(p):
        i = int(np.nonzero(p.train["opcode"] == int(F.Op.EMBED))[0][0])
        p.train["in"][i, 0] = p.header.label_ref
    assert verify(reseal(tokens_elsewhere)) != 0 and "staged input slot" in L.last_error()
    assert verify(reseal(lambda p: setattr(p.header, "batch", 0))) != 0


def test_feeder_serving_is_bit_exact(golden_dir, backend_lib):
    z = np.load(os.path.join(golden_dir, "feeder.npz"))
    x, y = z["f32/x"], z["f32/y"]
    cat = lambda ab: np.concatenate([ab[0].view(np.uint8), ab[1]])
    d = Dataset.from_memory(x, y)
    np.testing.assert_array_equal(np.stack([cat(d.fill_batch(8, 40, 32)) for _ in range(7)]),
                                  z["f32/sequential"])
    d.enable_shuffle(12345)
    np.testing.assert_array_equal(np.stack([cat(d.fill_batch(8, 40, 32)) for _ in range(9)]),
                                  z["f32/shuffled_seed12345"])
    d2 = Dataset.from_memory(x, y)
    v = d2.split_validation(0.3)
    assert [d2.num_samples(), v.num_samples()] == list(z["f32/split_sizes"])
    np.testing.assert_array_equal(cat(v.fill_batch(4, 20, 16)), z["f32/val_first"])
    t = Dataset.from_tokens(z["tok/records"])
    t.enable_shuffle(0)
    served = np.stack([cat(t.fill_batch(18, 18, 72)) for _ in range(8)])
    np.testing.assert_array_equal(served, z["tok/shuffled_seed0"])
    # token view: labels are the inputs shifted by one position within each record
    first = served[0]
    toks, labs = first[:72].view(np.int32).reshape(3, 6), first[72:].view(np.int32).reshape(3, 6)
    np.testing.assert_array_equal(toks[:, 1:], labs[:, :-1])
    t2 = Dataset.from_tokens(z["tok/records"])
    t2.enable_shuffle(3)
    t2.skip_served(18 * 5)
    np.testing.assert_array_equal(cat(t2.fill_batch(18, 18, 72)), z["tok/after_skip_5_batches_seed3"])


def test_dataset_file_round_trip_and_rejections(backend_lib, tmp_path):
    rng = np.random.default_rng(5)
    x, y = rng.standard_normal((9, 4)).astype(np.float32), rng.integers(0, 3, 9).astype(np.int32)
    p = str(tmp_path / "a.sds")
    F.write_sds(p, x, y)
    d = Dataset.load_from_file(p)
    assert d.num_samples() == 9
    inp, lab = d.fill_batch(9, 36, 36)
    np.testing.assert_array_equal(inp.view(np.float32).reshape(9, 4), x)
    np.testing.assert_array_equal(lab.view(np.int32), y)
    q = str(tmp_path / "b.sds")
    d.save_to_file(q)
    assert open(p, "rb").read() == open(q, "rb").read()
    toks = rng.integers(0, 20, (5, 9)).astype(np.int32)
    pt = str(tmp_path / "t.sds")
    F.write_token_sds(pt, toks)
    t = Dataset.load_from_file(pt)
    inp, lab = t.fill_batch(16, 16, 64)
    np.testing.assert_array_equal(inp.view(np.int32).reshape(2, 8), toks[:2, :-1])
    np.testing.assert_array_equal(lab.view(np.int32).reshape(2, 8), toks[:2, 1:])
    with pytest.raises(L.BackendError, match="outside"):
        t.validate_class_labels(10)
    raw = open(p, "rb").read()
    for bad, msg in ((raw[:20], "truncated header"), (b"XXXX" + raw[4:], "bad magic"),
                     (raw[:-7], "exceeds file size")):
        open(q, "wb").write(bad)
        with pytest.raises(L.BackendError, match=msg):
            Dataset.load_from_file(q)
    with pytest.raises(L.BackendError, match="negative token"):
        Dataset.from_tokens(np.array([[1, -2, 3]], np.int32))
    with pytest.raises(L.BackendError, match="validation fraction"):
        d.split_validation(1.5)


def test_data_parallel_entry_points_refuse_bad_arguments_with_attributable_errors(backend_lib):
    """The communicator layer binds NCCL at run time and never aborts: a rank outside the world,
    a missing id, a step on an engine that was never configured - each is an error string with
    a registered unit, with or without a GPU in the machine."""
    import ctypes as C
    lib = backend_lib
    raw = (C.c_uint8 * 128)()
    out = C.c_void_p()
    assert lib.seeml_b200_comm_init(0, raw, 3, 2, C.byref(out)) != 0
    assert L.last_error().startswith("UpdateEngine: rank / world size out of range")
    assert lib.seeml_b200_comm_init(0, None, 0, 1, C.byref(out)) != 0
    assert L.last_error().startswith("UpdateEngine: ")
    assert lib.seeml_b200_comm_unique_id(None) != 0 and L.last_error().startswith("UpdateEngine: ")
    assert lib.seeml_b200_engine_dp_configure(None, 8, 0, 1, None) != 0
    assert L.last_error() == "UpdateEngine: no plan loaded"
    loss = C.c_float()
    assert lib.seeml_b200_engine_dp_step_host(None, raw, raw, C.byref(loss)) != 0
    assert "not configured" in L.last_error()
    assert lib.seeml_b200_comm_rank(None) == 0 and lib.seeml_b200_comm_world(None) == 1
    lib.seeml_b200_comm_destroy(None)

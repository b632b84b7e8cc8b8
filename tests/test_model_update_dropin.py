"""The reference's generated `model_update` driver, unmodified, on this backend.

The reference's compiler packages a plan as update_plan_embedded.cc + update_main.cc (the
driver: LoadFromMemory -> VerifySourceModel -> Dataset::LoadFromFile -> SplitValidation ->
EnableShuffle -> Train -> gate -> RunMerge -> CommitToModel, exit codes 0 / 1 / 2 / 3;
compiler/backend/trainer/native_emitter.cc:92-326) and links it with its CPU runtime. Here
the same two generated files - emitted at test time by the reference's own emitter, compiled
into the parity checker - are compiled against include/seeml_compat (the reference's class
names over the C ABI) and linked with libseeml_b200.so instead. Nothing is edited."""
import os
import subprocess

import numpy as np
import pytest

import plancases
from oracle import pyoracle as O
from see_ml_b200 import _lib as L
from see_ml_b200 import formats as F
from see_ml_b200 import plansynth as PS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
needs_ref = pytest.mark.skipif(not O.have_ref(), reason="the reference build (oracle/_ref) is not present")


def _package(tmp_path, pc, labels=None, tokens=None):
    """model.smf, corpus.sds, a plan bound to the model's hash, and the built driver."""
    lib = L.lib()
    smf = str(tmp_path / "model.smf")
    pc.model.write_smf(smf)
    raw = np.fromfile(smf, np.uint8)
    pc.spec.source_model_hash = int(lib.seeml_b200_content_hash64(raw.ctypes.data, raw.size))
    blob, info = PS.synthesize(pc.model, pc.spec, hasher=lambda b, o: int(
        lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o)))
    sds = str(tmp_path / "corpus.sds")
    if pc.corpus_tokens is not None:
        F.write_token_sds(sds, pc.corpus_tokens if tokens is None else tokens)
    else:
        F.write_sds(sds, pc.corpus_x, pc.corpus_y if labels is None else labels)
    pkg = tmp_path / "pkg"
    # no checkout is handed to the emitter, so it writes its generated sources and stops before
    # vendoring the CPU runtime (whose headers would otherwise shadow include/seeml_compat)
    err = O.ref_emit_native_package(blob, str(pkg), None)
    assert "cannot vendor" in err
    main, emb = pkg / "update_main.cc", pkg / "update_plan_embedded.cc"
    assert main.exists() and emb.exists(), "the reference emitter did not write the generated sources"
    exe = str(pkg / "model_update")
    libdir = os.path.join(ROOT, "see_ml_b200")
    subprocess.run(["g++", "-std=c++23", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                    "-I", os.path.join(ROOT, "include", "seeml_compat"), str(main), str(emb),
                    "-L", libdir, "-lseeml_b200", f"-Wl,-rpath,{libdir}", "-o", exe], check=True)
    return exe, smf, sds, blob, info


def _run(exe, *args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([exe, *args], capture_output=True, text=True, env=e, timeout=600)


@needs_ref
def test_generated_driver_builds_unmodified_and_keeps_its_argument_contract(tmp_path):
    pc = next(p for p in plancases.plan_cases() if p.name == "mlp_tiny")
    exe, smf, sds, _, _ = _package(tmp_path, pc)
    r = _run(exe, "--help")
    assert r.returncode == 0 and r.stdout.startswith("usage: model_update")
    assert _run(exe, "--modle", smf).returncode == 2
    assert _run(exe, "--model", smf, "--data", sds, "--steps", "x").returncode == 2
    assert _run(exe, "--model", smf).returncode == 2


@needs_ref
def test_generated_driver_reports_a_missing_gpu_as_a_load_error(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    pc = next(p for p in plancases.plan_cases() if p.name == "mlp_tiny")
    exe, smf, sds, _, _ = _package(tmp_path, pc)
    r = _run(exe, "--model", smf, "--data", sds)
    assert r.returncode == 1 and "load: UpdateEngine: no CUDA device" in r.stderr


def _python_path(blob, sds, smf, out, steps, seed, val_frac, mode):
    from see_ml_b200.engine import Dataset, UpdateEngine
    e = UpdateEngine(0, mode, 1)
    e.load_from_memory(blob)
    ds = Dataset.load_from_file(sds)
    val = ds.split_validation(val_frac)
    ds.enable_shuffle(seed)
    res = e.train(ds, steps, validation=val)
    if res.improved:
        e.run_merge()
        e.commit_to_model(smf, out)
    e.close()
    return res


@needs_ref
@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mlp_tiny", "llama_tiny"])
def test_model_update_trains_gates_merges_and_commits_like_the_python_path(tmp_path, name):
    pc = next(p for p in plancases.plan_cases() if p.name == name)
    exe, smf, sds, blob, _ = _package(tmp_path, pc)
    out, log = str(tmp_path / "updated.smf"), str(tmp_path / "curve.csv")
    r = _run(exe, "--model", smf, "--data", sds, "--out", out, "--steps", "40", "--seed", "7", "--val-frac", "0.2",
             "--loss-log", log, env={"SEEML_B200_MODE": "fused", "SEEML_B200_GEMM": "f16x2"})
    assert r.returncode == 0, r.stderr
    assert "seeml-update: committed" in r.stderr and "validation loss" in r.stderr
    want_out = str(tmp_path / "updated_py.smf")
    res = _python_path(blob, sds, smf, want_out, 40, 7, 0.2, mode=1)
    assert res.improved
    np.testing.assert_array_equal(np.fromfile(out, np.uint8), np.fromfile(want_out, np.uint8))
    assert not np.array_equal(np.fromfile(out, np.uint8), np.fromfile(smf, np.uint8))
    rows = open(log).read().strip().split("\n")
    assert rows[0] == "step,loss" and len(rows) == 41
    got_curve = np.array([float(x.split(",")[1]) for x in rows[1:]])
    np.testing.assert_allclose(got_curve, res.loss_curve, atol=1e-6)
    # against the reference runtime on the same files: same gate verdict, loss curve within 0.5 %
    e = O.RefEngine(blob)
    ds = O.RefDataset.load(sds)
    val = ds.split_validation(0.2)
    ds.enable_shuffle(7)
    ref_curve, rep = e.train(ds, 40, validation=val)
    assert rep.improved == 1
    np.testing.assert_allclose(got_curve, ref_curve, rtol=5e-3, atol=1e-5)


@needs_ref
@pytest.mark.gpu
def test_model_update_rejected_gate_exits_3_and_leaves_no_model(tmp_path):
    pc = next(p for p in plancases.plan_cases() if p.name == "mlp_tiny")
    labels = np.random.default_rng(1).integers(0, 6, 80).astype(np.int32)    # nothing to learn: validation gets worse
    exe, smf, sds, blob, _ = _package(tmp_path, pc, labels=labels)
    out = str(tmp_path / "updated.smf")
    r = _run(exe, "--model", smf, "--data", sds, "--out", out, "--steps", "200", "--seed", "7", "--val-frac", "0.3")
    assert r.returncode == 3, r.stderr
    assert "REJECTED" in r.stderr and not os.path.exists(out)
    r = _run(exe, "--model", smf, "--data", sds, "--out", out, "--steps", "200", "--seed", "7", "--val-frac", "0.3",
             "--force")
    assert r.returncode == 0 and os.path.exists(out)
    # a model file other than the one the plan was compiled from is refused before training
    other = str(tmp_path / "other.smf")
    raw = np.fromfile(smf, np.uint8)
    raw[-1] ^= 1
    raw.tofile(other)
    r = _run(exe, "--model", other, "--data", sds, "--out", out)
    assert r.returncode == 1 and "model: UpdateEngine: source model does not match" in r.stderr

"""Whole-plan parity on the GPU, through the engine's C ABI: reference-compiled plans
(golden fixtures) executed by the CUDA backend against the reference engine's own
results, plus the engine lifecycle the reference's tests pin (checkpoint / resume
bitwise, evaluation without side effects, merge -> commit, gate metrics, LR schedule,
cancellation, non-finite abort)."""
import json
import os

import numpy as np
import pytest

import plancases
from oracle import pyoracle as O
from see_ml_b200 import _lib as L
from see_ml_b200 import formats as F

pytestmark = pytest.mark.gpu

TOL = dict(rtol=1e-3, atol=1e-4)


def _engine(blob, mode=0, gemm=0):
    from see_ml_b200.engine import UpdateEngine
    e = UpdateEngine(0, mode, gemm)
    e.load_from_memory(blob)
    return e


def _golden(golden_dir):
    return np.load(os.path.join(golden_dir, "plans.npz")), \
        json.load(open(os.path.join(golden_dir, "misc.json")))["plans"]


@pytest.mark.parametrize("pc", plancases.plan_cases(), ids=lambda p: p.name)
def test_every_arena_tensor_after_one_step_matches_oracle(golden_dir, pc):
    """Step-0 identity and gradients: feed one batch by hand, execute the train stream
    once, and compare the WHOLE arena with the C oracle's (every activation, cached
    statistic, gradient, moment and parameter; int slots bit-exact)."""
    z, _ = _golden(golden_dir)
    blob = z[pc.name].tobytes()
    plan = F.parse_plan(blob)
    h = plan.header
    e = _engine(blob)
    inp, lab = pc.first_batch()
    e.arena_write(h.input_ref, inp)
    e.arena_write(h.label_ref, lab)
    e.execute_train_once()
    got = e.arena_read(0, h.arena_size)
    want = np.zeros(F.align_up(h.arena_size), np.uint8)
    want[:h.persist_init_size] = plan.persist_init
    want[h.input_ref:h.input_ref + inp.nbytes] = inp.view(np.uint8)
    want[h.label_ref:h.label_ref + lab.nbytes] = lab.view(np.uint8)
    lr = O.port().orc_effective_lr(h.lr, h.lr_schedule, h.warmup_steps, h.default_steps, h.min_lr_factor, 1)
    O.execute("port", plan.train, want, np.asarray(plan.rodata), lr=lr, b1=h.beta1, b2=h.beta2, eps=h.eps,
              wd=h.weight_decay, step=1)
    want = want[:h.arena_size]
    # token / label slots are integers: bit-exact
    np.testing.assert_array_equal(got[h.input_ref:h.input_ref + inp.nbytes], inp.view(np.uint8))
    np.testing.assert_array_equal(got[h.label_ref:h.label_ref + lab.nbytes], lab.view(np.uint8))
    g, w = got.view(np.float32), want.view(np.float32)
    io = np.zeros(g.size, bool)
    io[h.input_ref // 4:(h.input_ref + inp.nbytes) // 4] = True
    io[h.label_ref // 4:(h.label_ref + lab.nbytes) // 4] = True
    fin = np.isfinite(w) & ~io
    np.testing.assert_allclose(g[fin], w[fin], **TOL)
    assert abs(e.loss_value() - float(z[pc.name + "/step1_loss"][0])) <= 1e-4
    # the persistent segment (adapters + AdamW moments) against the reference engine itself
    np.testing.assert_allclose(got[:h.persistent_size].view(np.float32),
                               z[pc.name + "/step1_persistent"].view(np.float32), **TOL)


@pytest.mark.parametrize("pc", plancases.plan_cases(), ids=lambda p: p.name)
def test_training_run_matches_reference_engine(golden_dir, pc):
    """Same corpus, split, shuffle seed and step count as the reference run that made the
    fixture: loss curve within 0.5 % at every step, gate metrics, merged deltas."""
    z, meta = _golden(golden_dir)
    e = _engine(z[pc.name].tobytes())
    ds = pc.dataset()
    val = ds.split_validation(0.25)
    ds.enable_shuffle(7)
    res = e.train(ds, pc.steps, validation=val)
    want = z[pc.name + "/curve"]
    assert res.steps == len(want) == meta[pc.name]["steps"]
    np.testing.assert_allclose(res.loss_curve, want, rtol=5e-3)
    m = meta[pc.name]
    assert abs(res.val_initial_loss - m["val_initial_loss"]) <= 5e-3 * abs(m["val_initial_loss"])
    assert abs(res.val_final_loss - m["val_final_loss"]) <= 5e-3 * abs(m["val_final_loss"])
    assert res.has_val_accuracy == bool(m["has_val_accuracy"])
    assert abs(res.val_initial_accuracy - m["val_initial_accuracy"]) <= 0.051
    assert res.improved == bool(m["improved"])
    assert abs(res.initial_avg_loss - m["initial_avg_loss"]) <= 5e-3 * m["initial_avg_loss"]
    h = e.header
    np.testing.assert_allclose(e.arena_read(0, h.persistent_size).view(np.float32),
                               z[pc.name + "/final_persistent"].view(np.float32), rtol=2e-2, atol=2e-4)
    e.run_merge()
    em = F.parse_plan(z[pc.name].tobytes()).emit
    deltas = np.concatenate([e.arena_read(int(x["arena_offset"]), int(x["byte_size"])) for x in em])
    np.testing.assert_allclose(deltas.view(np.float32), z[pc.name + "/deltas"].view(np.float32),
                               rtol=2e-2, atol=2e-4)


def test_runs_are_bit_reproducible_and_mode_independent(golden_dir):
    z, _ = _golden(golden_dir)
    pc = next(p for p in plancases.plan_cases() if p.name == "llama_tiny")
    outs = []
    for mode in (0, 0, 1):
        e = _engine(z[pc.name].tobytes(), mode=mode)
        ds = pc.dataset()
        ds.enable_shuffle(3)
        res = e.train(ds, 12)
        outs.append((res.loss_curve.copy(), e.arena_read(0, e.header.persistent_size)))
    np.testing.assert_array_equal(outs[0][0], outs[1][0])
    np.testing.assert_array_equal(outs[0][1], outs[1][1])
    # fused execution may reorder arithmetic: tolerance, not bits
    np.testing.assert_allclose(outs[2][0], outs[0][0], rtol=5e-3)


def test_checkpoint_resume_is_bitwise_equal_to_uninterrupted(golden_dir, tmp_path):
    z, _ = _golden(golden_dir)
    pc = next(p for p in plancases.plan_cases() if p.name == "gpt_tiny")
    blob = z[pc.name].tobytes()
    a = _engine(blob)
    da = pc.dataset(); da.enable_shuffle(11)
    ra = a.train(da, 20)
    ck = str(tmp_path / "state.sekp")
    b = _engine(blob)
    db = pc.dataset(); db.enable_shuffle(11)
    b.train(db, 9, checkpoint_path=ck, checkpoint_every=9)
    c = _engine(blob)
    dc = pc.dataset(); dc.enable_shuffle(11)
    rc = c.train(dc, 11, checkpoint_path=ck, resume=True)
    assert c.step() == 20
    np.testing.assert_array_equal(rc.loss_curve, ra.loss_curve[9:])
    np.testing.assert_array_equal(c.arena_read(0, c.header.persistent_size),
                                  a.arena_read(0, a.header.persistent_size))
    # a foreign or corrupt checkpoint is refused and leaves the state alone
    other = _engine(z["llama_tiny"].tobytes())
    with pytest.raises(L.BackendError, match="different plan"):
        other.load_checkpoint(ck)
    raw = bytearray(open(ck, "rb").read()); raw[-1] ^= 1
    open(ck, "wb").write(raw)
    with pytest.raises(L.BackendError, match="corrupt"):
        c.load_checkpoint(ck)


def test_evaluate_is_side_effect_free_and_accuracy_is_exact(golden_dir):
    z, _ = _golden(golden_dir)
    pc = next(p for p in plancases.plan_cases() if p.name == "mlp_tiny")
    e = _engine(z[pc.name].tobytes())
    ds = pc.dataset()
    before = e.arena_read(0, e.header.persistent_size)
    l1, a1, has = e.evaluate_metrics(ds)
    l2, a2, _ = e.evaluate_metrics(ds)
    assert has and (l1, a1) == (l2, a2)
    np.testing.assert_array_equal(before, e.arena_read(0, e.header.persistent_size))
    # reference engine on the same corpus
    if O.have_ref():
        r = O.RefEngine(z[pc.name].tobytes())
        lr, ar, _ = r.evaluate(pc.ref_dataset())
        assert abs(l1 - lr) <= 1e-4 and abs(a1 - ar) < 1e-6


def test_merge_then_commit_patches_w_plus_delta(golden_dir, tmp_path):
    """train -> merge (delta = (alpha/r) A@B to 1e-4) -> commit (patched == orig + delta
    exactly); commit before merge is refused (reference: update_system_test.cc:218-304)."""
    pc = next(p for p in plancases.plan_cases() if p.name == "mlp_tiny")
    smf = str(tmp_path / "model.smf")
    pc.model.write_smf(smf)
    raw = np.fromfile(smf, np.uint8)
    from see_ml_b200 import plansynth as PS
    lib = L.lib()
    pc.spec.source_model_hash = int(lib.seeml_b200_content_hash64(raw.ctypes.data, raw.size))
    blob, info = PS.synthesize(pc.model, pc.spec, hasher=lambda b, o: int(
        lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o)))
    e = _engine(blob)
    e.verify_source_model(smf)
    ds = pc.dataset()
    e.train(ds, 15)
    out = str(tmp_path / "patched.smf")
    with pytest.raises(L.BackendError, match="RunMerge"):
        e.commit_to_model(smf, out)
    e.run_merge()
    for ad in info.adapters:
        A = e.arena_read(ad["a_ref"], ad["k"] * ad["r"] * 4).view(np.float32).reshape(ad["k"], ad["r"])
        B = e.arena_read(ad["b_ref"], ad["r"] * ad["m"] * 4).view(np.float32).reshape(ad["r"], ad["m"])
        d = e.arena_read(ad["delta_ref"], ad["k"] * ad["m"] * 4).view(np.float32).reshape(ad["k"], ad["m"])
        np.testing.assert_allclose(d, ad["scale"] * (A.astype(np.float64) @ B), atol=1e-4)
        assert np.abs(d).max() > 0
    e.commit_to_model(smf, out)
    patched = np.fromfile(out, np.uint8)
    offs = pc.model.smf_offsets()
    for ad in info.adapters:
        o = offs[ad["weight"]]
        n = ad["k"] * ad["m"] * 4
        d = e.arena_read(ad["delta_ref"], n).view(np.float32)
        np.testing.assert_array_equal(patched[o:o + n].view(np.float32), raw[o:o + n].view(np.float32) + d)
    other = str(tmp_path / "other.smf")
    raw2 = raw.copy(); raw2[-1] ^= 1; raw2.tofile(other)
    with pytest.raises(L.BackendError, match="source_model_hash"):
        e.commit_to_model(other, out)
    e.train(ds, 1)      # training invalidates the merged deltas
    with pytest.raises(L.BackendError, match="RunMerge"):
        e.commit_to_model(smf, out)


def test_lr_schedule_cancellation_and_nonfinite_abort(golden_dir):
    z, _ = _golden(golden_dir)
    pc = next(p for p in plancases.plan_cases() if p.name == "mlp_fused")
    e = _engine(z[pc.name].tobytes())
    h = e.header
    port = O.port()
    for s in (0, 1, 5, 6, 17, 30, 31, 500):
        e.set_step(s)
        assert np.float32(e.effective_lr()) == np.float32(
            port.orc_effective_lr(h.lr, h.lr_schedule, h.warmup_steps, h.default_steps, h.min_lr_factor, s))
    e.set_step(0)
    ds = pc.dataset()
    calls = []
    res = e.train(ds, 10, should_stop=lambda: (calls.append(1), len(calls) > 4)[1])
    assert res.stopped_early and res.steps == 4 and e.step() == 4
    # the feeder must have un-consumed what it staged ahead: the next batch served is batch 4
    inp, _ = ds.fill_batch(h.batch, h.input_floats, h.label_bytes)
    ds2 = pc.dataset()
    for _ in range(4):
        ds2.fill_batch(h.batch, h.input_floats, h.label_bytes)
    np.testing.assert_array_equal(inp, ds2.fill_batch(h.batch, h.input_floats, h.label_bytes)[0])
    bad = pc.corpus_x.copy(); bad[3, 2] = np.inf
    from see_ml_b200.engine import Dataset
    with pytest.raises(L.BackendError, match="non-finite"):
        e.train(Dataset.from_memory(bad, pc.corpus_y), 5)


def test_dataset_contract_violations_are_refused(golden_dir):
    z, _ = _golden(golden_dir)
    from see_ml_b200.engine import Dataset
    e = _engine(z["llama_tiny"].tobytes())
    rng = np.random.default_rng(0)
    with pytest.raises(L.BackendError, match="feature rows"):
        e.train(Dataset.from_memory(rng.standard_normal((8, 4)).astype(np.float32), np.zeros(8, np.int32)), 1)
    with pytest.raises(L.BackendError, match="sequence length"):
        e.train(Dataset.from_tokens(rng.integers(0, 40, (4, 5)).astype(np.int32)), 1)
    with pytest.raises(L.BackendError, match="outside"):
        e.train(Dataset.from_tokens(rng.integers(0, 400, (4, 9)).astype(np.int32)), 1)
    m = _engine(z["mlp_tiny"].tobytes())
    with pytest.raises(L.BackendError, match="input width"):
        m.train(Dataset.from_memory(rng.standard_normal((8, 5)).astype(np.float32), np.zeros(8, np.int32)), 1)
    with pytest.raises(L.BackendError, match="outside"):
        m.train(Dataset.from_memory(rng.standard_normal((8, 12)).astype(np.float32), np.full(8, 6, np.int32)), 1)
    # a rejected re-load leaves the previous plan usable
    blob = bytearray(z["mlp_tiny"].tobytes()); blob[400] ^= 1
    with pytest.raises(L.BackendError, match="hash mismatch"):
        m.load_from_memory(bytes(blob))
    pc = next(p for p in plancases.plan_cases() if p.name == "mlp_tiny")
    assert m.train(pc.dataset(), 2).steps == 2


def test_fused_groups_match_contract_mode_and_oracle_on_tensor_core_shapes():
    """A decoder wide enough for the tensor-core GEMM and the LoRA group fusions (forward
    C' = [X|t].[W^T|aB^T]^T, backward dX = [p+][g|dt].[W|A]^T, rank-r kernels): every LoRA
    gradient and the loss after one hand-fed backward pass, fused vs one-kernel-per-
    instruction vs the C oracle. The geometry also takes the tensor-core attention kernels
    (scores + softmax in TMEM forward; dS from dP held in TMEM in fused mode). Adapters' B factors are made nonzero so every path carries
    signal."""
    from see_ml_b200 import plansynth as PS
    from see_ml_b200.engine import UpdateEngine
    lib = L.lib()
    rng = np.random.default_rng(11)
    V, D, H, Ff, S, T = 512, 256, 4, 512, 128, 1024     # 64-wide heads, S % 128 == 0: tensor-core attention
    model = PS.llama_decoder(V, D, H, Ff, 2, S, rng, std=0.05)
    spec = PS.TrainSpec(batch=T, lora_rank=16, lora_alpha=32.0,
                        targets=("wq", "wk", "wv", "wo", "w_up", "w_down"))
    blob, info = PS.synthesize(model, spec, hasher=lambda b, o: int(
        lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o)))
    plan = F.parse_plan(blob)
    h = plan.header
    recs = rng.integers(0, V, (T // S, S + 1)).astype(np.int32)
    tok, lab = recs[:, :-1].reshape(-1).copy(), recs[:, 1:].reshape(-1).copy()
    bvals = {ad["b_ref"]: (rng.standard_normal(ad["r"] * ad["m"]) * 0.05).astype(np.float32)
             for ad in info.adapters}
    opt_begin = int(np.nonzero(plan.train["opcode"] == int(F.Op.ADAMW))[0][0])
    want = np.zeros(F.align_up(h.arena_size), np.uint8)
    want[:h.persist_init_size] = plan.persist_init
    for ref, v in bvals.items():
        want[ref:ref + v.nbytes] = v.view(np.uint8)
    want[h.input_ref:h.input_ref + tok.nbytes] = tok.view(np.uint8)
    want[h.label_ref:h.label_ref + lab.nbytes] = lab.view(np.uint8)
    O.execute("port", plan.train[:opt_begin], want, np.asarray(plan.rodata))
    results = {}
    for mode in (0, 1):
        e = UpdateEngine(0, mode, 0)
        e.load_from_memory(blob)
        for ref, v in bvals.items():
            e.arena_write(ref, v)
        e.arena_write(h.input_ref, tok)
        e.arena_write(h.label_ref, lab)
        e.run_train_range(0, e.opt_begin())
        results[mode] = (e.loss_value(), {pid: e.arena_read(g, n * 4).view(np.float32) for pid, _, g, n in info.params},
                         e.last_launches())
        e.close()
    assert results[1][2] < results[0][2], "fused mode launched no fewer kernels: nothing was fused"
    wl = float(want[h.loss_ref:h.loss_ref + 4].view(np.float32)[0])
    for mode in (0, 1):
        assert abs(results[mode][0] - wl) <= 1e-4 * abs(wl)
        for pid, _, g, n in info.params:
            ref = want[g:g + n * 4].view(np.float32)
            np.testing.assert_allclose(results[mode][1][pid], ref, rtol=1e-3, atol=1e-4 * max(1.0, np.abs(ref).max()),
                                       err_msg=f"mode {mode} {pid}")


def test_hundred_step_loss_curve_on_tensor_core_shapes(golden_dir):
    """100 optimiser steps of a decoder that takes every tensor-core kernel (3xTF32 GEMMs with
    the LoRA tails, rank-16 factor kernels, attention with scores / dP held in TMEM), fed by
    the shuffled feeder: the loss at every step within 0.5 % of the reference runtime's curve
    (fixture made by tests/golden/make_tc_curve.py), in fused and in contract mode."""
    import json
    import os
    import tccase
    from see_ml_b200.engine import Dataset, UpdateEngine
    lib = L.lib()
    want = json.load(open(os.path.join(golden_dir, "tc_curve.json")))
    model, spec, toks = tccase.build()
    blob = tccase.plan(model, spec, lambda b, o: int(
        lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o)))
    for mode in (1, 0):
        e = UpdateEngine(0, mode, 0)
        e.load_from_memory(blob)
        ds = Dataset.from_tokens(toks)
        ds.enable_shuffle(7)
        res = e.train(ds, tccase.STEPS)
        assert res.steps == want["steps"] == tccase.STEPS
        np.testing.assert_allclose(res.loss_curve, want["curve"], rtol=5e-3, err_msg=f"mode {mode}")
        assert res.loss_curve[-1] < 0.7 * res.loss_curve[0]          # it actually learned
        assert abs(res.final_avg_loss - want["final_avg_loss"]) <= 5e-3 * want["final_avg_loss"]
        e.close()


def test_step_timing_split_accumulates_and_resets(golden_dir):
    """StepTimings (update_engine.h:84-89, ResetStepTimings :190): one sample per executed
    training stream, split at the loss-forward and first-optimiser boundaries; off by default;
    timed and untimed runs give the same bits."""
    z, _ = _golden(golden_dir)
    pc = next(p for p in plancases.plan_cases() if p.name == "llama_tiny")
    blob = z[pc.name].tobytes()
    e = _engine(blob, mode=1)
    ds = pc.dataset()
    e.train(ds, 3)
    assert e.step_timings() == (0, 0.0, 0.0, 0.0)
    e.enable_step_timing(True)
    e.train(ds, 5)
    steps, fwd, bwd, opt = e.step_timings()
    assert steps == 5 and fwd > 0 and bwd > 0 and opt > 0
    assert fwd + bwd + opt < 5.0          # seconds: five steps of a toy model
    e.reset_step_timings()
    assert e.step_timings() == (0, 0.0, 0.0, 0.0)
    e.enable_step_timing(False)
    timed = e.arena_read(0, e.header.persistent_size)
    plain = _engine(blob, mode=1)
    ds2 = pc.dataset()
    plain.train(ds2, 8)
    np.testing.assert_array_equal(timed, plain.arena_read(0, plain.header.persistent_size))


def test_larger_program_after_graph_capture_keeps_earlier_graphs_valid():
    """A context's captured range graphs hold the addresses of its scratch buffers; building a
    program that needs more scratch replaces those buffers, so the graphs must be dropped and
    recaptured, never replayed against freed memory."""
    import opcases
    from see_ml_b200.engine import Context
    from see_ml_b200.formats import Op
    rng = np.random.default_rng(12)
    rows, classes = 64, 40
    Lo = opcases.Layout()
    z = Lo.put(opcases._rn(rng, rows, classes))
    lab = Lo.put(rng.integers(0, classes, rows).astype(np.int32))
    loss, probs = Lo.out(1), Lo.out(rows * classes)
    tmp = [Lo.out(rows * classes) for _ in range(8)]
    big_rows = 4096
    z2 = Lo.put(opcases._rn(rng, big_rows, 8))
    lab2 = Lo.put(rng.integers(0, 8, big_rows).astype(np.int32))
    loss2, probs2 = Lo.out(1), Lo.out(big_rows * 8)
    arena, ro = Lo.done()
    I = opcases._ins
    prog = [I(Op.XENT_FWD, [z, lab, loss, probs], [rows, classes])]
    src = probs
    for t in tmp:                                         # a chain long enough to be graph-captured
        prog.append(I(Op.SCALE, [src, t, F.f32_bits(1.5)], [rows * classes]))
        src = t
    prog = np.concatenate(prog)
    ctx = Context(arena.size, ro)
    ctx.write(0, arena)
    pid = ctx.build(prog)
    outs = []
    for _ in range(3):                                    # direct run, capture, replay
        ctx.run(pid, 0, len(prog))
        outs.append(ctx.read(0, arena.size).copy())
    ctx.execute(I(Op.XENT_FWD, [z2, lab2, loss2, probs2], [big_rows, 8]))    # needs a larger loss scratch
    ctx.write(0, arena)
    ctx.run(pid, 0, len(prog))
    again = ctx.read(0, arena.size)
    ctx.close()
    np.testing.assert_array_equal(outs[0], outs[1])
    np.testing.assert_array_equal(outs[0], outs[2])
    np.testing.assert_array_equal(outs[0], again)

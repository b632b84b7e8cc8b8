"""GPU parity at the benchmark configurations' own shapes, against fixtures made by the
reference runtime (tests/golden/make_config_goldens.py): C1 / C2 / C3 loss curves through the
shuffled feeder in fused and contract mode, one 16384-row chunk of a two-layer slice of C4
(loss and every LoRA gradient), softmax cross-entropy at 32000 classes, the lm-head GEMM shape,
the MatMul / LoRA sweep at M = 16384, and the arithmetic modes other than the default."""
import os

import numpy as np
import pytest

import cfgcases
import opcases
import tol
from oracle import pyoracle as O
from see_ml_b200 import _lib as L
from see_ml_b200 import formats as F
from see_ml_b200 import plansynth as PS

pytestmark = pytest.mark.gpu


def _hasher():
    lib = L.lib()
    return lambda b, o: int(lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o))


@pytest.fixture(scope="module")
def golden(golden_dir):
    return np.load(os.path.join(golden_dir, "configs.npz"))


@pytest.mark.parametrize("mode", [1, 0], ids=["fused", "contract"])
@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_config_loss_curve_matches_the_reference_runtime(golden, name, mode):
    """Every step's training loss within 0.5 % of the reference's, the validation losses before
    and after likewise, through the engine's own feeder (validation tail split, shuffle seed 7)."""
    from see_ml_b200.engine import Dataset, UpdateEngine
    cfg, model, spec = cfgcases.model_and_spec(name)
    blob, _ = PS.synthesize(model, spec, hasher=_hasher())
    x, y = cfgcases.corpus(name)
    ds = Dataset.from_memory(x, y) if y is not None else Dataset.from_tokens(x)
    val = ds.split_validation(cfgcases.VAL_FRAC)
    ds.enable_shuffle(cfgcases.SEED)
    e = UpdateEngine(0, mode, 0)
    e.load_from_memory(blob)
    res = e.train(ds, cfgcases.STEPS[name], validation=val)
    want = golden[name + "/curve"]
    assert res.steps == len(want)
    np.testing.assert_allclose(res.loss_curve, want, rtol=5e-3, err_msg=name)
    np.testing.assert_allclose([res.val_initial_loss, res.val_final_loss], golden[name + "/val"], rtol=5e-3)
    got_p = e.arena_read(0, e.header.persistent_size).view(np.float32).astype(np.float64)
    want_p = golden[name + "/persistent"].astype(np.float64)
    # parameters after many AdamW steps: a norm-wise bound (a sign flip of a near-zero gradient moves one
    # element by 2 lr, so element-wise bars are not meaningful here)
    assert np.linalg.norm(got_p - want_p) <= 2e-2 * np.linalg.norm(want_p), name
    e.close()


@pytest.mark.parametrize("gemm", [0, 1], ids=["tf32x3", "f16x2"])
def test_c4_slice_chunk_loss_and_every_lora_gradient(golden, gemm):
    """One forward + backward pass over 16384 rows (32 sequences of 512) of two C4 layers: the
    persistent CTA-pair GEMM over 64 M-tile pairs at K / N in {1024, 2816, 8192}, the rank-16
    factor kernels, attention at 16 heads x 512, all against the reference runtime's values."""
    from see_ml_b200.engine import UpdateEngine
    cfg, model, spec, tok, lab = cfgcases.slice_inputs()
    blob, info = PS.synthesize(model, spec, hasher=_hasher())
    want_loss = float(golden["slice/loss"][0])
    want = golden["slice/grads"]
    for mode in (1, 0):
        e = UpdateEngine(0, mode, gemm)
        e.load_from_memory(blob)
        h = e.header
        for ref, v in cfgcases.b_values(info).items():
            e.arena_write(ref, v)
        e.arena_write(h.input_ref, tok)
        e.arena_write(h.label_ref, lab)
        e.run_train_range(0, e.opt_begin())
        assert abs(e.loss_value() - want_loss) <= 1e-4 * abs(want_loss), (mode, e.loss_value(), want_loss)
        at = 0
        for pid, _, g, n in info.params:
            tol.assert_close(e.arena_read(g, 4 * n).view(np.float32), want[at:at + n], f"mode {mode} gemm {gemm} {pid}")
            at += n
        assert at == want.size
        e.close()


def test_softmax_xent_forward_and_backward_at_32000_classes():
    from see_ml_b200.engine import Context
    rows, classes = 1024, 32000
    rng = np.random.default_rng(32000)
    logits = (rng.standard_normal((rows, classes)) * 2).astype(np.float32)
    labels = PS.zipf_tokens(rng, classes, rows)
    Lo = opcases.Layout()
    z, lab = Lo.put(logits), Lo.put(labels)
    loss, probs, seed, d = Lo.out(1), Lo.out(rows * classes), Lo.put(np.ones(1, np.float32)), Lo.out(rows * classes)
    arena, ro = Lo.done()
    I = opcases._ins
    prog = np.concatenate([I(F.Op.XENT_FWD, [z, lab, loss, probs], [rows, classes]),
                           I(F.Op.XENT_BWD, [probs, lab, seed, d], [rows, classes])])
    want = arena.copy()
    O.execute("port", prog, want, ro)
    ctx = Context(arena.size, ro)
    ctx.write(0, arena)
    ctx.execute(prog)
    got = ctx.read(0, arena.size)
    ctx.close()
    f = lambda a, off, n: a[off:off + 4 * n].view(np.float32)
    assert abs(f(got, loss, 1)[0] - f(want, loss, 1)[0]) <= 1e-5 * abs(f(want, loss, 1)[0])
    np.testing.assert_allclose(f(got, probs, rows * classes), f(want, probs, rows * classes), rtol=1e-4, atol=1e-9)
    np.testing.assert_allclose(f(got, d, rows * classes), f(want, d, rows * classes), rtol=1e-4, atol=1e-12)


@pytest.mark.parametrize("gemm", [0, 1], ids=["tf32x3", "f16x2"])
def test_lm_head_gemm_shape(gemm):
    """[2048 x 1024] . [1024 x 32000] against a frozen weight (forward, NN) and the matching
    dgrad [2048 x 32000] . W^T (NT), checked on sampled rows against an f64 product."""
    from see_ml_b200.engine import Context
    M, K, N = 2048, 1024, 32000
    rng = np.random.default_rng(7)
    X, W = opcases._rn(rng, M, K), (opcases._rn(rng, K, N) * 0.02).astype(np.float32)
    G = (opcases._rn(rng, M, N) * 1e-4).astype(np.float32)
    Lo = opcases.Layout()
    x, g, w = Lo.put(X), Lo.put(G), Lo.put(W, ro=True)
    y, dx = Lo.out(M * N), Lo.out(M * K)
    arena, ro = Lo.done()
    I = opcases._ins
    prog = np.concatenate([I(F.Op.GEMM_NN, [x, w, y], [M, N, K]), I(F.Op.GEMM_NT, [g, w, dx], [M, K, N])])
    ctx = Context(arena.size, ro, gemm=gemm)
    ctx.write(0, arena)
    ctx.execute(prog)
    rows = np.linspace(0, M - 1, 96).astype(int)
    Y = ctx.read(y, 4 * M * N).view(np.float32).reshape(M, N)[rows]
    DX = ctx.read(dx, 4 * M * K).view(np.float32).reshape(M, K)[rows]
    ctx.close()
    W64 = W.astype(np.float64)
    tol.assert_close(Y, X[rows].astype(np.float64) @ W64, "head forward")
    tol.assert_close(DX, G[rows].astype(np.float64) @ W64.T, "head dgrad")


@pytest.mark.parametrize("gemm", [0, 1], ids=["tf32x3", "f16x2"])
@pytest.mark.parametrize("kn", [(1024, 1024), (1024, 2816), (2816, 1024), (4096, 4096)], ids=lambda s: f"K{s[0]}xN{s[1]}")
def test_lora_matmul_sweep_at_16384_rows(kn, gemm):
    """The MatMul / LoRA sweep at M = 16384 (entries ~N(0,1), r = 16): forward, dgrad and both
    weight gradients as the compiler's instruction sequences, fused and per instruction, against
    f64 products (full for the reductions over M, sampled rows for the [M x .] outputs)."""
    _sweep_case(kn, 16, gemm)


@pytest.mark.parametrize("M", [2048, 16384])
@pytest.mark.parametrize("kn", [(1024, 2816), (2816, 1024)], ids=lambda s: f"K{s[0]}xN{s[1]}")
def test_lora_matmul_sweep_rank_64(kn, M):
    """The sweep's widest adapters (r = 64) in the default arithmetic, at its smallest M and at
    16384 rows: the low-rank term rides the fused GEMM as one 64-wide k-block, so the fused program
    must need fewer launches than the instruction path, with the same parity bar."""
    launches = _sweep_case(kn, 64, 1, M)
    assert launches[0] < launches[1], f"the rank-64 LoRA groups were not fused: {launches}"


def _sweep_case(kn, r, gemm, M=16384):
    from see_ml_b200.engine import Context, MODE_CONTRACT, MODE_FUSED
    from see_ml_b200.formats import Op
    K, N = kn
    alpha = 2.0 * r
    rng = np.random.default_rng(K * 11 + N)
    X, W = opcases._rn(rng, M, K), opcases._rn(rng, K, N)
    A, B = opcases._rn(rng, K, r), opcases._rn(rng, r, N)
    G = opcases._rn(rng, M, N)
    Lo = opcases.Layout()
    x, a, b, g = Lo.put(X), Lo.put(A), Lo.put(B), Lo.put(G)
    w = Lo.put(W, ro=True)
    c, t, u, s, y = Lo.out(M * N), Lo.out(M * r), Lo.out(M * N), Lo.out(M * N), Lo.out(M * N)
    ds, dt, dB, dx1, dA, dx2, dX = (Lo.out(M * N), Lo.out(M * r), Lo.out(r * N), Lo.out(M * K), Lo.out(K * r),
                                   Lo.out(M * K), Lo.out(M * K))
    arena, ro = Lo.done()
    sc = F.f32_bits(alpha / r)
    I = opcases._ins
    prog = np.concatenate([
        I(Op.GEMM_NN, [x, w, c], [M, N, K]), I(Op.GEMM_NN, [x, a, t], [M, r, K]),
        I(Op.GEMM_NN, [t, b, u], [M, N, r]), I(Op.SCALE, [u, s, sc], [M * N]), I(Op.ADD, [c, s, y], [M * N]),
        I(Op.SCALE, [g, ds, sc], [M * N]), I(Op.GEMM_NT, [ds, b, dt], [M, r, N]),
        I(Op.GEMM_TN, [t, ds, dB], [r, N, M]), I(Op.GEMM_NT, [dt, a, dx1], [M, K, r]),
        I(Op.GEMM_TN, [x, dt, dA], [K, r, M]), I(Op.GEMM_NT, [g, w, dx2], [M, K, N]),
        I(Op.ADD, [dx1, dx2, dX], [M * K])])
    rows = np.linspace(0, M - 1, 64).astype(int)
    X64, W64, A64, B64, G64 = (v.astype(np.float64) for v in (X, W, A, B, G))
    T64 = X64 @ A64
    dT64 = (alpha / r) * (G64 @ B64.T)
    ref = {"y": X64[rows] @ W64 + (alpha / r) * T64[rows] @ B64, "dB": T64.T @ ((alpha / r) * G64), "dA": X64.T @ dT64,
           "dX": dT64[rows] @ A64.T + G64[rows] @ W64.T}
    launches = []
    for mode in (MODE_FUSED, MODE_CONTRACT):
        ctx = Context(arena.size, ro, gemm=gemm)
        ctx.write(0, arena)
        pid = ctx.build(prog, mode=mode)
        ctx.run(pid, 0, len(prog))
        launches.append(ctx.launches(pid))
        f = lambda off, n: ctx.read(off, 4 * n).view(np.float32)
        tol.assert_close(f(y, M * N).reshape(M, N)[rows], ref["y"], f"K{K} N{N} r{r} mode {mode} y")
        tol.assert_close(f(dX, M * K).reshape(M, K)[rows], ref["dX"], f"K{K} N{N} r{r} mode {mode} dX")
        tol.assert_close(f(dB, r * N), ref["dB"], f"K{K} N{N} r{r} mode {mode} dB")
        tol.assert_close(f(dA, K * r), ref["dA"], f"K{K} N{N} r{r} mode {mode} dA")
        ctx.close()
    return launches


@pytest.mark.parametrize("gemm,name", [(1, "f16x2"), (3, "tf32")])
def test_other_arithmetic_modes_hold_the_loss_curve_criterion(golden_dir, gemm, name):
    """F16X2 (the two-term fp16 split) must meet the same 0.5 % loss-curve bar as the default;
    the single-product TF32 mode (10-bit operands, not f32-class per element) is accepted on that
    criterion alone, as the fast-arithmetic option."""
    import json
    import tccase
    from see_ml_b200.engine import Dataset, UpdateEngine
    want = json.load(open(os.path.join(golden_dir, "tc_curve.json")))
    model, spec, toks = tccase.build()
    blob = tccase.plan(model, spec, _hasher())
    e = UpdateEngine(0, 1, gemm)
    e.load_from_memory(blob)
    ds = Dataset.from_tokens(toks)
    ds.enable_shuffle(7)
    res = e.train(ds, tccase.STEPS)
    np.testing.assert_allclose(res.loss_curve, want["curve"], rtol=5e-3, err_msg=name)
    e.close()


def test_f16x2_gemm_keeps_f32_class_accuracy_at_extreme_operand_scales():
    """fp16 has five exponent bits: the power-of-two scaling ahead of the split must keep tiny
    gradients (1e-7) and large activations (3e4) at the accuracy of the three-product tf32 split."""
    from see_ml_b200.engine import Context
    M, N, K = 4096, 1024, 1024
    for sa, sb, seed in ((1e-7, 0.02, 3), (3e4, 50.0, 4), (1.0, 1.0, 5)):
        rng = np.random.default_rng(seed)
        A = (opcases._rn(rng, M, K) * sa).astype(np.float32)
        W = (opcases._rn(rng, N, K) * sb).astype(np.float32)
        Lo = opcases.Layout()
        a, w = Lo.put(A), Lo.put(W, ro=True)
        c = Lo.out(M * N)
        arena, ro = Lo.done()
        prog = opcases._ins(F.Op.GEMM_NT, [a, w, c], [M, N, K])
        rows = np.linspace(0, M - 1, 64).astype(int)
        want = A[rows].astype(np.float64) @ W.astype(np.float64).T
        errs = {}
        for gemm in (0, 1):
            ctx = Context(arena.size, ro, gemm=gemm)
            ctx.write(0, arena)
            ctx.execute(prog)
            got = ctx.read(c, 4 * M * N).view(np.float32).reshape(M, N)[rows]
            ctx.close()
            errs[gemm] = float(np.sqrt(np.mean((got - want) ** 2)))
        scale = float(np.sqrt(np.mean(want ** 2)))
        assert errs[1] <= max(2.0 * errs[0], 2e-7 * scale), (sa, sb, errs, scale)

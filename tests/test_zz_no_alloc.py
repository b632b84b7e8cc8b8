"""The allocation-free cross-entropy entry point against the regular instruction path.

Written for embedders that cannot let this library call cudaMalloc (their own pool owns
the device, or they call from a place where an allocation's implicit synchronisation is
unacceptable): the entry point keeps its scratch in a fixed array inside the library.
It runs the same kernels as the kXentFwd instruction, so its loss and probabilities must
equal that path's bit for bit — on a first call and again on a second call, which reuses
whatever the first left in the shared scratch. Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(rng, rows, classes):
    from see_ml_b200 import formats as F
    logits = (rng.standard_normal((rows, classes)) * 3).astype(np.float32)
    labels = rng.integers(0, classes, rows).astype(np.int32)
    off = {}
    cur = 0
    for name, nbytes in (("logits", logits.nbytes), ("labels", labels.nbytes), ("loss_a", 4),
                         ("probs_a", logits.nbytes), ("loss_b", 4), ("probs_b", logits.nbytes)):
        off[name] = cur
        cur = F.align_up(cur + nbytes, 256)
    return logits, labels, off, cur


# the last case sits at the row ceiling, where the chunk partials start right behind the last row term
@pytest.mark.parametrize("rows,classes", [(37, 10), (300, 513), (64, 5000), (65536, 4)])
def test_noalloc_entry_point_equals_instruction_path_twice(rows, classes):
    from see_ml_b200 import _lib as L
    from see_ml_b200 import formats as F
    from see_ml_b200.engine import Context
    lib = L.lib()
    rng = np.random.default_rng(rows * 7 + classes)
    logits, labels, off, size = _case(rng, rows, classes)
    ctx = Context(size)
    ctx.write(off["logits"], logits)
    ctx.write(off["labels"], labels)
    ins = np.zeros(1, dtype=F.INSTR_DTYPE)
    ins["in"] = F.NULL_REF
    ins["opcode"] = int(F.Op.XENT_FWD)
    ins["in"][0] = (off["logits"], off["labels"], off["loss_a"], off["probs_a"])
    ins["out"][0, :2] = (rows, classes)
    ctx.execute(ins)
    want_loss = ctx.read(off["loss_a"], 4).view(np.float32)[0]
    want_probs = ctx.read(off["probs_a"], logits.nbytes).view(np.float32)
    assert np.isfinite(want_loss)
    # the instruction path itself against the CPU statement of the reference's loss (loss.cc:43-58)
    z = logits.astype(np.float64)
    lse = np.log(np.exp(z - z.max(1, keepdims=True)).sum(1)) + z.max(1)
    ref_loss = float(np.mean(lse - z[np.arange(rows), labels]))
    assert abs(float(want_loss) - ref_loss) <= 1e-5 * max(1.0, abs(ref_loss))
    base = lib.seeml_b200_ctx_arena(ctx.h)
    stream = lib.seeml_b200_ctx_stream(ctx.h)
    for attempt in range(2):
        ctx.write(off["loss_b"], np.full(1, np.nan, np.float32))
        ctx.write(off["probs_b"], np.full(rows * classes, np.nan, np.float32))
        L.check(lib.seeml_b200_xent_fwd_noalloc(C.c_void_p(base + off["logits"]), C.c_void_p(base + off["labels"]),
                                                C.c_void_p(base + off["loss_b"]), C.c_void_p(base + off["probs_b"]),
                                                rows, classes, C.c_void_p(stream)))
        ctx.sync()
        got_loss = ctx.read(off["loss_b"], 4).view(np.float32)[0]
        got_probs = ctx.read(off["probs_b"], logits.nbytes).view(np.float32)
        assert got_loss.view(np.uint32) == want_loss.view(np.uint32), (attempt, got_loss, want_loss)
        np.testing.assert_array_equal(got_probs.view(np.uint32), want_probs.view(np.uint32))
    ctx.close()


def test_noalloc_entry_point_refuses_oversized_batches():
    from see_ml_b200 import _lib as L
    from see_ml_b200.engine import Context
    lib = L.lib()
    ctx = Context(4096)
    base = lib.seeml_b200_ctx_arena(ctx.h)
    rc = lib.seeml_b200_xent_fwd_noalloc(C.c_void_p(base), C.c_void_p(base), C.c_void_p(base), C.c_void_p(base),
                                         65537, 4, None)
    assert rc != 0 and "at most 65536 rows" in L.last_error()
    ctx.close()


def test_noalloc_entry_point_label_out_of_range_gives_nan_not_a_wild_read():
    from see_ml_b200 import _lib as L
    from see_ml_b200 import formats as F
    from see_ml_b200.engine import Context
    lib = L.lib()
    rows, classes = 8, 16
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((rows, classes)).astype(np.float32)
    labels = rng.integers(0, classes, rows).astype(np.int32)
    labels[3] = classes + 1000
    labels[5] = -7
    ctx = Context(8192)
    ctx.write(0, logits)
    ctx.write(1024, labels)
    base = lib.seeml_b200_ctx_arena(ctx.h)
    L.check(lib.seeml_b200_xent_fwd_noalloc(C.c_void_p(base), C.c_void_p(base + 1024), C.c_void_p(base + 2048),
                                            C.c_void_p(base + 4096), rows, classes,
                                            C.c_void_p(lib.seeml_b200_ctx_stream(ctx.h))))
    ctx.sync()
    assert np.isnan(ctx.read(2048, 4).view(np.float32)[0])
    probs = ctx.read(4096, logits.nbytes).view(np.float32).reshape(rows, classes)
    np.testing.assert_allclose(probs.sum(1), 1.0, rtol=1e-5)
    ctx.close()


def test_noalloc_entry_point_refuses_host_pointers():
    from see_ml_b200 import _lib as L
    from see_ml_b200.engine import Context
    lib = L.lib()
    ctx = Context(4096)       # makes a device current
    host = np.zeros(64, np.float32)
    base = lib.seeml_b200_ctx_arena(ctx.h)
    rc = lib.seeml_b200_xent_fwd_noalloc(host.ctypes.data_as(C.c_void_p), C.c_void_p(base), C.c_void_p(base),
                                         C.c_void_p(base), 4, 4, None)
    assert rc != 0 and "logits" in L.last_error()
    ctx.close()

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


@pytest.mark.parametrize("rows,classes", [(37, 10), (300, 513), (64, 5000)])
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

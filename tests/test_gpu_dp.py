"""The K-chunk data-parallel step on one GPU against the oracle: K executions of the train
stream up to the first optimiser instruction on K different batches, the per-chunk LoRA
gradients summed in the fixed binary tree over the chunk index and scaled by 1/K, then the
optimiser instructions once. Reference semantics: K consecutive reference batches through
update_engine.cc:736-771 with the gradient mean taken over the global batch."""
import numpy as np
import pytest

import tccase
from oracle import pyoracle as O
from see_ml_b200 import _lib as L
from see_ml_b200 import formats as F
from see_ml_b200 import plansynth as PS
from see_ml_b200.dp import gradient_spans, tree_sum_host

pytestmark = pytest.mark.gpu


def _case():
    lib = L.lib()
    model, spec, toks = tccase.build()
    blob, info = PS.synthesize(model, spec, hasher=lambda b, o: int(
        lib.seeml_b200_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o)))
    return blob, info, toks


@pytest.mark.parametrize("mode", [1, 0], ids=["fused", "contract"])
def test_k_chunk_step_matches_oracle_chunks_tree_and_optimizer(mode):
    from see_ml_b200.dp import DataParallelTrainer
    K = 4
    blob, info, toks = _case()
    plan = F.parse_plan(blob)
    h = plan.header
    per = h.batch // tccase.S
    recs = toks[:K * per].reshape(K, per, tccase.S + 1)
    tok = np.ascontiguousarray(recs[:, :, :-1]).reshape(K, -1)
    lab = np.ascontiguousarray(recs[:, :, 1:]).reshape(K, -1)
    rng = np.random.default_rng(2)
    bvals = {ad["b_ref"]: (rng.standard_normal(ad["r"] * ad["m"]) * 0.05).astype(np.float32) for ad in info.adapters}
    opt_begin = int(np.nonzero(plan.train["opcode"] == int(F.Op.ADAMW))[0][0])
    offs, counts = gradient_spans(plan.train)

    # oracle: each chunk from the same parameters, then the tree, then the optimiser stream
    base = np.zeros(F.align_up(h.arena_size), np.uint8)
    base[:h.persist_init_size] = plan.persist_init
    for ref, v in bvals.items():
        base[ref:ref + v.nbytes] = v.view(np.uint8)
    sets, losses = [], []
    for c in range(K):
        a = base.copy()
        a[h.input_ref:h.input_ref + tok[c].nbytes] = tok[c].view(np.uint8)
        a[h.label_ref:h.label_ref + lab[c].nbytes] = lab[c].view(np.uint8)
        O.execute("port", plan.train[:opt_begin], a, np.asarray(plan.rodata))
        sets.append(np.concatenate([a[int(o):int(o) + 4 * int(n)].view(np.float32) for o, n in zip(offs, counts)]))
        losses.append(a[h.loss_ref:h.loss_ref + 4].view(np.float32)[0])
    want_grad = tree_sum_host(np.stack(sets)) * np.float32(1.0 / K)
    want_loss = float(tree_sum_host(np.array(losses, np.float32).reshape(K, 1))[0] * np.float32(1.0 / K))

    runs = []
    for _ in range(2):
        tr = DataParallelTrainer(blob, K, mode=mode)
        for ref, v in bvals.items():
            tr.engine.arena_write(ref, v)
        loss = tr.step(tok, lab)
        got_grad = np.concatenate([tr.engine.arena_read(int(o), 4 * int(n)).view(np.float32) for o, n in zip(offs, counts)])
        runs.append((loss, got_grad, tr.persistent().copy()))
        tr.close()
    loss, got_grad, got_p = runs[0]
    assert abs(loss - want_loss) <= 1e-4 * abs(want_loss)
    at = 0
    for n in counts:
        n = int(n)
        ref = want_grad[at:at + n]
        np.testing.assert_allclose(got_grad[at:at + n], ref, rtol=1e-3, atol=1e-4 * max(1.0, float(np.abs(ref).max())))
        at += n
    # the optimiser half, bit for bit: the oracle's AdamW on the very gradients the GPU reduced
    a = base.copy()
    at = 0
    for o, n in zip(offs, counts):
        o, n = int(o), int(n)
        a[o:o + 4 * n] = got_grad[at:at + n].view(np.uint8)
        at += n
    O.execute("port", plan.train[opt_begin:], a, np.asarray(plan.rodata), lr=h.lr, b1=h.beta1, b2=h.beta2, eps=h.eps,
              wd=h.weight_decay, step=1)
    np.testing.assert_array_equal(got_p.view(np.uint32), a[:h.persistent_size].view(np.uint32))
    # and the whole step is bit-reproducible run to run
    assert runs[1][0] == loss
    np.testing.assert_array_equal(runs[1][2], got_p)


def test_collective_wait_has_a_deadline_and_aborts_the_communicator():
    """Failure detection without a GPU fault: the host-side wait on the exchange polls the
    communicator and the stream; when the stream does not drain before the deadline (here: a
    bounded one-second device sleep stands in for a rank that never posts) the call returns an
    attributable error and aborts the communicator instead of blocking. The context stays usable."""
    import ctypes as C
    import torch
    lib = L.lib()
    raw = (C.c_uint8 * 128)()
    L.check(lib.seeml_b200_comm_unique_id(raw))
    comm = C.c_void_p()
    L.check(lib.seeml_b200_comm_init(0, raw, 0, 1, C.byref(comm)))
    from see_ml_b200.engine import Context
    ctx = Context(1 << 20)
    stream = torch.cuda.ExternalStream(lib.seeml_b200_ctx_stream(ctx.h), device=torch.device("cuda", 0))
    # a healthy exchange first: world 1 all-gather of 256 floats, waited for with a generous deadline
    base = lib.seeml_b200_ctx_arena(ctx.h)
    ctx.write(0, np.arange(256, dtype=np.float32))
    L.check(lib.seeml_b200_comm_allgather(comm, C.c_void_p(base), C.c_void_p(base + 4096), 256,
                                          C.c_void_p(lib.seeml_b200_ctx_stream(ctx.h))))
    L.check(lib.seeml_b200_comm_wait(comm, C.c_void_p(lib.seeml_b200_ctx_stream(ctx.h)), 30.0))
    np.testing.assert_array_equal(ctx.read(4096, 1024).view(np.float32), np.arange(256, dtype=np.float32))
    with torch.cuda.stream(stream):
        torch.cuda._sleep(int(2.0e9))            # about a second of bounded device time
    rc = lib.seeml_b200_comm_wait(comm, C.c_void_p(lib.seeml_b200_ctx_stream(ctx.h)), 0.05)
    assert rc != 0 and "did not finish within" in L.last_error() and L.last_error().startswith("UpdateEngine: ")
    assert lib.seeml_b200_comm_allgather(comm, C.c_void_p(base), C.c_void_p(base + 4096), 256,
                                         C.c_void_p(lib.seeml_b200_ctx_stream(ctx.h))) != 0
    assert "aborted" in L.last_error()
    torch.cuda.synchronize()
    ctx.write(0, np.ones(4, np.float32))         # the context still works
    lib.seeml_b200_comm_destroy(comm)
    ctx.close()

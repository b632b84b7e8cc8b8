"""The C restatement (oracle/) against fixtures produced by the unmodified reference.

These are the pins that make the oracle trustworthy: every per-instruction case,
whole training steps and loss curves of reference-compiled plans, the hashes and the
LR schedule must reproduce the reference's bytes."""
import json
import os

import numpy as np
import pytest

import opcases
import plancases
from oracle import pyoracle as O
from see_ml_b200 import formats as F


def test_every_op_case_reproduces_reference_digest(golden_dir, port):
    import hashlib
    digests = json.load(open(os.path.join(golden_dir, "ops_digests.json")))
    cases = opcases.all_cases()
    assert {c.name for c in cases} == set(digests), "case list drifted: regenerate the fixtures"
    for c in cases:
        sha_in = hashlib.sha256(c.arena.tobytes()).hexdigest()
        assert sha_in == digests[c.name]["in"], f"{c.name}: seeded inputs drifted"
        a = c.arena.copy()
        O.execute("port", c.instr, a, c.rodata, **c.scalars)
        assert hashlib.sha256(a.tobytes()).hexdigest() == digests[c.name]["out"], c.name


def test_small_cases_full_tensors(golden_dir, port):
    z = np.load(os.path.join(golden_dir, "ops_small.npz"))
    names = sorted({k.rsplit("/", 1)[0] for k in z.files})
    assert len(names) > 50
    for n in names:
        arena = z[n + "/in"].copy()
        instr = z[n + "/instr"].view(F.INSTR_DTYPE)
        sc = {}
        if n.startswith("ADAMW") or n.startswith("SGD"):
            c = next(c for c in opcases.all_cases() if c.name == n)
            sc = c.scalars
        O.execute("port", instr, arena, z[n + "/ro"], **sc)
        np.testing.assert_array_equal(arena, z[n + "/out"], err_msg=n)


@pytest.mark.parametrize("pc", plancases.plan_cases(), ids=lambda p: p.name)
def test_oracle_runs_reference_plans_bit_exactly(golden_dir, port, pc):
    """Interpret the reference-compiled plan with the C oracle: one hand-fed step must
    give the reference engine's persistent segment and loss, bit for bit."""
    z = np.load(os.path.join(golden_dir, "plans.npz"))
    plan = F.parse_plan(z[pc.name].tobytes())
    h = plan.header
    arena = np.zeros(F.align_up(h.arena_size), np.uint8)
    arena[:h.persist_init_size] = plan.persist_init
    inp, lab = pc.first_batch()
    arena[h.input_ref:h.input_ref + inp.nbytes] = inp.view(np.uint8)
    arena[h.label_ref:h.label_ref + lab.nbytes] = lab.view(np.uint8)
    lr = port.orc_effective_lr(h.lr, h.lr_schedule, h.warmup_steps, h.default_steps, h.min_lr_factor, 1)
    O.execute("port", plan.train, arena, np.asarray(plan.rodata), lr=lr, b1=h.beta1, b2=h.beta2,
              eps=h.eps, wd=h.weight_decay, step=1)
    np.testing.assert_array_equal(arena[:h.persistent_size], z[pc.name + "/step1_persistent"])
    loss = arena[h.loss_ref:h.loss_ref + 4].view(np.float32)[0]
    assert loss == z[pc.name + "/step1_loss"][0]


def test_hashes_match_reference(golden_dir, port):
    m = json.load(open(os.path.join(golden_dir, "misc.json")))["misc"]["hash"]
    for n_s, want in m.items():
        n = int(n_s)
        buf = np.random.default_rng(n).integers(0, 256, n, dtype=np.uint8)
        p = buf.ctypes.data if n else None
        assert port.orc_content_hash64(p, n) == int(want["content"])
        assert port.orc_plan_self_hash(p, n, 216) == int(want["self216"])
        if n <= 4096:
            assert F.content_hash64(buf.tobytes()) == int(want["content"])


def test_lr_schedule_matches_reference(golden_dir, port):
    rows = json.load(open(os.path.join(golden_dir, "misc.json")))["misc"]["lr"]
    assert len(rows) > 30
    for r in rows:
        s = r["sched"]
        got = port.orc_effective_lr(np.float32(5e-3), s.get("lr_schedule", 0), s.get("warmup_steps", 0), 100,
                                    s.get("min_lr_factor", 0.0), r["step"])
        assert np.float32(got) == np.float32(r["lr"]), r


@pytest.mark.skipif(not O.have_ref(), reason="reference build (oracle/_ref) not present")
def test_port_equals_live_reference_on_all_cases(port):
    for c in opcases.all_cases(seed=77):
        a1, a2 = c.arena.copy(), c.arena.copy()
        O.execute("port", c.instr, a1, c.rodata, **c.scalars)
        O.execute("ref", c.instr, a2, c.rodata, **c.scalars)
        np.testing.assert_array_equal(a1, a2, err_msg=c.name)

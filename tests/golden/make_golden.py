"""Regenerates the golden fixtures from the UNMODIFIED reference (oracle/_ref).

Run where the reference checkout is present:

    make -C oracle ref && python tests/golden/make_golden.py

Everything written here is produced by the reference's own code paths through
oracle/ref_harness.cc: its kernels (per-instruction cases), its compiler (plan
bytes), its engine (arena after a step, loss curves, evaluation, merge deltas),
its feeder (served batches), its hashes, LR schedule and validator verdicts.
The fixtures pin the C restatement (oracle/) and the host-side logic of the
backend; they are small on purpose (digests for the bulk, full tensors only for
tiny cases).
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import opcases  # noqa: E402
import plancases  # noqa: E402
from oracle import pyoracle as O  # noqa: E402
from see_ml_b200 import formats as F  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    assert O.have_ref(), "build oracle/_ref first (make -C oracle ref)"
    ref = O.ref()
    ref.ref_set_threads(4)

    # --- per-instruction cases -------------------------------------------------------
    digests, small = {}, {}
    for c in opcases.all_cases():
        a = c.arena.copy()
        O.execute("ref", c.instr, a, c.rodata, **c.scalars)
        digests[c.name] = {"in": sha(c.arena), "out": sha(a)}
        if c.arena.size <= 4096:
            small[c.name + "/in"] = c.arena
            small[c.name + "/ro"] = c.rodata
            small[c.name + "/instr"] = c.instr.view(np.uint8)
            small[c.name + "/out"] = a
    with open(os.path.join(HERE, "ops_digests.json"), "w") as f:
        json.dump(digests, f, indent=0, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "ops_small.npz"), **small)

    # --- plans: reference-compiled bytes + engine behaviour -----------------------------
    tmp = tempfile.mkdtemp()
    plans = {}
    meta = {}
    for pc in plancases.plan_cases():
        smf = os.path.join(tmp, pc.name + ".smf")
        pc.model.write_smf(smf)
        blob = O.ref_compile(smf, os.path.join(tmp, pc.name + ".seeu"), pc.spec.batch, pc.spec.lora_rank,
                             pc.spec.lora_alpha, pc.spec.lora_seed, ",".join(pc.spec.targets),
                             lr=pc.spec.lr, steps=pc.spec.default_steps,
                             fuse_epilogues=int(pc.spec.fuse_epilogues), clip_norm=pc.spec.clip_norm,
                             lr_schedule=pc.spec.lr_schedule, warmup=pc.spec.warmup_steps,
                             min_lr_factor=pc.spec.min_lr_factor)
        plans[pc.name] = np.frombuffer(blob, np.uint8)
        h = F.PlanHeader.unpack(blob)
        # one executed step from fixed I/O slots: whole arena digest + persistent segment
        e = O.RefEngine(blob)
        inp, lab = pc.first_batch()
        arena = e.arena()
        arena[h.input_ref:h.input_ref + inp.nbytes] = inp.view(np.uint8)
        arena[h.label_ref:h.label_ref + lab.nbytes] = lab.view(np.uint8)
        e.execute_train_once()
        plans[pc.name + "/step1_persistent"] = arena[:h.persistent_size].copy()
        plans[pc.name + "/step1_loss"] = np.array([e.loss()], np.float32)
        # training run through the reference feeder: loss curve, gate metrics, merge deltas
        e2 = O.RefEngine(blob)
        ds = pc.ref_dataset()
        val = ds.split_validation(0.25)
        ds.enable_shuffle(7)
        curve, rep = e2.train(ds, pc.steps, validation=val)
        plans[pc.name + "/curve"] = curve
        plans[pc.name + "/final_persistent"] = e2.arena()[:h.persistent_size].copy()
        e2.run_merge()
        em = F.parse_plan(blob).emit
        plans[pc.name + "/deltas"] = np.concatenate(
            [e2.arena()[int(x["arena_offset"]):int(x["arena_offset"] + x["byte_size"])] for x in em])
        meta[pc.name] = dict(val_initial_loss=float(rep.val_initial_loss),
                             val_final_loss=float(rep.val_final_loss),
                             has_val_accuracy=int(rep.has_val_accuracy),
                             val_initial_accuracy=float(rep.val_initial_accuracy),
                             val_final_accuracy=float(rep.val_final_accuracy),
                             improved=int(rep.improved), steps=int(rep.steps),
                             initial_avg_loss=float(rep.initial_avg_loss),
                             final_avg_loss=float(rep.final_avg_loss))
    np.savez_compressed(os.path.join(HERE, "plans.npz"), **plans)

    # --- feeder: served batches ------------------------------------------------------------
    feeder = {}
    rng = np.random.default_rng(99)
    x = rng.standard_normal((23, 5)).astype(np.float32)
    y = rng.integers(0, 4, 23).astype(np.int32)
    d = O.RefDataset.from_memory(x, y)
    feeder["f32/x"], feeder["f32/y"] = x, y
    seq = [np.concatenate([a.view(np.uint8), b]) for a, b in (d.fill_batch(8, 40, 32) for _ in range(7))]
    feeder["f32/sequential"] = np.stack(seq)
    d.enable_shuffle(12345)
    seq = [np.concatenate([a.view(np.uint8), b]) for a, b in (d.fill_batch(8, 40, 32) for _ in range(9))]
    feeder["f32/shuffled_seed12345"] = np.stack(seq)
    d2 = O.RefDataset.from_memory(x, y)
    v = d2.split_validation(0.3)
    feeder["f32/split_sizes"] = np.array([d2.num_samples(), v.num_samples()], np.int64)
    a, b = v.fill_batch(4, 20, 16)
    feeder["f32/val_first"] = np.concatenate([a.view(np.uint8), b])
    toks = rng.integers(0, 50, (11, 7)).astype(np.int32)
    t = O.RefDataset.from_tokens(toks)
    feeder["tok/records"] = toks
    t.enable_shuffle(0)
    seq = [np.concatenate([a.view(np.uint8), b]) for a, b in (t.fill_batch(18, 18, 72) for _ in range(8))]
    feeder["tok/shuffled_seed0"] = np.stack(seq)
    t2 = O.RefDataset.from_tokens(toks)
    t2.enable_shuffle(3)
    ref.ref_dataset_skip_served(t2.h, 18 * 5)
    a, b = t2.fill_batch(18, 18, 72)
    feeder["tok/after_skip_5_batches_seed3"] = np.concatenate([a.view(np.uint8), b])
    np.savez_compressed(os.path.join(HERE, "feeder.npz"), **feeder)

    # --- hashes, LR schedule, validator verdicts ------------------------------------------------
    misc = {"hash": {}, "lr": [], "validator": []}
    for n in (0, 1, 7, 8, 9, 4096, (1 << 20) + 3, 3 * (1 << 20) + 17):
        buf = np.random.default_rng(n).integers(0, 256, n, dtype=np.uint8)
        p = buf.ctypes.data if n else None
        misc["hash"][str(n)] = {"content": str(ref.ref_content_hash64(p, n)),
                                "self216": str(ref.ref_plan_self_hash(p, n, 216))}
    name = "mlp_tiny"
    blob = bytes(plans[name])
    for sched in (dict(lr_schedule=0), dict(lr_schedule=1, warmup_steps=10, min_lr_factor=0.1),
                  dict(lr_schedule=1, warmup_steps=0, min_lr_factor=0.0),
                  dict(lr_schedule=1, warmup_steps=50, min_lr_factor=0.5)):
        p = F.parse_plan(blob)
        for k, val in sched.items():
            setattr(p.header, k, val)
        p.header.default_steps = 100
        nb = F.assemble_plan(p.header, p.train, p.merge, p.eval, p.rodata, p.persist_init, p.emit,
                             hasher=lambda b, o: int(ref.ref_plan_self_hash(
                                 np.frombuffer(b, np.uint8).ctypes.data, len(b), o)))
        e = O.RefEngine(nb)
        for step in (0, 1, 5, 10, 11, 50, 51, 99, 100, 101, 1000):
            e.set_step(step)
            misc["lr"].append(dict(sched=sched, step=step, lr=float(np.float32(e.effective_lr()))))
    import ctypes as C
    for case in plancases.validator_cases():
        err = C.create_string_buffer(512)
        rc = ref.ref_validate_instruction(case["instr"].ctypes.data, case["arena"], case["rodata"],
                                          case["version"], err, 512)
        misc["validator"].append(dict(name=case["name"], accepted=int(rc == 0), message=err.value.decode()))
    with open(os.path.join(HERE, "misc.json"), "w") as f:
        json.dump({"misc": misc, "plans": meta}, f, indent=1, sort_keys=True)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()

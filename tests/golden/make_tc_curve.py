"""Generates tests/golden/tc_curve.json: the reference runtime's 100-step loss curve on a
decoder wide enough for the tensor-core kernels (64-wide heads, sequence length 128, 1024
rows per step, LoRA rank 16 on every projection). Run here, where the reference sources
are present:  python tests/golden/make_tc_curve.py

The plan itself is not stored: tests rebuild it with see_ml_b200.plansynth from the same
seeds (byte-identical to the reference compiler's output, which this script asserts)."""
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import tccase  # noqa: E402
from oracle import pyoracle as O  # noqa: E402


def main():
    O.build_ref()
    model, spec, toks = tccase.build()
    hasher = lambda b, o: int(O.ref().ref_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o))
    tmp = tempfile.mkdtemp()
    smf = os.path.join(tmp, "tc.smf")
    model.write_smf(smf)
    raw = np.fromfile(smf, np.uint8)
    spec.source_model_hash = int(O.ref().ref_content_hash64(raw.ctypes.data, raw.size))   # as the compiler stamps it
    blob = tccase.plan(model, spec, hasher)
    spec.source_model_hash = 0
    blob0 = tccase.plan(model, spec, hasher)           # what the test builds: no model file, hash field 0
    ref_blob = O.ref_compile(smf, os.path.join(tmp, "tc.seeu"), spec.batch, spec.lora_rank, spec.lora_alpha,
                             spec.lora_seed, ",".join(spec.targets), lr=spec.lr, steps=spec.default_steps,
                             fuse_epilogues=int(spec.fuse_epilogues), clip_norm=spec.clip_norm,
                             lr_schedule=spec.lr_schedule, warmup=spec.warmup_steps,
                             min_lr_factor=spec.min_lr_factor)
    assert bytes(ref_blob) == bytes(blob), "plansynth output differs from the reference compiler's"
    O.ref().ref_set_threads(os.cpu_count() or 1)
    e = O.RefEngine(blob0)
    ds = O.RefDataset.from_tokens(toks)
    ds.enable_shuffle(7)
    curve, rep = e.train(ds, tccase.STEPS)
    out = dict(steps=int(rep.steps), curve=[float(v) for v in curve],
               initial_avg_loss=float(rep.initial_avg_loss), final_avg_loss=float(rep.final_avg_loss))
    json.dump(out, open(os.path.join(HERE, "tc_curve.json"), "w"))
    print("steps", rep.steps, "loss", curve[0], "->", curve[-1])


if __name__ == "__main__":
    main()

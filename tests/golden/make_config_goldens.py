"""Generates tests/golden/configs.npz: what the reference runtime computes on the benchmark
configurations at their own shapes. Run here, where the reference sources are present:

    python tests/golden/make_config_goldens.py [c1 c2 c3 slice]

* c1 / c2 / c3: the loss at every optimiser step through the shuffled feeder (seed 7, a 10 %
  validation tail split off first), the validation losses before and after, and the persistent
  segment (adapters + AdamW moments) at the end.
* slice: one 16384-row chunk of a two-layer slice of C4 (d 1024, 16 heads, ffn 2816, seq 512,
  rank-16 LoRA on q/k/v/o/up/down): the loss and every LoRA gradient of one forward + backward
  pass, with the B factors set to seeded non-zero values.

Plans are not stored: tests rebuild them with see_ml_b200.plansynth from the same seeds."""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import cfgcases  # noqa: E402
from oracle import pyoracle as O  # noqa: E402
from see_ml_b200 import formats as F  # noqa: E402
from see_ml_b200 import plansynth as PS  # noqa: E402

OUT = os.path.join(HERE, "configs.npz")


def hasher(b, o):
    return int(O.ref().ref_plan_self_hash(np.frombuffer(b, np.uint8).ctypes.data, len(b), o))


def curve_case(name, out):
    cfg, model, spec = cfgcases.model_and_spec(name)
    blob, _ = PS.synthesize(model, spec, hasher=hasher)
    x, y = cfgcases.corpus(name)
    ds = O.RefDataset.from_memory(x, y) if y is not None else O.RefDataset.from_tokens(x)
    val = ds.split_validation(cfgcases.VAL_FRAC)
    ds.enable_shuffle(cfgcases.SEED)
    e = O.RefEngine(blob)
    t0 = time.time()
    curve, rep = e.train(ds, cfgcases.STEPS[name], validation=val)
    h = e.header
    out[name + "/curve"] = curve.astype(np.float32)
    out[name + "/val"] = np.array([rep.val_initial_loss, rep.val_final_loss], np.float32)
    out[name + "/persistent"] = e.arena()[:h.persistent_size].view(np.float32).copy()
    print(name, "steps", rep.steps, "loss", curve[0], "->", curve[-1], "val", rep.val_initial_loss, "->",
          rep.val_final_loss, f"{time.time() - t0:.1f}s", flush=True)


def slice_case(out):
    cfg, model, spec, tok, lab = cfgcases.slice_inputs()
    blob, info = PS.synthesize(model, spec, hasher=hasher)
    e = O.RefEngine(blob)
    h = e.header
    arena = e.arena()
    for ref, v in cfgcases.b_values(info).items():
        arena[ref:ref + v.nbytes] = v.view(np.uint8)
    arena[h.input_ref:h.input_ref + tok.nbytes] = tok.view(np.uint8)
    arena[h.label_ref:h.label_ref + lab.nbytes] = lab.view(np.uint8)
    t0 = time.time()
    e.execute_train_once()          # the gradient slots keep their values through the optimiser instructions
    out["slice/loss"] = np.array([e.loss()], np.float32)
    out["slice/grads"] = np.concatenate([arena[g:g + 4 * n].view(np.float32) for _, _, g, n in info.params])
    print("slice loss", e.loss(), "grad floats", out["slice/grads"].size, f"{time.time() - t0:.1f}s", flush=True)


def main():
    O.build_ref()
    O.ref().ref_set_threads(os.cpu_count() or 1)
    which = sys.argv[1:] or ["c1", "c2", "c3", "slice"]
    out = dict(np.load(OUT)) if os.path.exists(OUT) else {}
    for w in which:
        if w == "slice":
            slice_case(out)
        else:
            curve_case(w, out)
        np.savez(OUT, **out)


if __name__ == "__main__":
    main()

"""The tensor-core-sized training case shared by its fixture generator and its GPU test."""
import numpy as np

from see_ml_b200 import plansynth as PS

STEPS = 100
V, D, H, FF, LAYERS, S, ROWS = 512, 256, 4, 512, 2, 128, 1024


def build():
    rng = np.random.default_rng(31)
    model = PS.llama_decoder(V, D, H, FF, LAYERS, S, rng, std=0.05)
    spec = PS.TrainSpec(batch=ROWS, lora_rank=16, lora_alpha=32.0, lr=2e-3, default_steps=STEPS,
                        targets=("wq", "wk", "wv", "wo", "w_up", "w_down"))
    toks = rng.integers(0, V, (96, S + 1)).astype(np.int32)
    toks[:, 1::2] = (toks[:, 0:-1:2] * 3 + 1) % V          # every second token follows from the one before
    return model, spec, toks


def plan(model, spec, hasher):
    blob, _ = PS.synthesize(model, spec, hasher=hasher)
    return blob

"""The benchmark configurations at their own shapes (C1 MLP, C2 LayerNorm/GELU decoder, C3 and
a two-layer slice of C4, both RMSNorm/RoPE/SwiGLU decoders), shared by the fixture generator
(tests/golden/make_config_goldens.py, which runs the reference runtime on them) and the GPU
parity tests. Models, corpora and plans are rebuilt from seeds; only the reference's results
are stored."""
import numpy as np

import bench
from see_ml_b200 import plansynth as PS

STEPS = {"c1": 100, "c2": 100, "c3": 40}      # optimiser steps of the stored loss curves
SEED, VAL_FRAC = 7, 0.1


def model_and_spec(name):
    cfg = dict(bench.CONFIGS[name])
    model = bench.build_model(cfg)
    rows = cfg["rows"] if cfg["kind"] == "mlp" else cfg["seqs"] * cfg["seq"]
    spec = PS.TrainSpec(batch=rows, lora_rank=cfg["rank"], lora_alpha=cfg["alpha"], targets=cfg["targets"],
                        lr=cfg["lr"], default_steps=1000)
    return cfg, model, spec


def corpus(name):
    """C1: 4096 rows of N(0,1) features with uniform labels; C2: 256 uniform-token sequences;
    C3: 8192 Zipf(1.1) sequences (records of seq + 1 ids)."""
    cfg = bench.CONFIGS[name]
    rng = np.random.default_rng({"c1": 11, "c2": 12, "c3": 13}[name])
    if cfg["kind"] == "mlp":
        x = rng.standard_normal((4096, cfg["dims"][0])).astype(np.float32)
        y = rng.integers(0, cfg["dims"][-1], 4096).astype(np.int32)
        return x, y
    if name == "c2":
        return rng.integers(0, cfg["vocab"], (256, cfg["seq"] + 1)).astype(np.int32), None
    return PS.zipf_tokens(rng, cfg["vocab"], (8192, cfg["seq"] + 1)), None


def slice_inputs():
    """One chunk of the C4 slice: 32 Zipf(1.1) sequences of 512 tokens, and non-zero values for
    the LoRA B factors (they start at zero, which would zero every A gradient)."""
    cfg, model, spec = model_and_spec("c4-slice")
    tok, lab = bench.synth_batches(cfg, spec.batch, 1, seed=77)
    return cfg, model, spec, tok[0].copy(), lab[0].copy()


def b_values(info, seed=5):
    rng = np.random.default_rng(seed)
    return {ad["b_ref"]: (rng.standard_normal(ad["r"] * ad["m"]) * 0.02).astype(np.float32) for ad in info.adapters}

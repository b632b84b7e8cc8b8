"""Seeded whole-plan cases (tiny versions of the benchmark configurations) and a set
of well-formed / malformed instruction words for the validator."""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from see_ml_b200 import formats as F  # noqa: E402
from see_ml_b200 import plansynth as PS  # noqa: E402
from see_ml_b200.formats import Op  # noqa: E402


@dataclass
class PlanCase:
    name: str
    model: F.ModelGraph
    spec: PS.TrainSpec
    steps: int
    corpus_x: np.ndarray | None      # f32 rows (feature plans)
    corpus_y: np.ndarray | None
    corpus_tokens: np.ndarray | None  # [N, S+1] i32 (token plans)

    def first_batch(self):
        """Input/label slot contents for a single fed-by-hand step."""
        T = self.spec.batch
        if self.corpus_tokens is not None:
            S = self.model.seq_len
            recs = self.corpus_tokens[:T // S]
            return recs[:, :-1].reshape(-1).astype(np.int32), recs[:, 1:].reshape(-1).astype(np.int32)
        return self.corpus_x[:T].astype(np.float32).reshape(-1), self.corpus_y[:T].astype(np.int32)

    def ref_dataset(self):
        from oracle import pyoracle as O
        if self.corpus_tokens is not None:
            return O.RefDataset.from_tokens(self.corpus_tokens)
        return O.RefDataset.from_memory(self.corpus_x, self.corpus_y)

    def dataset(self):
        from see_ml_b200.engine import Dataset
        if self.corpus_tokens is not None:
            return Dataset.from_tokens(self.corpus_tokens)
        return Dataset.from_memory(self.corpus_x, self.corpus_y)


def plan_cases():
    rng = np.random.default_rng(2024)
    out = []
    # C1 in miniature: MLP with biases, ReLU / GELU, LoRA on every MatMul
    m = PS.mlp_model([12, 24, 24, 6], ["relu", "gelu", None], rng)
    x = rng.standard_normal((80, 12)).astype(np.float32)
    w = rng.standard_normal((12, 6)).astype(np.float32)
    y = np.argmax(x @ w, axis=1).astype(np.int32)           # learnable labels
    out.append(PlanCase("mlp_tiny", m, PS.TrainSpec(batch=8, lora_rank=4, lora_alpha=8.0, lr=5e-3,
                                                    default_steps=40), 40, x, y, None))
    # un-adapted layers with bias: GEMM epilogue flags, SiLU, cosine schedule, clipping
    m = PS.mlp_model([12, 16, 16, 6], ["relu", "silu", None], rng)
    out.append(PlanCase("mlp_fused", m, PS.TrainSpec(batch=8, lora_rank=2, lora_alpha=4.0, lr=1e-2,
                                                     targets=("w2",), default_steps=30, clip_norm=0.5,
                                                     lr_schedule=1, warmup_steps=5, min_lr_factor=0.1),
                        30, x, y, None))
    # C2 in miniature: LayerNorm + GELU decoder, LoRA on q and v
    V, D, H, Ff, S = 40, 16, 2, 32, 8
    m = PS.gpt_decoder(V, D, H, Ff, 2, S, rng, std=0.2)
    toks = rng.integers(0, V, (24, S + 1)).astype(np.int32)
    toks[:, 1::2] = (toks[:, 0:-1:2] + 1) % V               # learnable structure
    out.append(PlanCase("gpt_tiny", m, PS.TrainSpec(batch=2 * S, lora_rank=4, lora_alpha=8.0, lr=5e-3,
                                                    targets=("wq", "wv"), default_steps=30), 30,
                        None, None, toks))
    # C3/C4 in miniature: RMSNorm + RoPE + SwiGLU decoder, LoRA on q,k,v,o,up,down
    m = PS.llama_decoder(V, D, H, 24, 2, S, rng, std=0.2)
    out.append(PlanCase("llama_tiny", m, PS.TrainSpec(batch=3 * S, lora_rank=4, lora_alpha=8.0, lr=5e-3,
                                                      targets=("wq", "wk", "wv", "wo", "w_up", "w_down"),
                                                      default_steps=30), 30, None, None, toks))
    return out


def _ins(op, ins=(), outs=(), flags=0):
    i = np.zeros(1, dtype=F.INSTR_DTYPE)
    i["in"] = F.NULL_REF
    i["opcode"], i["flags"] = int(op), flags
    for k, w in enumerate(ins):
        i["in"][0, k] = w
    for k, w in enumerate(outs):
        i["out"][0, k] = w
    return i


def validator_cases():
    """Instruction words with the verdict the reference's validator gives each
    (the verdicts themselves are recorded in the golden fixtures)."""
    A, R, RO = 1 << 16, 1 << 12, F.RODATA_BIT
    c = []

    def add(name, instr, version=7, arena=A, rodata=R):
        c.append(dict(name=name, instr=instr, version=version, arena=arena, rodata=rodata))
    add("gemm_ok", _ins(Op.GEMM_NN, [0, 4096, 8192], [8, 8, 8]))
    add("gemm_rodata_b", _ins(Op.GEMM_NN, [0, RO | 0, 8192], [8, 8, 8]))
    add("gemm_write_rodata", _ins(Op.GEMM_NN, [0, 4096, RO | 0], [8, 8, 8]))
    add("gemm_oob", _ins(Op.GEMM_NN, [0, 4096, A - 64], [8, 8, 8]))
    add("gemm_alias", _ins(Op.GEMM_NN, [0, 4096, 128], [8, 8, 8]))
    add("gemm_zero_dim", _ins(Op.GEMM_NN, [0, 4096, 8192], [0, 8, 8]))
    add("gemm_overflow", _ins(Op.GEMM_NN, [0, 4096, 8192], [1 << 40, 1 << 40, 8]))
    add("gemm_misaligned", _ins(Op.GEMM_NN, [2, 4096, 8192], [8, 8, 8]))
    add("gemm_null", _ins(Op.GEMM_NN, [0, F.NULL_REF, 8192], [8, 8, 8]))
    add("gemm_bias_flag", _ins(Op.GEMM_NN, [0, 4096, 8192, RO | 64], [8, 8, 8], flags=1 | (2 << 1)))
    add("gemm_bias_flag_missing_ref", _ins(Op.GEMM_NN, [0, 4096, 8192], [8, 8, 8], flags=1))
    add("gemm_nt_flags_rejected", _ins(Op.GEMM_NT, [0, 4096, 8192], [8, 8, 8], flags=2))
    add("unknown_flag_bit", _ins(Op.GEMM_NN, [0, 4096, 8192], [8, 8, 8], flags=8))
    add("flags_in_v4_plan", _ins(Op.GEMM_NN, [0, 4096, 8192], [8, 8, 8], flags=2), version=4)
    add("q8_ok", _ins(Op.GEMM_NN_Q8, [0, RO | 0, 8192, F.f32_bits(0.1)], [8, 8, 8]))
    add("q8_b_in_arena", _ins(Op.GEMM_NN_Q8, [0, 4096, 8192, F.f32_bits(0.1)], [8, 8, 8]))
    add("q8_bias_flag", _ins(Op.GEMM_NN_Q8, [0, RO | 0, 8192, F.f32_bits(0.1)], [8, 8, 8], flags=1))
    add("add_ok", _ins(Op.ADD, [0, 4096, 8192], [100]))
    add("add_inplace_alias", _ins(Op.ADD, [0, 4096, 0], [100]))
    add("adamw_ok", _ins(Op.ADAMW, [0, 4096, 8192, 12288], [64]))
    add("adamw_m_aliases_p", _ins(Op.ADAMW, [0, 4096, 0, 12288], [64]))
    add("rope_odd_head", _ins(Op.ROPE_FWD, [0, 8192], [F.pack32(2, 4), F.pack32(2, 3), F.f32_bits(1e4)]))
    add("rope_ok", _ins(Op.ROPE_FWD, [0, 8192], [F.pack32(2, 4), F.pack32(2, 4), F.f32_bits(1e4)]))
    add("rope_in_v5_plan", _ins(Op.ROPE_FWD, [0, 8192], [F.pack32(2, 4), F.pack32(2, 4), F.f32_bits(1e4)]),
        version=5)
    add("attn_ok", _ins(Op.ATTN_FWD, [0, 1024, 2048, 3072], [8192, F.pack32(2, 4), F.pack32(2, 4)]))
    add("attn_probs_oob", _ins(Op.ATTN_FWD, [0, 1024, 2048, 3072], [A - 128, F.pack32(2, 4), F.pack32(2, 4)]))
    add("attn_zero_heads", _ins(Op.ATTN_FWD, [0, 1024, 2048, 3072], [8192, F.pack32(2, 4), F.pack32(0, 4)]))
    add("embed_ok", _ins(Op.EMBED, [0, RO | 0, 4096], [8, F.pack32(16, 4)]))
    add("embed_table_in_arena", _ins(Op.EMBED, [0, 8192, 4096], [8, F.pack32(16, 4)]))
    add("embed_in_v6_plan", _ins(Op.EMBED, [0, RO | 0, 4096], [8, F.pack32(16, 4)]), version=6)
    add("embed_table_oob", _ins(Op.EMBED, [0, RO | 0, 4096], [8, F.pack32(1 << 20, 4)]))
    add("layernorm_ok", _ins(Op.LAYERNORM_FWD, [0, RO | 0, RO | 256, 4096], [F.pack32(4, 8), 8192, 8256]))
    add("layernorm_stats_alias", _ins(Op.LAYERNORM_FWD, [0, RO | 0, RO | 256, 4096], [F.pack32(4, 8), 8192, 8192]))
    add("xent_ok", _ins(Op.XENT_FWD, [0, 4096, 8192, 12288], [8, 10]))
    add("fill_ok", _ins(Op.FILL, [0, F.f32_bits(1.0)], [1]))
    add("fill_zero", _ins(Op.FILL, [0, F.f32_bits(1.0)], [0]))
    add("nop", _ins(Op.NOP))
    add("unknown_opcode", _ins(77))
    add("kl_ok", _ins(Op.KL_FWD, [0, 1024, 2048, 3072], [4096, F.pack32(4, 8), F.f32_bits(2.0)]))
    add("clip_ok", _ins(Op.CLIP_NORM, [0, F.f32_bits(1.0)], [16]))
    add("softmax_rows_ok", _ins(Op.SOFTMAX_ROWS_BWD, [0, 4096, 8192], [F.pack32(8, 8)]))
    return c

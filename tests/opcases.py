"""Seeded single-instruction cases for every opcode of the update ISA.

Each case lays its operands out in a small arena (+ rodata), so the same bytes can
be executed by the reference kernels, the C restatement and the CUDA backend, and
the written ranges compared. Shapes include ragged ones (sizes that are not
multiples of any tile or vector width), single rows, and sizes around chunk
boundaries of the ordered reductions.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from see_ml_b200 import formats as F  # noqa: E402
from see_ml_b200.formats import Op  # noqa: E402


@dataclass
class Case:
    name: str
    instr: np.ndarray                 # 1-element INSTR_DTYPE array
    arena: np.ndarray                 # uint8
    rodata: np.ndarray                # uint8
    outputs: dict = field(default_factory=dict)   # name -> (offset, count, dtype)
    scalars: dict = field(default_factory=dict)
    rtol: float = 1e-3
    atol: float = 1e-4
    exact: bool = False               # bit-exact expected on the GPU


class Layout:
    def __init__(self):
        self.arena = bytearray()
        self.ro = bytearray()

    def put(self, data, ro=False, pad=0) -> int:
        buf = self.ro if ro else self.arena
        off = F.align_up(len(buf))
        buf.extend(b"\0" * (off - len(buf)))
        raw = np.ascontiguousarray(data).tobytes()
        buf.extend(raw)
        buf.extend(b"\xAB" * pad)       # canary padding after the operand
        return off | (F.RODATA_BIT if ro else 0)

    def out(self, count, fill=0x7F) -> int:
        """Output slot pre-filled with a NaN-ish pattern so unwritten elements show."""
        off = F.align_up(len(self.arena))
        self.arena.extend(b"\0" * (off - len(self.arena)))
        self.arena.extend(bytes([fill]) * (count * 4))
        self.arena.extend(b"\xAB" * 64)
        return off

    def done(self):
        a = np.frombuffer(bytes(self.arena), dtype=np.uint8).copy()
        r = np.frombuffer(bytes(self.ro), dtype=np.uint8).copy()
        pad = F.align_up(a.size) - a.size
        if pad:
            a = np.concatenate([a, np.zeros(pad, np.uint8)])
        return a, r


def _ins(op, ins=(), outs=(), flags=0):
    i = np.zeros(1, dtype=F.INSTR_DTYPE)
    i["in"] = F.NULL_REF
    i["opcode"], i["flags"] = int(op), flags
    for k, w in enumerate(ins):
        i["in"][0, k] = w
    for k, w in enumerate(outs):
        i["out"][0, k] = w
    return i


def _rn(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


def gemm_cases(rng, big=False):
    cases = []
    shapes = [(2, 2, 3), (33, 29, 21), (64, 64, 64), (5, 10, 256), (32, 512, 256), (128, 16, 40),
              (70, 130, 33), (1, 7, 9)]
    if big:
        shapes += [(256, 384, 512), (512, 1024, 256), (300, 200, 1000)]
    for (M, N, K) in shapes:
        for op in (Op.GEMM_NN, Op.GEMM_NT, Op.GEMM_TN, Op.GEMM_ACC_NN):
            for ro in ((False, True) if op in (Op.GEMM_NN, Op.GEMM_NT) else (False,)):
                L = Layout()
                A = _rn(rng, K, M) if op == Op.GEMM_TN else _rn(rng, M, K)
                B = _rn(rng, N, K) if op == Op.GEMM_NT else _rn(rng, K, N)
                a, b = L.put(A), L.put(B, ro=ro)
                if op == Op.GEMM_ACC_NN:
                    c = L.put(_rn(rng, M, N))
                    ins = _ins(op, [a, b, c, F.f32_bits(0.75)], [M, N, K])
                else:
                    c = L.out(M * N)
                    ins = _ins(op, [a, b, c], [M, N, K])
                ar, r = L.done()
                cases.append(Case(f"{op.name}_{M}x{N}x{K}{'_ro' if ro else ''}", ins, ar, r,
                                  {"C": (c, M * N, np.float32)}))
    # split-K territory: few tiles, long reduction (the LoRA wgrad shape)
    for (M, N, K) in [(16, 48, 4100), (40, 8, 8192)] + ([(1024, 16, 16384)] if big else []):
        L = Layout()
        a, b = L.put(_rn(rng, K, M)), L.put(_rn(rng, K, N))
        c = L.out(M * N)
        ar, r = L.done()
        cases.append(Case(f"GEMM_TN_splitk_{M}x{N}x{K}", _ins(Op.GEMM_TN, [a, b, c], [M, N, K]), ar, r,
                          {"C": (c, M * N, np.float32)}, rtol=2e-3, atol=2e-3))
    # rank-r shapes: narrow output, tiny reduction, long skinny TN (the LoRA factor GEMMs)
    for (M, N, K) in [(300, 16, 520), (200, 8, 132), (70, 32, 256), (200, 132, 16), (65, 260, 8), (40, 68, 31)]:
        for op in (Op.GEMM_NN, Op.GEMM_NT):
            L = Layout()
            a = L.put(_rn(rng, M, K))
            b = L.put(_rn(rng, N, K) if op == Op.GEMM_NT else _rn(rng, K, N))
            c = L.out(M * N)
            ar, r = L.done()
            cases.append(Case(f"{op.name}_skinny_{M}x{N}x{K}", _ins(op, [a, b, c], [M, N, K]), ar, r,
                              {"C": (c, M * N, np.float32)}))
    for (M, N, K) in [(16, 200, 2100), (200, 8, 1500), (130, 64, 1024), (4, 70, 1030)]:
        L = Layout()
        a, b = L.put(_rn(rng, K, M)), L.put(_rn(rng, K, N))
        c = L.out(M * N)
        ar, r = L.done()
        cases.append(Case(f"GEMM_TN_skinny_{M}x{N}x{K}", _ins(Op.GEMM_TN, [a, b, c], [M, N, K]), ar, r,
                          {"C": (c, M * N, np.float32)}, rtol=1e-3, atol=5e-4))
    # fused epilogues on GEMM_NN: bias and/or activation
    for act in (0, 1, 2, 3):
        for bias in (False, True):
            if act == 0 and not bias:
                continue
            M, N, K = 17, 24, 31
            L = Layout()
            a, b = L.put(_rn(rng, M, K)), L.put(_rn(rng, K, N), ro=True)
            bb = L.put(_rn(rng, N), ro=True)
            c = L.out(M * N)
            ins = _ins(Op.GEMM_NN, [a, b, c] + ([bb] if bias else []), [M, N, K],
                       flags=(1 if bias else 0) | (act << 1))
            ar, r = L.done()
            cases.append(Case(f"GEMM_NN_epi_b{int(bias)}_a{act}", ins, ar, r, {"C": (c, M * N, np.float32)}))
    # int8 frozen weights
    for op in (Op.GEMM_NN_Q8, Op.GEMM_NT_Q8):
        M, N, K = 19, 22, 37
        L = Layout()
        a = L.put(_rn(rng, M, K))
        q = rng.integers(-127, 128, size=(N, K) if op == Op.GEMM_NT_Q8 else (K, N)).astype(np.int8)
        b = L.put(q, ro=True)
        c = L.out(M * N)
        ins = _ins(op, [a, b, c, F.f32_bits(0.0123)], [M, N, K], flags=(2 << 1) if op == Op.GEMM_NN_Q8 else 0)
        ar, r = L.done()
        cases.append(Case(f"{op.name}", ins, ar, r, {"C": (c, M * N, np.float32)}))
    if big:
        # LoRA-factor shapes long enough for the tensor-core rank-r kernels (ragged M and K included)
        for (M, N, K) in [(2048, 16, 1024), (1100, 32, 520), (1024, 64, 256)]:
            for op in (Op.GEMM_NN, Op.GEMM_NT):
                L = Layout()
                a = L.put(_rn(rng, M, K))
                b = L.put(_rn(rng, N, K) if op == Op.GEMM_NT else _rn(rng, K, N))
                c = L.out(M * N)
                ar, r = L.done()
                cases.append(Case(f"{op.name}_rank_{M}x{N}x{K}", _ins(op, [a, b, c], [M, N, K]), ar, r,
                                  {"C": (c, M * N, np.float32)}))
        for (M, N, K) in [(16, 256, 4096), (384, 32, 8192), (128, 64, 4096)]:
            L = Layout()
            a, b = L.put(_rn(rng, K, M)), L.put(_rn(rng, K, N))
            c = L.out(M * N)
            ar, r = L.done()
            cases.append(Case(f"GEMM_TN_rank_{M}x{N}x{K}", _ins(Op.GEMM_TN, [a, b, c], [M, N, K]), ar, r,
                              {"C": (c, M * N, np.float32)}, rtol=1e-3, atol=5e-4))
    return cases


def elementwise_cases(rng):
    cases = []
    for n in (1, 3, 4, 5, 1000, 32768 + 7):
        for op in (Op.ADD, Op.MUL, Op.RELU_BWD, Op.GELU_BWD, Op.SILU_BWD):
            L = Layout()
            x, y = L.put(_rn(rng, n, scale=2.0)), L.put(_rn(rng, n, scale=2.0))
            o = L.out(n)
            ar, r = L.done()
            cases.append(Case(f"{op.name}_{n}", _ins(op, [x, y, o], [n]), ar, r,
                              {"o": (o, n, np.float32)}, exact=op in (Op.ADD, Op.MUL, Op.RELU_BWD),
                              rtol=1e-5, atol=1e-6))
        for op in (Op.RELU_FWD, Op.GELU_FWD, Op.SILU_FWD, Op.COPY):
            L = Layout()
            x = L.put(_rn(rng, n, scale=3.0))
            o = L.out(n)
            ar, r = L.done()
            cases.append(Case(f"{op.name}_{n}", _ins(op, [x, o], [n]), ar, r, {"o": (o, n, np.float32)},
                              exact=op in (Op.RELU_FWD, Op.COPY), rtol=1e-5, atol=1e-6))
        L = Layout()
        x = L.put(_rn(rng, n))
        o = L.out(n)
        ar, r = L.done()
        cases.append(Case(f"SCALE_{n}", _ins(Op.SCALE, [x, o, F.f32_bits(1.7)], [n]), ar, r,
                          {"o": (o, n, np.float32)}, exact=True))
        L = Layout()
        o = L.out(n)
        ar, r = L.done()
        cases.append(Case(f"FILL_{n}", _ins(Op.FILL, [o, F.f32_bits(1.0)], [n]), ar, r,
                          {"o": (o, n, np.float32)}, exact=True))
    # saturated GELU backward: huge |x| must not produce NaN
    L = Layout()
    xs = np.array([1e30, -1e30, 3e38, -3e38, 50.0, -50.0, 0.0, 1e-30], np.float32)
    dy, x = L.put(np.ones_like(xs)), L.put(xs)
    o = L.out(xs.size)
    ar, r = L.done()
    cases.append(Case("GELU_BWD_saturated", _ins(Op.GELU_BWD, [dy, x, o], [xs.size]), ar, r,
                      {"o": (o, xs.size, np.float32)}, rtol=1e-5, atol=1e-6))
    for rows, cols in ((1, 1), (7, 10), (32, 512), (5, 33)):
        L = Layout()
        x, b = L.put(_rn(rng, rows, cols)), L.put(_rn(rng, cols), ro=True)
        o = L.out(rows * cols)
        ar, r = L.done()
        cases.append(Case(f"ADD_BIAS_{rows}x{cols}", _ins(Op.ADD_BIAS, [x, b, o], [rows, cols]), ar, r,
                          {"o": (o, rows * cols, np.float32)}, exact=True))
        L = Layout()
        x = L.put(_rn(rng, rows, cols))
        o = L.out(cols)
        ar, r = L.done()
        cases.append(Case(f"REDUCE_ROWS_{rows}x{cols}", _ins(Op.REDUCE_ROWS, [x, o], [rows, cols]), ar, r,
                          {"o": (o, cols, np.float32)}, exact=True))
    for T, V, D in ((1, 3, 2), (37, 50, 12), (64, 512, 128), (9, 5, 7)):
        L = Layout()
        tok = L.put(rng.integers(0, V, size=T).astype(np.int32))
        tab = L.put(_rn(rng, V, D), ro=True)
        o = L.out(T * D)
        ar, r = L.done()
        cases.append(Case(f"EMBED_{T}x{V}x{D}", _ins(Op.EMBED, [tok, tab, o], [T, F.pack32(V, D)]), ar, r,
                          {"o": (o, T * D, np.float32)}, exact=True))
    return cases


def norm_cases(rng):
    cases = []
    for rows, cols in ((1, 1), (3, 5), (16, 128), (7, 1000), (2, 4096), (5, 2500)):
        x = _rn(rng, rows, cols, scale=2.0) + 0.5
        g, b = 1.0 + 0.1 * _rn(rng, cols), 0.1 * _rn(rng, cols)
        dy = _rn(rng, rows, cols)
        # LayerNorm fwd
        L = Layout()
        rx, rg, rb = L.put(x), L.put(g, ro=True), L.put(b, ro=True)
        y, mean, rstd = L.out(rows * cols), L.out(rows), L.out(rows)
        ar, r = L.done()
        cases.append(Case(f"LAYERNORM_FWD_{rows}x{cols}",
                          _ins(Op.LAYERNORM_FWD, [rx, rg, rb, y], [F.pack32(rows, cols), mean, rstd]), ar, r,
                          {"y": (y, rows * cols, np.float32), "mean": (mean, rows, np.float32),
                           "rstd": (rstd, rows, np.float32)}, rtol=1e-5, atol=1e-5))
        mu = x.mean(1).astype(np.float32)
        rs = (1.0 / np.sqrt(x.var(1) + 1e-5)).astype(np.float32)
        L = Layout()
        rdy, rx, rg = L.put(dy), L.put(x), L.put(g, ro=True)
        rmu, rrs = L.put(mu), L.put(rs)
        dx = L.out(rows * cols)
        ar, r = L.done()
        cases.append(Case(f"LAYERNORM_BWD_{rows}x{cols}",
                          _ins(Op.LAYERNORM_BWD, [rdy, rx, rg, dx], [rmu, rrs, F.pack32(rows, cols)]), ar, r,
                          {"dx": (dx, rows * cols, np.float32)}, rtol=1e-4, atol=1e-5))
        # RMSNorm
        L = Layout()
        rx, rg = L.put(x), L.put(g, ro=True)
        y, rstd = L.out(rows * cols), L.out(rows)
        ar, r = L.done()
        cases.append(Case(f"RMSNORM_FWD_{rows}x{cols}",
                          _ins(Op.RMSNORM_FWD, [rx, rg, y, rstd], [F.pack32(rows, cols)]), ar, r,
                          {"y": (y, rows * cols, np.float32), "rstd": (rstd, rows, np.float32)},
                          rtol=1e-5, atol=1e-5))
        rs2 = (1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(1) + 1e-5)).astype(np.float32)
        L = Layout()
        rdy, rx, rg, rrs = L.put(dy), L.put(x), L.put(g, ro=True), L.put(rs2)
        dx = L.out(rows * cols)
        ar, r = L.done()
        cases.append(Case(f"RMSNORM_BWD_{rows}x{cols}",
                          _ins(Op.RMSNORM_BWD, [rdy, rx, rg, dx], [rrs, F.pack32(rows, cols)]), ar, r,
                          {"dx": (dx, rows * cols, np.float32)}, rtol=1e-4, atol=1e-5))
    # zero-variance row (LayerNorm eps keeps it finite)
    L = Layout()
    x = np.full((2, 8), 3.0, np.float32)
    rx, rg, rb = L.put(x), L.put(np.ones(8, np.float32), ro=True), L.put(np.zeros(8, np.float32), ro=True)
    y, mean, rstd = L.out(16), L.out(2), L.out(2)
    ar, r = L.done()
    cases.append(Case("LAYERNORM_FWD_zero_variance",
                      _ins(Op.LAYERNORM_FWD, [rx, rg, rb, y], [F.pack32(2, 8), mean, rstd]), ar, r,
                      {"y": (y, 16, np.float32), "rstd": (rstd, 2, np.float32)}, rtol=1e-5, atol=1e-5))
    return cases


def attention_cases(rng, big=False):
    cases = []
    geos = [(1, 1, 1, 2), (2, 5, 2, 4), (1, 33, 3, 6), (2, 64, 2, 32), (1, 70, 1, 64)]
    if big:
        geos += [(2, 128, 4, 64), (1, 512, 2, 64)]
    for (B, S, H, d) in geos:
        T, D = B * S, H * d
        q, k, v, dO = (_rn(rng, T, D) for _ in range(4))
        bs, hd = F.pack32(B, S), F.pack32(H, d)
        for op in (Op.ROPE_FWD, Op.ROPE_BWD):
            L = Layout()
            x = L.put(q)
            y = L.out(T * D)
            ar, r = L.done()
            cases.append(Case(f"{op.name}_{B}x{S}x{H}x{d}", _ins(op, [x, y], [bs, hd, F.f32_bits(10000.0)]),
                              ar, r, {"y": (y, T * D, np.float32)}, rtol=1e-6, atol=1e-6, exact=True))
        L = Layout()
        rq, rk, rv = L.put(q), L.put(k), L.put(v)
        o, P = L.out(T * D), L.out(B * H * S * S)
        ar, r = L.done()
        cases.append(Case(f"ATTN_FWD_{B}x{S}x{H}x{d}", _ins(Op.ATTN_FWD, [rq, rk, rv, o], [P, bs, hd]), ar, r,
                          {"o": (o, T * D, np.float32), "P": (P, B * H * S * S, np.float32)},
                          rtol=1e-4, atol=1e-5))
        # a valid causal P / dS for the backward primitives
        Pm = np.zeros((B * H, S, S), np.float32)
        for z in range(B * H):
            for i in range(S):
                e = rng.random(i + 1).astype(np.float32) + 0.01
                Pm[z, i, :i + 1] = e / e.sum()
        dSm = np.tril(_rn(rng, B * H, S, S))
        L = Layout()
        rdo, rv = L.put(dO), L.put(v)
        dP = L.out(B * H * S * S)
        ar, r = L.done()
        cases.append(Case(f"ATTN_DP_{B}x{S}x{H}x{d}", _ins(Op.ATTN_DP, [rdo, rv, dP], [bs, hd]), ar, r,
                          {"dP": (dP, B * H * S * S, np.float32)}, rtol=1e-4, atol=1e-5))
        for op, lhs, rhs in ((Op.ATTN_DV, Pm, dO), (Op.ATTN_DQ, dSm, k), (Op.ATTN_DK, dSm, q)):
            L = Layout()
            a, b = L.put(lhs), L.put(rhs)
            o = L.out(T * D)
            ar, r = L.done()
            cases.append(Case(f"{op.name}_{B}x{S}x{H}x{d}", _ins(op, [a, b, o], [bs, hd]), ar, r,
                              {"o": (o, T * D, np.float32)}, rtol=1e-4, atol=1e-5))
        L = Layout()
        rp, rdp = L.put(Pm), L.put(np.tril(_rn(rng, B * H, S, S)))
        ds = L.out(B * H * S * S)
        ar, r = L.done()
        cases.append(Case(f"SOFTMAX_ROWS_BWD_{B}x{S}x{H}x{d}",
                          _ins(Op.SOFTMAX_ROWS_BWD, [rp, rdp, ds], [F.pack32(B * H * S, S)]), ar, r,
                          {"dS": (ds, B * H * S * S, np.float32)}, rtol=1e-5, atol=1e-6))
    return cases


def loss_cases(rng):
    cases = []
    for N, C in ((1, 2), (32, 10), (7, 33), (300, 5), (64, 512), (9, 5000), (4, 40000)):
        logits = _rn(rng, N, C, scale=3.0)
        labels = rng.integers(0, C, size=N).astype(np.int32)
        L = Layout()
        rl, rlab = L.put(logits), L.put(labels)
        loss, probs = L.out(1), L.out(N * C)
        ar, r = L.done()
        cases.append(Case(f"XENT_FWD_{N}x{C}", _ins(Op.XENT_FWD, [rl, rlab, loss, probs], [N, C]), ar, r,
                          {"loss": (loss, 1, np.float32), "probs": (probs, N * C, np.float32)},
                          rtol=2e-4, atol=1e-7))   # the reference sums the denominator serially in f32
        p = np.exp(logits - logits.max(1, keepdims=True))
        p = (p / p.sum(1, keepdims=True)).astype(np.float32)
        L = Layout()
        rp, rlab, seed = L.put(p), L.put(labels), L.put(np.array([1.0], np.float32))
        d = L.out(N * C)
        ar, r = L.done()
        cases.append(Case(f"XENT_BWD_{N}x{C}", _ins(Op.XENT_BWD, [rp, rlab, seed, d], [N, C]), ar, r,
                          {"d": (d, N * C, np.float32)}, exact=True))
        # KL distillation
        L = Layout()
        rs, rt = L.put(logits), L.put(_rn(rng, N, C, scale=3.0))
        loss, ps, pt = L.out(1), L.out(N * C), L.out(N * C)
        ar, r = L.done()
        cases.append(Case(f"KL_FWD_{N}x{C}",
                          _ins(Op.KL_FWD, [rs, rt, loss, ps], [pt, F.pack32(N, C), F.f32_bits(2.0)]), ar, r,
                          {"loss": (loss, 1, np.float32), "ps": (ps, N * C, np.float32),
                           "pt": (pt, N * C, np.float32)}, rtol=2e-4, atol=1e-7))
        L = Layout()
        rps, rpt, seed = L.put(p), L.put(p[::-1].copy()), L.put(np.array([0.5], np.float32))
        d = L.out(N * C)
        ar, r = L.done()
        cases.append(Case(f"KL_BWD_{N}x{C}",
                          _ins(Op.KL_BWD, [rps, rpt, seed, d], [F.pack32(N, C), F.f32_bits(2.0)]), ar, r,
                          {"d": (d, N * C, np.float32)}, exact=True))
    for n in (1, 5, 1000, 32768 * 2 + 11):
        pr, tg = _rn(rng, n), _rn(rng, n)
        L = Layout()
        a, b = L.put(pr), L.put(tg)
        loss = L.out(1)
        ar, r = L.done()
        cases.append(Case(f"MSE_FWD_{n}", _ins(Op.MSE_FWD, [a, b, loss], [n]), ar, r,
                          {"loss": (loss, 1, np.float32)}, rtol=1e-6, atol=1e-7))
        L = Layout()
        a, b, seed = L.put(pr), L.put(tg), L.put(np.array([1.0], np.float32))
        d = L.out(n)
        ar, r = L.done()
        cases.append(Case(f"MSE_BWD_{n}", _ins(Op.MSE_BWD, [a, b, seed, d], [n]), ar, r,
                          {"d": (d, n, np.float32)}, exact=True))
    # NaN logits must surface as a NaN loss, not a clamped finite one
    L = Layout()
    lg = _rn(rng, 4, 6)
    lg[2, 3] = np.nan
    rl, rlab = L.put(lg), L.put(np.array([0, 1, 3, 2], np.int32))
    loss, probs = L.out(1), L.out(24)
    ar, r = L.done()
    cases.append(Case("XENT_FWD_nan", _ins(Op.XENT_FWD, [rl, rlab, loss, probs], [4, 6]), ar, r,
                      {"loss": (loss, 1, np.float32), "probs": (probs, 24, np.float32)}))
    return cases


def optimizer_cases(rng):
    cases = []
    for n in (1, 3, 16, 4099, 32768 + 5):
        p, g = _rn(rng, n), _rn(rng, n, scale=0.1)
        m, v = _rn(rng, n, scale=0.01), np.abs(_rn(rng, n, scale=0.001))
        for step in (1, 2, 1000):
            L = Layout()
            rp, rg, rm, rv = L.put(p), L.put(g), L.put(m), L.put(v)
            ar, r = L.done()
            cases.append(Case(f"ADAMW_{n}_step{step}", _ins(Op.ADAMW, [rp, rg, rm, rv], [n]), ar, r,
                              {"p": (rp, n, np.float32), "m": (rm, n, np.float32), "v": (rv, n, np.float32)},
                              scalars=dict(lr=3e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, step=step),
                              exact=True))
        L = Layout()
        rp, rg = L.put(p), L.put(g)
        ar, r = L.done()
        cases.append(Case(f"SGD_{n}", _ins(Op.SGD, [rp, rg], [n]), ar, r, {"p": (rp, n, np.float32)},
                          scalars=dict(lr=1e-2, wd=0.1), exact=True))
        for mx in (1e-3, 1e6, 0.0):
            L = Layout()
            rg = L.put(g)
            ar, r = L.done()
            cases.append(Case(f"CLIP_NORM_{n}_{mx}", _ins(Op.CLIP_NORM, [rg, F.f32_bits(mx)], [n]), ar, r,
                              {"g": (rg, n, np.float32)}, rtol=1e-6, atol=1e-9))
    return cases


def all_cases(seed=1234, big=False):
    rng = np.random.default_rng(seed)
    return (gemm_cases(rng, big) + elementwise_cases(rng) + norm_cases(rng) + attention_cases(rng, big)
            + loss_cases(rng) + optimizer_cases(rng))


def read_output(arena: np.ndarray, spec):
    off, count, dt = spec
    return arena[off:off + count * 4].view(dt).copy()

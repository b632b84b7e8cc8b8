"""Plan synthesiser: frozen model graph + LoRA/optimiser request -> sealed SEEU plan.

The backend executes *plans*; this module exists so that the bench and the
parity tests can produce them for any synthetic configuration without the
reference toolchain (which does not travel to the GPU box). It emits the same
instruction patterns the reference compiler emits, so the plans load in the
reference runtime too (checked by tests against the reference itself):

* forward graph over the SMF op vocabulary (reference:
  compiler/frontend/parser/parser.cc:12-253),
* softmax-xent / MSE loss graft (compiler/driver/update_compiler.cc:131-199),
* LoRA graft  C' = C + (alpha/r)*(X@A)@B  (compiler/analysis/algebra/lora_grafter.cc:24-178),
* reverse-mode autodiff pruned to the adapters
  (compiler/analysis/calculus/autodiff.cc:66-444),
* AdamW / SGD step per trainable tensor, sorted by id
  (compiler/analysis/calculus/optimizer.cc:12-57),
* merge program  delta = (alpha/r) A@B  (compiler/analysis/algebra/merge_builder.cc:12-68),
* optional GEMM-epilogue fusion (compiler/analysis/algebra/epilogue_fuser.cc:36-118),
* arena binding [persistent | io | transient] with first-fit liveness reuse
  (compiler/backend/trainer/arena_binder.cc:25-185),
* lowering to 64-byte instructions (compiler/backend/trainer/instruction_lowering.cc:18-349),
* counter-based SplitMix64 + Box-Muller initial adapter image
  (compiler/driver/update_compiler.cc:411-442).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import formats as F
from .formats import Op


# --- a small SSA IR -------------------------------------------------------------
class Value:
    __slots__ = ("id", "shape", "dtype", "def_op")

    def __init__(self, id_, shape, dtype="f32", def_op=None):
        self.id, self.shape, self.dtype, self.def_op = id_, tuple(int(d) for d in shape), dtype, def_op

    @property
    def volume(self):
        v = 1
        for d in self.shape:
            v *= d
        return v

    @property
    def nbytes(self):
        return self.volume * 4


class Node:
    __slots__ = ("mn", "operands", "results", "attrs")

    def __init__(self, mn, operands=(), attrs=None):
        self.mn, self.operands, self.results, self.attrs = mn, list(operands), [], dict(attrs or {})

    def add_result(self, id_, shape, dtype="f32"):
        v = Value(id_, shape, dtype, self)
        self.results.append(v)
        return v


class Block:
    def __init__(self):
        self.args: list[Value] = []
        self.ops: list[Node] = []

    def append(self, mn, operands=(), attrs=None) -> Node:
        n = Node(mn, operands, attrs)
        self.ops.append(n)
        return n

    def users(self, v: Value):
        return [op for op in self.ops if any(o is v for o in op.operands)]


@dataclass
class TrainSpec:
    """The compilation request (reference: source/plan/config.h:18-81)."""
    batch: int                      # plan rows T (sequences * seq_len for token plans)
    lora_rank: int = 8
    lora_alpha: float = 16.0
    lora_seed: int = 42
    targets: tuple = ()             # substring filters on weight names; () = all
    loss: str = "xent"              # "xent" | "mse"
    optimizer: str = "adamw"        # "adamw" | "sgd"
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    clip_norm: float = 0.0
    lr_schedule: int = 0
    warmup_steps: int = 0
    min_lr_factor: float = 0.0
    default_steps: int = 1000
    fuse_epilogues: bool = True
    emit_optimizer: bool = True
    source_model_hash: int = 0


@dataclass
class SynthInfo:
    """Debug hooks: where parameters, gradients and deltas live in the arena."""
    params: list = field(default_factory=list)     # (id, param_ref, grad_ref, count)
    adapters: list = field(default_factory=list)   # dict per adapter
    values: dict = field(default_factory=dict)     # id -> (ref, shape)


# --- forward graph ----------------------------------------------------------------
def _build_forward(model: F.ModelGraph, batch: int, blk: Block, weights: dict):
    if model.token_input:
        x = Value(model.input_name, (batch,), "i32")
    else:
        x = Value(model.input_name, (batch, model.input_dim))
    blk.args.append(x)
    env = {model.input_name: x}

    def resolve(name):
        if name in env:
            return env[name]
        arr = model.tensors[name]
        n = blk.append("sc_mem.weight")
        v = n.add_result(name, arr.shape)
        weights[v] = name
        env[name] = v
        return v

    for kind, name, inputs, output, attr0 in model.ops:
        ins = [resolve(i) for i in inputs]
        if kind == F.SMF_MATMUL:
            n = blk.append("sc_high.matmul", ins)
            env[output] = n.add_result(output, (ins[0].shape[0], ins[1].shape[1]))
        elif kind == F.SMF_ADDBIAS:
            n = blk.append("sc_high.add_bias", ins)
            env[output] = n.add_result(output, ins[0].shape)
        elif kind in (F.SMF_RELU, F.SMF_GELU, F.SMF_SILU):
            mn = {F.SMF_RELU: "sc_high.relu", F.SMF_GELU: "sc_high.gelu",
                  F.SMF_SILU: "sc_high.silu"}[kind]
            n = blk.append(mn, ins)
            env[output] = n.add_result(output, ins[0].shape)
        elif kind == F.SMF_MUL:
            n = blk.append("sc_high.mul", ins)
            env[output] = n.add_result(output, ins[0].shape)
        elif kind == F.SMF_ADD:
            n = blk.append("sc_high.add", ins)
            env[output] = n.add_result(output, ins[0].shape)
        elif kind == F.SMF_EMBEDDING:
            n = blk.append("sc_high.embedding", ins)
            env[output] = n.add_result(output, (ins[0].shape[0], ins[1].shape[1]))
        elif kind == F.SMF_RMSNORM:
            n = blk.append("sc_high.rms_norm", ins)
            env[output] = n.add_result(output, ins[0].shape)
            n.add_result(output + ".rstd", (ins[0].shape[0],))
        elif kind == F.SMF_LAYERNORM:
            n = blk.append("sc_high.layer_norm", ins)
            env[output] = n.add_result(output, ins[0].shape)
            n.add_result(output + ".mean", (ins[0].shape[0],))
            n.add_result(output + ".rstd", (ins[0].shape[0],))
        elif kind == F.SMF_ROPE:
            n = blk.append("sc_high.rope", ins, {"heads": attr0, "seq": model.seq_len,
                                                 "base": 10000.0})
            env[output] = n.add_result(output, ins[0].shape)
        elif kind == F.SMF_ATTENTION:
            n = blk.append("sc_high.attention", ins, {"heads": attr0, "seq": model.seq_len})
            env[output] = n.add_result(output, ins[0].shape)
            n.add_result(output + ".probs", (ins[0].shape[0] * attr0, model.seq_len))
        else:
            raise ValueError(f"unknown op kind {kind}")
    return x, env[model.output_name]


# --- LoRA graft ---------------------------------------------------------------------
def _graft_lora(blk: Block, spec: TrainSpec, weights: dict):
    targets = []
    for op in blk.ops:
        if op.mn != "sc_high.matmul" or len(op.operands) != 2:
            continue
        w = op.operands[1]
        if w.def_op is None or w.def_op.mn != "sc_mem.weight":
            continue
        if any(u.mn != "sc_high.matmul" or len(u.operands) != 2 or u.operands[1] is not w
               or u.operands[0] is w for u in blk.users(w)):
            continue
        if spec.targets and not any(t in w.id for t in spec.targets):
            continue
        targets.append(op)
    if not targets:
        raise ValueError("no eligible MatMul targets found")
    adapters, by_weight, sites = [], {}, {}
    scale = float(np.float32(spec.lora_alpha) / np.float32(spec.lora_rank))
    r = spec.lora_rank
    for tgt in targets:
        x, w, c = tgt.operands[0], tgt.operands[1], tgt.results[0]
        n, k, m = x.shape[0], w.shape[0], w.shape[1]
        consumers = blk.users(c)
        base = w.id
        site = sites.get(base, 0)
        sites[base] = site + 1
        if site > 0:
            base += f"@{site}"
        new_ops = []
        if w not in by_weight:
            a_op = Node("sc_mem.param", attrs={"trainable": 1, "init": "randn",
                                               "std": float(np.float32(1.0) / np.sqrt(np.float32(k))),
                                               "seed": spec.lora_seed + len(adapters)})
            a = a_op.add_result(base + ".lora_A", (k, r))
            b_op = Node("sc_mem.param", attrs={"trainable": 1, "init": "zeros"})
            b = b_op.add_result(base + ".lora_B", (r, m))
            new_ops += [a_op, b_op]
            by_weight[w] = len(adapters)
            adapters.append(dict(weight=w, A=a, B=b, scale=scale, id_base=base))
        else:
            a, b = adapters[by_weight[w]]["A"], adapters[by_weight[w]]["B"]
        t_op = Node("sc_high.matmul", [x, a])
        t = t_op.add_result(base + ".lora_t", (n, r))
        u_op = Node("sc_high.matmul", [t, b])
        u = u_op.add_result(base + ".lora_u", (n, m))
        s_op = Node("sc_high.scale", [u], {"alpha": scale})
        s = s_op.add_result(base + ".lora_s", (n, m))
        add_op = Node("sc_high.add", [c, s])
        cp = add_op.add_result(base + ".lora_out", (n, m))
        new_ops += [t_op, u_op, s_op, add_op]
        at = blk.ops.index(tgt) + 1
        blk.ops[at:at] = new_ops
        for cons in consumers:
            cons.operands = [cp if o is c else o for o in cons.operands]
    return adapters


# --- autodiff ------------------------------------------------------------------------
def _autodiff(blk: Block, loss: Value, trainables: list):
    needs = set(id(p) for p in trainables)
    for op in blk.ops:
        if any(id(o) in needs for o in op.operands):
            for r in op.results:
                needs.add(id(r))
    if id(loss) not in needs:
        raise ValueError("loss does not depend on any trainable parameter")
    adj: dict[int, Value] = {}
    counter = [0]

    def fresh():
        counter[0] += 1
        return counter[0] - 1

    def need(v):
        return id(v) in needs

    def accumulate(primal, grad):
        if not need(primal):
            return
        if id(primal) not in adj:
            adj[id(primal)] = grad
            return
        n = blk.append("sc_high.add", [adj[id(primal)], grad])
        adj[id(primal)] = n.add_result(f"{primal.id}.grad_acc{fresh()}", grad.shape)

    def emit1(mn, operands, like, attrs=None):
        n = blk.append(mn, operands, attrs)
        return n.add_result(f"{like.id}.d{fresh()}", like.shape)

    seed = blk.append("sc_low.fill", attrs={"value": 1.0}).add_result(loss.id + ".seed", loss.shape)
    adj[id(loss)] = seed
    for op in reversed(list(blk.ops)):
        if op.mn.startswith("sc_mem.") or not op.results or id(op.results[0]) not in adj:
            continue
        if not any(need(o) for o in op.operands):
            continue
        g = adj[id(op.results[0])]
        mn = op.mn
        if mn == "sc_high.matmul":
            x, w = op.operands[0], op.operands[1]
            if need(x):
                accumulate(x, emit1("sc_low.matmul_nt", [g, w], x))
            if need(w):
                accumulate(w, emit1("sc_low.matmul_tn", [x, g], w))
        elif mn == "sc_high.add":
            accumulate(op.operands[0], g)
            accumulate(op.operands[1], g)
        elif mn == "sc_high.add_bias":
            accumulate(op.operands[0], g)
            if need(op.operands[1]):
                accumulate(op.operands[1], emit1("sc_low.reduce_rows", [g], op.operands[1]))
        elif mn in ("sc_high.relu", "sc_high.gelu", "sc_high.silu"):
            x = op.operands[0]
            accumulate(x, emit1("sc_low." + mn.split(".")[1] + "_grad", [g, x], x))
        elif mn == "sc_high.mul":
            x, y = op.operands
            if need(x):
                accumulate(x, emit1("sc_low.mul", [g, y], x))
            if need(y):
                accumulate(y, emit1("sc_low.mul", [g, x], y))
        elif mn == "sc_high.layer_norm":
            x = op.operands[0]
            if need(x):
                accumulate(x, emit1("sc_low.layer_norm_grad",
                                    [g, x, op.operands[1], op.results[1], op.results[2]], x))
        elif mn == "sc_high.rms_norm":
            x = op.operands[0]
            if need(x):
                accumulate(x, emit1("sc_low.rms_norm_grad", [g, x, op.operands[1], op.results[1]], x))
        elif mn == "sc_high.rope":
            x = op.operands[0]
            if need(x):
                accumulate(x, emit1("sc_low.rope_grad", [g], x, dict(op.attrs)))
        elif mn == "sc_high.attention":
            q, k, v = op.operands
            probs = op.results[1]
            at = dict(op.attrs)
            if need(v):
                accumulate(v, emit1("sc_low.attn_dv", [probs, g], v, at))
            if need(q) or need(k):
                dp = emit1("sc_low.attn_dp", [g, v], probs, at)
                ds = emit1("sc_low.softmax_rows_grad", [probs, dp], probs, at)
                if need(q):
                    accumulate(q, emit1("sc_low.attn_dq", [ds, k], q, at))
                if need(k):
                    accumulate(k, emit1("sc_low.attn_dk", [ds, q], k, at))
        elif mn == "sc_high.scale":
            x = op.operands[0]
            accumulate(x, emit1("sc_low.scale", [g], x, {"alpha": op.attrs["alpha"]}))
        elif mn == "sc_high.softmax_xent":
            logits, labels = op.operands
            if need(logits):
                accumulate(logits, emit1("sc_low.softmax_xent_grad",
                                         [op.results[1], labels, g], logits))
        elif mn == "sc_high.mse":
            pred, target = op.operands
            if need(pred):
                accumulate(pred, emit1("sc_low.mse_grad", [pred, target, g], pred))
        elif mn == "sc_high.embedding":
            pass
        else:
            raise ValueError(f"no VJP rule for {mn}")
    grads = {}
    for p in trainables:
        if id(p) not in adj:
            raise ValueError(f"no gradient reached {p.id}")
        grads[id(p)] = (p, adj[id(p)])
    return grads


def _synth_optimizer(blk: Block, grads: dict, spec: TrainSpec):
    for p, g in sorted(grads.values(), key=lambda pg: pg[0].id):
        if spec.clip_norm > 0:
            blk.append("sc_low.clip_norm", [g], {"max_norm": spec.clip_norm})
        if spec.optimizer == "sgd":
            blk.append("sc_low.sgd_step", [p, g])
            continue
        m = blk.append("sc_mem.param", attrs={"init": "zeros"}).add_result(p.id + ".adam_m", p.shape)
        v = blk.append("sc_mem.param", attrs={"init": "zeros"}).add_result(p.id + ".adam_v", p.shape)
        blk.append("sc_low.adamw_step", [p, g, m, v])


_ACT_OF = {"sc_high.relu": "relu", "sc_high.gelu": "gelu", "sc_high.silu": "silu"}


def _fuse_epilogues(blk: Block, protected: set, primal_ops: list):
    """GEMM -> AddBias -> activation chains fold into a flagged GEMM when the
    intermediates have no other reader."""
    dead = []

    def replace_uses(old, new):
        for op in blk.ops:
            op.operands = [new if o is old else o for o in op.operands]

    for gemm in list(blk.ops):
        if gemm.mn != "sc_high.matmul" or len(gemm.operands) != 2 or len(gemm.results) != 1:
            continue
        c = gemm.results[0]
        users = blk.users(c)
        if len(users) != 1 or id(c) in protected:
            continue
        user = users[0]
        if user.mn == "sc_high.add_bias" and user.operands[0] is c:
            y, bias = user.results[0], user.operands[1]
            bdef = bias.def_op
            if bdef is not None and blk.ops.index(bdef) > blk.ops.index(gemm):
                if not bdef.mn.startswith("sc_mem."):
                    continue
                blk.ops.remove(bdef)
                blk.ops.insert(blk.ops.index(gemm), bdef)
            yu = blk.users(y)
            act = yu[0] if len(yu) == 1 else None
            if (act is not None and act.mn in _ACT_OF and len(act.operands) == 1
                    and id(y) not in protected and id(act.results[0]) not in protected):
                gemm.operands.append(bias)
                gemm.attrs["epilogue_act"] = _ACT_OF[act.mn]
                replace_uses(act.results[0], c)
                dead += [user, act]
            elif id(y) not in protected:
                gemm.operands.append(bias)
                replace_uses(y, c)
                dead.append(user)
        elif user.mn in _ACT_OF and len(user.operands) == 1 and id(user.results[0]) not in protected:
            gemm.attrs["epilogue_act"] = _ACT_OF[user.mn]
            replace_uses(user.results[0], c)
            dead.append(user)
    for d in dead:
        blk.ops.remove(d)
        if d in primal_ops:
            primal_ops.remove(d)


# --- arena binding ----------------------------------------------------------------------
def _linear_scan(ops, base, bound: dict, pinned: set, refs: dict):
    birth, death, order = {}, {}, []
    for tick, op in enumerate(ops):
        if not op.mn.startswith("sc_mem."):
            for r in op.results:
                if id(r) in bound:
                    continue
                birth[id(r)] = death[id(r)] = tick
                order.append(r)
        for o in op.operands:
            if id(o) in death:
                death[id(o)] = tick
    INF = 1 << 62
    ivs = [(birth[id(v)], INF if id(v) in pinned else death[id(v)], F.align_up(v.nbytes), v)
           for v in order]
    ivs.sort(key=lambda t: t[0])          # stable: ties keep discovery order
    active = []                           # (start, end, free_after) sorted by start
    high = base
    for start_tick, end_tick, nbytes, v in ivs:
        active = [ab for ab in active if ab[2] == INF or ab[2] >= start_tick]
        off = base
        for s, e, _ in active:
            if off + nbytes <= s:
                break
            off = max(off, e)
        refs[id(v)] = off
        pos = 0
        while pos < len(active) and active[pos][0] <= off:
            pos += 1
        active.insert(pos, (off, off + nbytes, end_tick))
        high = max(high, off + nbytes)
    return high


def _counter_randn(seed: int, count: int, std: float) -> np.ndarray:
    """Element j = f(seed, j): two SplitMix64 draws -> Box-Muller, times std."""
    G = np.uint64(0x9E3779B97F4A7C15)
    with np.errstate(over="ignore"):
        idx = np.arange(count, dtype=np.uint64)
        s = np.uint64(seed) + G * (np.uint64(2) * idx + np.uint64(1))

        def nxt(s):
            s = s + G
            z = s
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            return s, z ^ (z >> np.uint64(31))
        s, z1 = nxt(s)
        s, z2 = nxt(s)
    u1 = ((z1 >> np.uint64(11)).astype(np.float64) + 1.0) * 2.0 ** -53
    u2 = (z2 >> np.uint64(11)).astype(np.float64) * 2.0 ** -53
    g = (np.sqrt(-2.0 * np.log(u1)) * np.cos(6.283185307179586476925286766559 * u2)).astype(np.float32)
    return g * np.float32(std)


# --- lowering ----------------------------------------------------------------------------
def _lower(ops, ref_of):
    out = []
    for op in ops:
        mn = op.mn
        if mn.startswith("sc_mem."):
            continue
        ins = np.zeros((), dtype=F.INSTR_DTYPE)
        ins["in"] = F.NULL_REF
        R = ref_of
        o, r = op.operands, op.results

        def setop(code, in_=(), out_=()):
            ins["opcode"] = int(code)
            for i, w in enumerate(in_):
                ins["in"][i] = w
            for i, w in enumerate(out_):
                ins["out"][i] = w
        if mn in ("sc_high.matmul", "sc_low.matmul_nt", "sc_low.matmul_tn"):
            c = r[0]
            code = {"sc_high.matmul": Op.GEMM_NN, "sc_low.matmul_nt": Op.GEMM_NT,
                    "sc_low.matmul_tn": Op.GEMM_TN}[mn]
            kdim = o[0].shape[0] if mn == "sc_low.matmul_tn" else o[0].shape[1]
            setop(code, [R(o[0]), R(o[1]), R(c)], [c.shape[0], c.shape[1], kdim])
            bias = mn == "sc_high.matmul" and len(o) == 3
            if bias:
                ins["in"][3] = R(o[2])
            act = {"relu": 1, "gelu": 2, "silu": 3}.get(op.attrs.get("epilogue_act"), 0)
            ins["flags"] = (1 if bias else 0) | (act << 1)
        elif mn == "sc_low.gemm_acc":
            setop(Op.GEMM_ACC_NN, [R(o[0]), R(o[1]), R(o[2]), F.f32_bits(op.attrs["alpha"])],
                  [o[0].shape[0], o[1].shape[1], o[0].shape[1]])
        elif mn == "sc_high.add":
            setop(Op.ADD, [R(o[0]), R(o[1]), R(r[0])], [r[0].volume])
        elif mn in ("sc_high.mul", "sc_low.mul"):
            setop(Op.MUL, [R(o[0]), R(o[1]), R(r[0])], [r[0].volume])
        elif mn == "sc_high.add_bias":
            setop(Op.ADD_BIAS, [R(o[0]), R(o[1]), R(r[0])], [r[0].shape[0], r[0].shape[1]])
        elif mn in ("sc_high.relu", "sc_high.gelu", "sc_high.silu"):
            code = {"sc_high.relu": Op.RELU_FWD, "sc_high.gelu": Op.GELU_FWD,
                    "sc_high.silu": Op.SILU_FWD}[mn]
            setop(code, [R(o[0]), R(r[0])], [r[0].volume])
        elif mn in ("sc_low.relu_grad", "sc_low.gelu_grad", "sc_low.silu_grad"):
            code = {"sc_low.relu_grad": Op.RELU_BWD, "sc_low.gelu_grad": Op.GELU_BWD,
                    "sc_low.silu_grad": Op.SILU_BWD}[mn]
            setop(code, [R(o[0]), R(o[1]), R(r[0])], [r[0].volume])
        elif mn == "sc_high.layer_norm":
            setop(Op.LAYERNORM_FWD, [R(o[0]), R(o[1]), R(o[2]), R(r[0])],
                  [F.pack32(*r[0].shape), R(r[1]), R(r[2])])
        elif mn == "sc_low.layer_norm_grad":
            setop(Op.LAYERNORM_BWD, [R(o[0]), R(o[1]), R(o[2]), R(r[0])],
                  [R(o[3]), R(o[4]), F.pack32(*r[0].shape)])
        elif mn == "sc_high.embedding":
            setop(Op.EMBED, [R(o[0]), R(o[1]), R(r[0])], [r[0].shape[0], F.pack32(*o[1].shape)])
        elif mn == "sc_high.rms_norm":
            setop(Op.RMSNORM_FWD, [R(o[0]), R(o[1]), R(r[0]), R(r[1])], [F.pack32(*r[0].shape)])
        elif mn == "sc_low.rms_norm_grad":
            setop(Op.RMSNORM_BWD, [R(o[0]), R(o[1]), R(o[2]), R(r[0])],
                  [R(o[3]), F.pack32(*r[0].shape)])
        elif mn in ("sc_high.rope", "sc_low.rope_grad", "sc_high.attention", "sc_low.attn_dp",
                    "sc_low.attn_dv", "sc_low.attn_dq", "sc_low.attn_dk"):
            act = o[0] if mn in ("sc_high.attention", "sc_low.attn_dp") else r[0]
            heads, seq = op.attrs["heads"], op.attrs["seq"]
            rows, width = act.shape
            assert heads > 0 and seq > 0 and rows % seq == 0 and width % heads == 0
            bs, hd = F.pack32(rows // seq, seq), F.pack32(heads, width // heads)
            if mn in ("sc_high.rope", "sc_low.rope_grad"):
                setop(Op.ROPE_FWD if mn == "sc_high.rope" else Op.ROPE_BWD, [R(o[0]), R(r[0])],
                      [bs, hd, F.f32_bits(op.attrs.get("base", 10000.0))])
            elif mn == "sc_high.attention":
                setop(Op.ATTN_FWD, [R(o[0]), R(o[1]), R(o[2]), R(r[0])], [R(r[1]), bs, hd])
            else:
                code = {"sc_low.attn_dp": Op.ATTN_DP, "sc_low.attn_dv": Op.ATTN_DV,
                        "sc_low.attn_dq": Op.ATTN_DQ, "sc_low.attn_dk": Op.ATTN_DK}[mn]
                setop(code, [R(o[0]), R(o[1]), R(r[0])], [bs, hd])
        elif mn == "sc_low.softmax_rows_grad":
            setop(Op.SOFTMAX_ROWS_BWD, [R(o[0]), R(o[1]), R(r[0])], [F.pack32(*r[0].shape)])
        elif mn == "sc_low.clip_norm":
            setop(Op.CLIP_NORM, [R(o[0]), F.f32_bits(op.attrs["max_norm"])], [o[0].volume])
        elif mn in ("sc_high.scale", "sc_low.scale"):
            setop(Op.SCALE, [R(o[0]), R(r[0]), F.f32_bits(op.attrs["alpha"])], [r[0].volume])
        elif mn == "sc_low.reduce_rows":
            setop(Op.REDUCE_ROWS, [R(o[0]), R(r[0])], [o[0].shape[0], o[0].shape[1]])
        elif mn == "sc_high.softmax_xent":
            setop(Op.XENT_FWD, [R(o[0]), R(o[1]), R(r[0]), R(r[1])], [o[0].shape[0], o[0].shape[1]])
        elif mn == "sc_low.softmax_xent_grad":
            setop(Op.XENT_BWD, [R(o[0]), R(o[1]), R(o[2]), R(r[0])], [r[0].shape[0], r[0].shape[1]])
        elif mn == "sc_high.mse":
            setop(Op.MSE_FWD, [R(o[0]), R(o[1]), R(r[0])], [o[0].volume])
        elif mn == "sc_low.mse_grad":
            setop(Op.MSE_BWD, [R(o[0]), R(o[1]), R(o[2]), R(r[0])], [r[0].volume])
        elif mn == "sc_low.sgd_step":
            setop(Op.SGD, [R(o[0]), R(o[1])], [o[0].volume])
        elif mn == "sc_low.adamw_step":
            setop(Op.ADAMW, [R(o[0]), R(o[1]), R(o[2]), R(o[3])], [o[0].volume])
        elif mn == "sc_low.fill":
            setop(Op.FILL, [R(r[0]), F.f32_bits(op.attrs["value"])], [r[0].volume])
        else:
            raise ValueError(f"cannot lower {mn}")
        out.append(ins)
    return np.array(out, dtype=F.INSTR_DTYPE) if out else np.zeros(0, dtype=F.INSTR_DTYPE)


# --- driver ----------------------------------------------------------------------------
def synthesize(model: F.ModelGraph, spec: TrainSpec, hasher=None):
    """Returns (plan_bytes, SynthInfo)."""
    blk = Block()
    weights: dict = {}
    x_in, out = _build_forward(model, spec.batch, blk, weights)
    batch, out_dim = out.shape
    if spec.loss == "xent":
        labels = Value("labels", (batch,), "i32")
        blk.args.append(labels)
        label_kind, label_bytes = 1, batch * 4
        n = blk.append("sc_high.softmax_xent", [out, labels])
        loss = n.add_result("loss.xent", ())
        n.add_result("loss.xent_probs", (batch, out_dim))
    elif spec.loss == "mse":
        labels = Value("labels", (batch, out_dim))
        blk.args.append(labels)
        label_kind, label_bytes = 2, batch * out_dim * 4
        loss = blk.append("sc_high.mse", [out, labels]).add_result("loss.mse", ())
    else:
        raise ValueError(spec.loss)

    adapters = _graft_lora(blk, spec, weights)
    trainables = [v for a in adapters for v in (a["A"], a["B"])]
    primal_ops = list(blk.ops)
    grads = _autodiff(blk, loss, trainables)
    if spec.emit_optimizer:
        _synth_optimizer(blk, grads, spec)

    # merge program: fill delta = 0 ; delta += scale * A @ B
    merge_ops, merge_deltas = [], []
    for a in adapters:
        fill = Node("sc_low.fill", attrs={"value": 0.0})
        delta = fill.add_result(a["id_base"] + ".delta", a["weight"].shape)
        acc = Node("sc_low.gemm_acc", [a["A"], a["B"], delta], {"alpha": a["scale"]})
        merge_ops += [fill, acc]
        merge_deltas.append(delta)

    protected = {id(loss)} | {id(g) for _, g in grads.values()}
    if spec.fuse_epilogues:
        _fuse_epilogues(blk, protected, primal_ops)

    # --- binding
    refs: dict[int, int] = {}
    cursor = 0
    params = []
    for op in blk.ops:
        if op.mn == "sc_mem.param":
            v = op.results[0]
            refs[id(v)] = cursor
            params.append((v, cursor, op.attrs))
            cursor += F.align_up(v.nbytes)
    persistent_size = cursor
    for a in blk.args:
        refs[id(a)] = cursor
        cursor += F.align_up(a.nbytes)
    io_end = cursor
    ro_chunks, ro_size = [], 0
    for op in blk.ops:
        if op.mn == "sc_mem.weight":
            v = op.results[0]
            off = F.align_up(ro_size)
            ro_chunks.append((off, model.tensors[weights[v]]))
            ro_size = off + v.nbytes
            refs[id(v)] = off | F.RODATA_BIT
    rodata = np.zeros(ro_size, dtype=np.uint8)
    for off, arr in ro_chunks:
        rodata[off:off + arr.nbytes] = arr.reshape(-1).view(np.uint8)
    arena_size = _linear_scan(blk.ops, F.align_up(io_end), refs, protected, refs)
    merge_high = _linear_scan(merge_ops, F.align_up(arena_size), refs,
                              {id(d) for d in merge_deltas}, refs)
    arena_size = max(arena_size, merge_high)

    def ref_of(v):
        return refs[id(v)]

    train = _lower(blk.ops, ref_of)
    eval_ = _lower(primal_ops, ref_of)
    merge = _lower(merge_ops, ref_of)

    persist = np.zeros(persistent_size, dtype=np.uint8)
    for v, off, attrs in params:
        if attrs.get("init") == "randn":
            vals = _counter_randn(attrs["seed"], v.volume, attrs["std"])
            persist[off:off + v.nbytes] = vals.view(np.uint8)

    smf_off = model.smf_offsets()
    emit = np.zeros(len(adapters), dtype=F.EMIT_DTYPE)
    for i, (a, d) in enumerate(zip(adapters, merge_deltas)):
        emit[i] = (smf_off[weights[a["weight"]]], a["weight"].nbytes, refs[id(d)])

    h = F.PlanHeader()
    h.arena_size = F.align_up(arena_size)
    h.persistent_size = persistent_size
    h.input_ref = refs[id(x_in)]
    h.input_floats = batch if model.token_input else batch * model.input_dim
    h.input_kind = 1 if model.token_input else 0
    h.seq_len = model.seq_len
    h.label_ref = refs[id(labels)]
    h.label_bytes, h.label_kind = label_bytes, label_kind
    h.optimizer_kind = 1 if spec.optimizer == "adamw" else 0
    h.loss_ref = refs[id(loss)]
    h.lr, h.beta1, h.beta2, h.eps, h.weight_decay = spec.lr, spec.beta1, spec.beta2, spec.eps, \
        spec.weight_decay
    h.batch, h.default_steps = batch, spec.default_steps
    h.lr_schedule, h.warmup_steps, h.min_lr_factor = spec.lr_schedule, spec.warmup_steps, \
        spec.min_lr_factor
    h.clip_norm = spec.clip_norm
    h.source_model_hash = spec.source_model_hash
    blob = F.assemble_plan(h, train, merge, eval_, rodata, persist, emit, hasher=hasher)

    info = SynthInfo()
    for p, g in sorted(grads.values(), key=lambda pg: pg[0].id):
        info.params.append((p.id, refs[id(p)], refs[id(g)], p.volume))
    for a, d in zip(adapters, merge_deltas):
        info.adapters.append(dict(weight=a["weight"].id, weight_ref=refs[id(a["weight"])],
                                  a_ref=refs[id(a["A"])], b_ref=refs[id(a["B"])],
                                  delta_ref=refs[id(d)], k=a["weight"].shape[0],
                                  m=a["weight"].shape[1], r=spec.lora_rank, scale=a["scale"]))
    for op in blk.ops:
        for r in op.results:
            if id(r) in refs:
                info.values[r.id] = (refs[id(r)], r.shape)
    return blob, info


# --- model families of the benchmark configurations ----------------------------------------
def mlp_model(dims, acts, rng: np.random.Generator, bias=True) -> F.ModelGraph:
    """Feed-forward MLP: Linear(dims[i] -> dims[i+1]) [+ bias] + acts[i] (None = no activation).
    Weights ~ N(0, 1/fan_in), stored [in, out]."""
    g = F.ModelGraph("x", dims[0])
    prev = "x"
    for i in range(len(dims) - 1):
        fan_in = dims[i]
        g.tensor(f"w{i}", rng.standard_normal((dims[i], dims[i + 1])) / np.sqrt(fan_in))
        prev = g.op(F.SMF_MATMUL, f"mm{i}", [prev, f"w{i}"], f"z{i}")
        if bias:
            g.tensor(f"b{i}", rng.standard_normal(dims[i + 1]) * 0.01)
            prev = g.op(F.SMF_ADDBIAS, f"ab{i}", [prev, f"b{i}"], f"zb{i}")
        a = acts[i] if i < len(acts) else None
        if a:
            kind = {"relu": F.SMF_RELU, "gelu": F.SMF_GELU, "silu": F.SMF_SILU}[a]
            prev = g.op(kind, f"act{i}", [prev], f"h{i}")
    return g


def llama_decoder(vocab, d_model, heads, ffn, layers, seq, rng: np.random.Generator,
                  std=0.02) -> F.ModelGraph:
    """Token-native pre-norm decoder: Embedding, L x {RMSNorm, q/k/v, RoPE(q,k), causal
    attention, o, residual, RMSNorm, SwiGLU(gate, up, down), residual}, RMSNorm, lm head."""
    g = F.ModelGraph("x", d_model, seq_len=seq, token_input=True)

    def w(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))
    g.tensor("emb", w(vocab, d_model))
    prev = g.op(F.SMF_EMBEDDING, "embed", ["x", "emb"], "e")
    for i in range(layers):
        p = f"l{i}."
        g.tensor(p + "ln1_g", np.ones(d_model))
        g.op(F.SMF_RMSNORM, p + "ln1", [prev, p + "ln1_g"], p + "n1")
        for nm in ("wq", "wk", "wv"):
            g.tensor(p + nm, w(d_model, d_model))
            g.op(F.SMF_MATMUL, p + "mm_" + nm, [p + "n1", p + nm], p + nm[1])
        g.op(F.SMF_ROPE, p + "rope_q", [p + "q"], p + "qr", heads)
        g.op(F.SMF_ROPE, p + "rope_k", [p + "k"], p + "kr", heads)
        g.op(F.SMF_ATTENTION, p + "attn", [p + "qr", p + "kr", p + "v"], p + "a", heads)
        g.tensor(p + "wo", w(d_model, d_model))
        g.op(F.SMF_MATMUL, p + "mm_wo", [p + "a", p + "wo"], p + "o")
        g.op(F.SMF_ADD, p + "res1", [prev, p + "o"], p + "x1")
        g.tensor(p + "ln2_g", np.ones(d_model))
        g.op(F.SMF_RMSNORM, p + "ln2", [p + "x1", p + "ln2_g"], p + "n2")
        g.tensor(p + "w_gate", w(d_model, ffn))
        g.tensor(p + "w_up", w(d_model, ffn))
        g.op(F.SMF_MATMUL, p + "mm_gate", [p + "n2", p + "w_gate"], p + "g")
        g.op(F.SMF_MATMUL, p + "mm_up", [p + "n2", p + "w_up"], p + "u")
        g.op(F.SMF_SILU, p + "silu", [p + "g"], p + "s")
        g.op(F.SMF_MUL, p + "swiglu", [p + "s", p + "u"], p + "m")
        g.tensor(p + "w_down", w(ffn, d_model))
        g.op(F.SMF_MATMUL, p + "mm_down", [p + "m", p + "w_down"], p + "d")
        prev = g.op(F.SMF_ADD, p + "res2", [p + "x1", p + "d"], p + "x2")
    g.tensor("lnf_g", np.ones(d_model))
    g.op(F.SMF_RMSNORM, "lnf", [prev, "lnf_g"], "nf")
    g.tensor("w_head", w(d_model, vocab))
    g.op(F.SMF_MATMUL, "mm_head", ["nf", "w_head"], "logits")
    return g


def gpt_decoder(vocab, d_model, heads, ffn, layers, seq, rng: np.random.Generator,
                std=0.02) -> F.ModelGraph:
    """Token-native pre-norm decoder with LayerNorm and a GELU MLP (no RoPE):
    Embedding, L x {LayerNorm, q/k/v, causal attention, o, residual, LayerNorm,
    MatMul d->ffn, GELU, MatMul ffn->d, residual}, LayerNorm, lm head."""
    g = F.ModelGraph("x", d_model, seq_len=seq, token_input=True)

    def w(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))
    g.tensor("emb", w(vocab, d_model))
    prev = g.op(F.SMF_EMBEDDING, "embed", ["x", "emb"], "e")

    def ln(name, src, out):
        g.tensor(name + "_g", 1.0 + 0.1 * rng.standard_normal(d_model))
        g.tensor(name + "_b", 0.1 * rng.standard_normal(d_model))
        return g.op(F.SMF_LAYERNORM, name, [src, name + "_g", name + "_b"], out)
    for i in range(layers):
        p = f"l{i}."
        ln(p + "ln1", prev, p + "n1")
        for nm in ("wq", "wk", "wv"):
            g.tensor(p + nm, w(d_model, d_model))
            g.op(F.SMF_MATMUL, p + "mm_" + nm, [p + "n1", p + nm], p + nm[1])
        g.op(F.SMF_ATTENTION, p + "attn", [p + "q", p + "k", p + "v"], p + "a", heads)
        g.tensor(p + "wo", w(d_model, d_model))
        g.op(F.SMF_MATMUL, p + "mm_wo", [p + "a", p + "wo"], p + "o")
        g.op(F.SMF_ADD, p + "res1", [prev, p + "o"], p + "x1")
        ln(p + "ln2", p + "x1", p + "n2")
        g.tensor(p + "w_fc", w(d_model, ffn))
        g.op(F.SMF_MATMUL, p + "mm_fc", [p + "n2", p + "w_fc"], p + "f")
        g.op(F.SMF_GELU, p + "gelu", [p + "f"], p + "ga")
        g.tensor(p + "w_proj", w(ffn, d_model))
        g.op(F.SMF_MATMUL, p + "mm_proj", [p + "ga", p + "w_proj"], p + "d")
        prev = g.op(F.SMF_ADD, p + "res2", [p + "x1", p + "d"], p + "x2")
    ln("lnf", prev, "nf")
    g.tensor("w_head", w(d_model, vocab))
    g.op(F.SMF_MATMUL, "mm_head", ["nf", "w_head"], "logits")
    return g


def zipf_tokens(rng: np.random.Generator, vocab: int, shape, s: float = 1.1) -> np.ndarray:
    """i32 token ids with P(k) ~ 1/(k+1)^s over [0, vocab) (bounded Zipf)."""
    p = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    p /= p.sum()
    return rng.choice(vocab, size=shape, p=p).astype(np.int32)

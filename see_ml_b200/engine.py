"""Python mirror of the reference's runtime API over the C ABI: ``UpdateEngine``
(runtime/engine/update_engine.h:119-190), ``Dataset`` (runtime/feeder/dataset.h:43-152)
and the lower-level device ``Context`` used for per-instruction parity checks.
Same method names and argument meaning; errors raise ``BackendError`` carrying the
"<unit>: <message>" diagnostic.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib as L
from .formats import PlanHeader, parse_plan

MODE_CONTRACT, MODE_FUSED = 0, 1
GEMM_TF32X3, GEMM_F16X2, GEMM_FP32_SIMT, GEMM_TF32 = 0, 1, 2, 3


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Dataset:
    def __init__(self, handle):
        if not handle:
            raise L.BackendError(L.last_error())
        self.h = handle

    @classmethod
    def load_from_file(cls, path: str):
        return cls(L.lib().seeml_b200_dataset_load(path.encode()))

    @classmethod
    def from_tokens(cls, records: np.ndarray):
        a = np.ascontiguousarray(records, dtype=np.int32)
        return cls(L.lib().seeml_b200_dataset_from_tokens(_p(a), a.shape[0], a.shape[1] - 1))

    @classmethod
    def from_memory(cls, inputs: np.ndarray, labels, label_kind: int = 1):
        x = np.ascontiguousarray(inputs, dtype=np.float32)
        n, d = x.shape
        if labels is None:
            return cls(L.lib().seeml_b200_dataset_from_memory(_p(x), None, n, d, 0, 0))
        if label_kind == 1:
            lab = np.ascontiguousarray(labels, dtype=np.int32)
            return cls(L.lib().seeml_b200_dataset_from_memory(_p(x), _p(lab), n, d, 1, 0))
        lab = np.ascontiguousarray(labels, dtype=np.float32).reshape(n, -1)
        return cls(L.lib().seeml_b200_dataset_from_memory(_p(x), _p(lab), n, d, 2, lab.shape[1]))

    def num_samples(self):
        return int(L.lib().seeml_b200_dataset_num_samples(self.h))

    def enable_shuffle(self, seed: int):
        L.lib().seeml_b200_dataset_enable_shuffle(self.h, seed)

    def rewind(self):
        L.lib().seeml_b200_dataset_rewind(self.h)

    def split_validation(self, fraction: float) -> "Dataset":
        return Dataset(L.lib().seeml_b200_dataset_split_validation(self.h, fraction))

    def fill_batch(self, batch: int, input_words: int, label_bytes: int):
        inp = np.zeros(input_words, dtype=np.uint32)
        lab = np.zeros(max(label_bytes, 1), dtype=np.uint8)
        L.lib().seeml_b200_dataset_fill_batch(self.h, batch, _p(inp), _p(lab) if label_bytes else None)
        return inp, lab[:label_bytes]

    def skip_served(self, rows: int):
        L.check(L.lib().seeml_b200_dataset_skip_served(self.h, rows))

    def validate_class_labels(self, num_classes: int):
        L.check(L.lib().seeml_b200_dataset_validate_labels(self.h, num_classes))

    def save_to_file(self, path: str):
        L.check(L.lib().seeml_b200_dataset_save(self.h, path.encode()))

    def close(self):
        if getattr(self, "h", None):
            L.lib().seeml_b200_dataset_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class TrainResult:
    steps: int
    stopped_early: bool
    initial_avg_loss: float
    final_avg_loss: float
    has_validation: bool
    val_initial_loss: float
    val_final_loss: float
    has_val_accuracy: bool
    val_initial_accuracy: float
    val_final_accuracy: float
    improved: bool
    loss_curve: np.ndarray


class UpdateEngine:
    def __init__(self, device: int = 0, mode: int = MODE_CONTRACT, gemm: int = GEMM_TF32X3):
        self.h = L.lib().seeml_b200_engine_create(device, mode, gemm)
        if not self.h:
            raise L.BackendError(L.last_error())
        self._plan = None
        self.header: PlanHeader | None = None

    def load_from_memory(self, plan: bytes):
        buf = np.frombuffer(plan, dtype=np.uint8)
        L.check(L.lib().seeml_b200_engine_load_memory(self.h, _p(buf), buf.size))
        self._plan = buf
        self._read_header()

    def load_from_file(self, path: str):
        L.check(L.lib().seeml_b200_engine_load_file(self.h, path.encode()))
        self._read_header()

    def _read_header(self):
        raw = (C.c_uint8 * 280)()
        L.check(L.lib().seeml_b200_engine_header(self.h, raw))
        self.header = PlanHeader.unpack(bytes(raw))

    def train(self, data: Dataset, steps: int, validation: Dataset | None = None,
              record_loss_curve: bool = True, checkpoint_path: str = "", checkpoint_every: int = 0,
              resume: bool = False, log_every: int = 0, should_stop=None) -> TrainResult:
        n = steps or self.header.default_steps
        curve = np.zeros(max(n, 1), dtype=np.float32)
        opt = L.TrainOptions()
        opt.checkpoint_path = checkpoint_path.encode() if checkpoint_path else None
        opt.checkpoint_every = checkpoint_every
        opt.log_every = log_every
        opt.resume = int(resume)
        opt.validation = validation.h if validation else None
        cb = L.STOP_FN(lambda _u: int(bool(should_stop()))) if should_stop else L.STOP_FN(0)
        opt.should_stop = cb
        opt.loss_curve = curve.ctypes.data_as(C.POINTER(C.c_float)) if record_loss_curve else None
        rep = L.TrainReport()
        L.check(L.lib().seeml_b200_engine_train(self.h, data.h, steps, C.byref(opt), C.byref(rep)))
        return TrainResult(rep.steps, bool(rep.stopped_early), rep.initial_avg_loss, rep.final_avg_loss,
                           bool(rep.has_validation), rep.val_initial_loss, rep.val_final_loss,
                           bool(rep.has_val_accuracy), rep.val_initial_accuracy,
                           rep.val_final_accuracy, bool(rep.improved), curve[:rep.steps].copy())

    def evaluate_metrics(self, data: Dataset):
        loss, acc, has = C.c_float(), C.c_float(), C.c_int32()
        L.check(L.lib().seeml_b200_engine_evaluate(self.h, data.h, C.byref(loss), C.byref(acc),
                                                   C.byref(has)))
        return loss.value, acc.value, bool(has.value)

    def evaluate(self, data: Dataset) -> float:
        return self.evaluate_metrics(data)[0]

    def run_merge(self):
        L.check(L.lib().seeml_b200_engine_run_merge(self.h))

    def commit_to_model(self, source_model_path: str, out_path: str):
        L.check(L.lib().seeml_b200_engine_commit(self.h, source_model_path.encode(), out_path.encode()))

    def verify_source_model(self, path: str):
        L.check(L.lib().seeml_b200_engine_verify_source_model(self.h, path.encode()))

    def save_checkpoint(self, path: str):
        L.check(L.lib().seeml_b200_engine_save_checkpoint(self.h, path.encode()))

    def load_checkpoint(self, path: str):
        L.check(L.lib().seeml_b200_engine_load_checkpoint(self.h, path.encode()))

    def loss_value(self) -> float:
        v = C.c_float()
        L.check(L.lib().seeml_b200_engine_loss(self.h, C.byref(v)))
        return v.value

    def step(self) -> int:
        return int(L.lib().seeml_b200_engine_step(self.h))

    def set_step(self, s: int):
        L.lib().seeml_b200_engine_set_step(self.h, s)

    def effective_lr(self) -> float:
        return float(L.lib().seeml_b200_engine_effective_lr(self.h))

    def execute_train_once(self):
        L.check(L.lib().seeml_b200_engine_execute_train_once(self.h))

    def arena_read(self, offset: int, nbytes: int) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        L.check(L.lib().seeml_b200_engine_arena_read(self.h, offset, _p(out), nbytes))
        return out

    def arena_write(self, offset: int, data: np.ndarray):
        a = np.ascontiguousarray(data)
        L.check(L.lib().seeml_b200_engine_arena_write(self.h, offset, _p(a), a.nbytes))

    def ctx(self):
        return L.lib().seeml_b200_engine_ctx(self.h)

    def opt_begin(self) -> int:
        return int(L.lib().seeml_b200_engine_opt_begin(self.h))

    def run_train_range(self, begin: int, end: int):
        L.check(L.lib().seeml_b200_engine_run_train_range(self.h, begin, end))

    def last_launches(self) -> int:
        return int(L.lib().seeml_b200_engine_last_launches(self.h))

    def enable_step_timing(self, on=True):
        L.check(L.lib().seeml_b200_engine_enable_step_timing(self.h, int(on)))

    def step_timings(self):
        s, a, b, c = C.c_uint64(), C.c_double(), C.c_double(), C.c_double()
        L.check(L.lib().seeml_b200_engine_step_timings(self.h, C.byref(s), C.byref(a), C.byref(b),
                                                       C.byref(c)))
        return s.value, a.value, b.value, c.value

    def reset_step_timings(self):
        L.check(L.lib().seeml_b200_engine_reset_step_timings(self.h))

    def close(self):
        if getattr(self, "h", None):
            L.lib().seeml_b200_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Context:
    """A bare device arena + rodata, for running instruction words one at a time."""

    def __init__(self, arena_bytes: int, rodata: np.ndarray | None = None, device: int = 0,
                 gemm: int = GEMM_TF32X3, persist_init: np.ndarray | None = None):
        ro = np.ascontiguousarray(rodata) if rodata is not None and rodata.size else None
        pi = np.ascontiguousarray(persist_init) if persist_init is not None and persist_init.size else None
        out = C.c_void_p()
        L.check(L.lib().seeml_b200_ctx_create(device, arena_bytes, _p(ro) if ro is not None else None,
                                              ro.nbytes if ro is not None else 0,
                                              _p(pi) if pi is not None else None,
                                              pi.nbytes if pi is not None else 0, None, C.byref(out)))
        self.h = out
        self.arena_bytes = arena_bytes
        L.check(L.lib().seeml_b200_ctx_set_gemm(self.h, gemm))

    def write(self, offset: int, data: np.ndarray):
        a = np.ascontiguousarray(data)
        L.check(L.lib().seeml_b200_h2d(self.h, offset, _p(a), a.nbytes))

    def read(self, offset: int, nbytes: int) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        L.check(L.lib().seeml_b200_d2h(self.h, offset, _p(out), nbytes))
        return out

    def build(self, instrs: np.ndarray, version: int = 7, mode: int = MODE_CONTRACT) -> int:
        prog = np.ascontiguousarray(instrs)
        pid = C.c_int(-1)
        L.check(L.lib().seeml_b200_program_build(self.h, _p(prog), len(prog), version, mode,
                                                 C.byref(pid)))
        return pid.value

    def run(self, pid: int, begin: int, end: int, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, step=1,
            sync=True):
        sc = L.Scalars(lr, b1, b2, eps, wd, 0, step)
        L.check(L.lib().seeml_b200_program_run(self.h, pid, begin, end, C.byref(sc)))
        if sync:
            L.check(L.lib().seeml_b200_sync(self.h))

    def execute(self, instrs: np.ndarray, **scalars):
        pid = self.build(instrs)
        self.run(pid, 0, len(instrs), **scalars)

    def launches(self, pid: int) -> int:
        return int(L.lib().seeml_b200_program_launches(self.h, pid))

    def sync(self):
        L.check(L.lib().seeml_b200_sync(self.h))

    def close(self):
        if getattr(self, "h", None):
            L.lib().seeml_b200_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

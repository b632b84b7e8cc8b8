"""TEST INFRASTRUCTURE — ctypes bindings for the parity checkers.

``port()`` loads oracle/_build/libseeml_oracle.so (our C restatement, built by
``make -C oracle port``); ``ref()`` loads oracle/_ref/libseeml_ref.so (the
unmodified reference plus oracle/ref_harness.cc, built by ``make -C oracle ref``
where the reference checkout is present). Only tests, the smoke check and the
bench's cpu_baseline / reference arm may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = os.path.join(_HERE, "_build", "libseeml_oracle.so")
_REF = os.path.join(_HERE, "_ref", "libseeml_ref.so")

u64, f32, i32, vp = C.c_uint64, C.c_float, C.c_int32, C.c_void_p


def build_port():
    subprocess.run(["make", "-C", _HERE, "port"], check=True, capture_output=True)


def reference_root():
    """Where a read-only checkout of the reference lies: $SEEML_REFERENCE_ROOT, else a
    directory named ``reference`` beside this repository; None when there is none."""
    root = os.environ.get("SEEML_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return root if os.path.isdir(os.path.join(root, "runtime", "engine")) else None


def build_ref(ref_root=None):
    ref_root = ref_root or reference_root()
    if ref_root:
        subprocess.run(["make", "-C", _HERE, "-j8", "ref", f"REF={ref_root}"], check=True,
                       capture_output=True)


_port = None
_ref = None


def port():
    global _port
    if _port is None:
        if not os.path.exists(_PORT):
            build_port()
        lib = C.CDLL(_PORT)
        lib.orc_execute.restype = C.c_int
        lib.orc_execute.argtypes = [vp, C.c_size_t, vp, vp, f32, f32, f32, f32, f32, u64]
        lib.orc_effective_lr.restype = f32
        lib.orc_effective_lr.argtypes = [f32, C.c_uint32, u64, u64, f32, u64]
        lib.orc_content_hash64.restype = u64
        lib.orc_content_hash64.argtypes = [vp, C.c_size_t]
        lib.orc_plan_self_hash.restype = u64
        lib.orc_plan_self_hash.argtypes = [vp, C.c_size_t, C.c_size_t]
        _port = lib
    return _port


def have_ref() -> bool:
    return os.path.exists(_REF)


def ref():
    global _ref
    if _ref is None:
        lib = C.CDLL(_REF)
        lib.ref_set_threads.argtypes = [u64]
        lib.ref_threads.restype = u64
        lib.ref_plan_self_hash.restype = u64
        lib.ref_plan_self_hash.argtypes = [vp, u64, u64]
        lib.ref_content_hash64.restype = u64
        lib.ref_content_hash64.argtypes = [vp, u64]
        lib.ref_validate_instruction.argtypes = [vp, u64, u64, C.c_uint32, C.c_char_p, u64]
        lib.ref_exec.argtypes = [vp, u64, vp, vp, f32, f32, f32, f32, f32, u64]
        lib.ref_exec.restype = None
        lib.ref_compile.argtypes = [C.c_char_p, C.c_char_p, C.c_int64, C.c_int64, f32, u64,
                                    C.c_char_p, C.c_int, C.c_int, f32, f32, f32, C.c_int, u64, f32,
                                    u64, C.c_int, C.c_int, C.c_int, C.c_char_p, u64]
        for name in ("ref_dataset_load",):
            getattr(lib, name).restype = vp
        lib.ref_dataset_load.argtypes = [C.c_char_p, C.c_char_p, u64]
        lib.ref_dataset_from_tokens.restype = vp
        lib.ref_dataset_from_tokens.argtypes = [vp, u64, u64, C.c_char_p, u64]
        lib.ref_dataset_from_memory.restype = vp
        lib.ref_dataset_from_memory.argtypes = [vp, vp, u64, u64, C.c_uint32, u64, C.c_char_p, u64]
        lib.ref_dataset_free.argtypes = [vp]
        lib.ref_dataset_num_samples.restype = u64
        lib.ref_dataset_num_samples.argtypes = [vp]
        lib.ref_dataset_enable_shuffle.argtypes = [vp, u64]
        lib.ref_dataset_rewind.argtypes = [vp]
        lib.ref_dataset_split_validation.restype = vp
        lib.ref_dataset_split_validation.argtypes = [vp, C.c_double, C.c_char_p, u64]
        lib.ref_dataset_fill_batch.argtypes = [vp, u64, vp, vp]
        lib.ref_dataset_skip_served.argtypes = [vp, u64]
        lib.ref_dataset_save.argtypes = [vp, C.c_char_p]
        lib.ref_engine_new.restype = vp
        lib.ref_engine_free.argtypes = [vp]
        lib.ref_engine_load_file.argtypes = [vp, C.c_char_p, C.c_char_p, u64]
        lib.ref_engine_load_memory.argtypes = [vp, vp, u64, C.c_char_p, u64]
        lib.ref_engine_arena.restype = vp
        lib.ref_engine_arena.argtypes = [vp]
        lib.ref_engine_header.argtypes = [vp, vp]
        lib.ref_engine_execute_train_once.argtypes = [vp]
        lib.ref_engine_loss.restype = f32
        lib.ref_engine_loss.argtypes = [vp]
        lib.ref_engine_step.restype = u64
        lib.ref_engine_step.argtypes = [vp]
        lib.ref_engine_set_step.argtypes = [vp, u64]
        lib.ref_engine_effective_lr.restype = f32
        lib.ref_engine_effective_lr.argtypes = [vp]
        lib.ref_engine_train.argtypes = [vp, vp, u64, vp, vp, vp, C.c_char_p, u64]
        lib.ref_engine_evaluate.argtypes = [vp, vp, vp, vp, vp, C.c_char_p, u64]
        lib.ref_engine_run_merge.argtypes = [vp, C.c_char_p, u64]
        lib.ref_engine_commit.argtypes = [vp, C.c_char_p, C.c_char_p, C.c_char_p, u64]
        lib.ref_engine_save_checkpoint.argtypes = [vp, C.c_char_p, C.c_char_p, u64]
        lib.ref_engine_load_checkpoint.argtypes = [vp, C.c_char_p, C.c_char_p, u64]
        lib.ref_engine_step_timings.argtypes = [vp, vp, vp, vp, vp]
        lib.ref_emit_native_package.argtypes = [vp, u64, C.c_char_p, C.c_char_p, C.c_char_p, u64]
        _ref = lib
    return _ref


class RefTrainReport(C.Structure):
    _fields_ = [("steps", u64), ("stopped_early", i32), ("initial_avg_loss", f32),
                ("final_avg_loss", f32), ("has_validation", i32), ("val_initial_loss", f32),
                ("val_final_loss", f32), ("has_val_accuracy", i32), ("val_initial_accuracy", f32),
                ("val_final_accuracy", f32), ("improved", i32)]


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(vp)


def execute(lib_kind: str, program: np.ndarray, arena: np.ndarray, rodata: np.ndarray,
            lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, step=1):
    """Runs an instruction array against host (arena, rodata) byte buffers in place."""
    prog = np.ascontiguousarray(program)
    ro = rodata if rodata.size else np.zeros(64, dtype=np.uint8)
    if lib_kind == "port":
        rc = port().orc_execute(_ptr(prog), len(prog), _ptr(arena), _ptr(ro), lr, b1, b2, eps, wd,
                                step)
        if rc:
            raise RuntimeError(f"oracle: unknown opcode at instruction {rc - 1}")
    else:
        ref().ref_exec(_ptr(prog), len(prog), _ptr(arena), _ptr(ro), lr, b1, b2, eps, wd, step)


class RefEngine:
    """The reference UpdateEngine behind ref_harness.cc."""

    def __init__(self, plan_bytes: bytes):
        self.lib = ref()
        self.blob = np.frombuffer(plan_bytes, dtype=np.uint8).copy()   # kept alive: borrowed
        self.h = self.lib.ref_engine_new()
        err = C.create_string_buffer(512)
        if self.lib.ref_engine_load_memory(self.h, _ptr(self.blob), self.blob.size, err, 512):
            msg = err.value.decode()
            self.lib.ref_engine_free(self.h)
            self.h = None
            raise RuntimeError(msg)
        from see_ml_b200.formats import PlanHeader
        raw = (C.c_uint8 * 280)()
        self.lib.ref_engine_header(self.h, raw)
        self.header = PlanHeader.unpack(bytes(raw))

    def close(self):
        if self.h:
            self.lib.ref_engine_free(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def arena(self) -> np.ndarray:
        n = (self.header.arena_size + 63) & ~63
        p = self.lib.ref_engine_arena(self.h)
        return np.ctypeslib.as_array((C.c_uint8 * n).from_address(p))

    def execute_train_once(self):
        self.lib.ref_engine_execute_train_once(self.h)

    def loss(self) -> float:
        return float(self.lib.ref_engine_loss(self.h))

    def set_step(self, s):
        self.lib.ref_engine_set_step(self.h, s)

    def step(self):
        return int(self.lib.ref_engine_step(self.h))

    def effective_lr(self):
        return float(self.lib.ref_engine_effective_lr(self.h))

    def train(self, ds, steps, validation=None):
        curve = np.zeros(max(steps, 1), dtype=np.float32)
        rep = RefTrainReport()
        err = C.create_string_buffer(512)
        rc = self.lib.ref_engine_train(self.h, ds.h, steps, validation.h if validation else None,
                                       _ptr(curve), C.byref(rep), err, 512)
        if rc:
            raise RuntimeError(err.value.decode())
        return curve[:rep.steps].copy(), rep

    def evaluate(self, ds):
        loss, acc, has = f32(), f32(), i32()
        err = C.create_string_buffer(512)
        if self.lib.ref_engine_evaluate(self.h, ds.h, C.byref(loss), C.byref(acc), C.byref(has),
                                        err, 512):
            raise RuntimeError(err.value.decode())
        return loss.value, acc.value, bool(has.value)

    def run_merge(self):
        err = C.create_string_buffer(512)
        if self.lib.ref_engine_run_merge(self.h, err, 512):
            raise RuntimeError(err.value.decode())

    def step_timings(self):
        steps, a, b, c = u64(), C.c_double(), C.c_double(), C.c_double()
        self.lib.ref_engine_step_timings(self.h, C.byref(steps), C.byref(a), C.byref(b), C.byref(c))
        return steps.value, a.value, b.value, c.value


class RefDataset:
    def __init__(self, handle):
        self.lib = ref()
        self.h = handle

    @classmethod
    def load(cls, path):
        err = C.create_string_buffer(512)
        h = ref().ref_dataset_load(path.encode(), err, 512)
        if not h:
            raise RuntimeError(err.value.decode())
        return cls(h)

    @classmethod
    def from_tokens(cls, records: np.ndarray):
        a = np.ascontiguousarray(records, dtype=np.int32)
        err = C.create_string_buffer(512)
        h = ref().ref_dataset_from_tokens(_ptr(a), a.shape[0], a.shape[1] - 1, err, 512)
        if not h:
            raise RuntimeError(err.value.decode())
        return cls(h)

    @classmethod
    def from_memory(cls, x: np.ndarray, labels: np.ndarray | None, label_kind=1):
        x = np.ascontiguousarray(x, dtype=np.float32)
        n, d = x.shape
        if labels is None:
            lab, label_kind, ld = np.zeros(1, np.uint8), 0, 0
        elif label_kind == 1:
            lab, ld = np.ascontiguousarray(labels, dtype=np.int32).view(np.uint8), 0
        else:
            l2 = np.ascontiguousarray(labels, dtype=np.float32).reshape(n, -1)
            lab, ld = l2.view(np.uint8), l2.shape[1]
        err = C.create_string_buffer(512)
        h = ref().ref_dataset_from_memory(_ptr(x), _ptr(lab), n, d, label_kind, ld, err, 512)
        if not h:
            raise RuntimeError(err.value.decode())
        return cls(h)

    def num_samples(self):
        return int(self.lib.ref_dataset_num_samples(self.h))

    def enable_shuffle(self, seed):
        self.lib.ref_dataset_enable_shuffle(self.h, seed)

    def rewind(self):
        self.lib.ref_dataset_rewind(self.h)

    def split_validation(self, frac):
        err = C.create_string_buffer(512)
        h = self.lib.ref_dataset_split_validation(self.h, frac, err, 512)
        if not h:
            raise RuntimeError(err.value.decode())
        return RefDataset(h)

    def fill_batch(self, batch, input_words, label_bytes):
        inp = np.zeros(input_words, dtype=np.uint32)
        lab = np.zeros(max(label_bytes, 1), dtype=np.uint8)
        self.lib.ref_dataset_fill_batch(self.h, batch, _ptr(inp), _ptr(lab) if label_bytes else None)
        return inp, lab[:label_bytes]

    def close(self):
        if self.h:
            self.lib.ref_dataset_free(self.h)
            self.h = None

    def __del__(self):
        self.close()


def ref_compile(smf_path, out_path, batch, lora_rank=8, lora_alpha=16.0, lora_seed=42,
                targets="", loss=0, optimizer=1, lr=1e-3, weight_decay=0.01, clip_norm=0.0,
                lr_schedule=0, warmup=0, min_lr_factor=0.0, steps=1000, fuse_epilogues=1,
                quantize_base=0, emit_optimizer=1):
    err = C.create_string_buffer(1024)
    rc = ref().ref_compile(smf_path.encode(), out_path.encode(), batch, lora_rank, lora_alpha,
                           lora_seed, targets.encode(), loss, optimizer, lr, weight_decay, clip_norm,
                           lr_schedule, warmup, min_lr_factor, steps, fuse_epilogues, quantize_base,
                           emit_optimizer, err, 1024)
    if rc:
        raise RuntimeError(f"reference compile failed ({rc}): {err.value.decode()}")
    with open(out_path, "rb") as f:
        return f.read()


def ref_emit_native_package(plan: bytes, out_dir: str, repo_root: str | None = None):
    """Runs the reference compiler's packaging step on `plan`: the generated driver
    (update_main.cc) and the embedded-plan translation unit land in `out_dir`. Returns the
    emitter's error text ('' when the whole package, vendored runtime included, was written;
    the vendoring needs a reference checkout, the two generated files do not)."""
    buf = np.frombuffer(plan, np.uint8)
    err = C.create_string_buffer(1024)
    rc = ref().ref_emit_native_package(buf.ctypes.data, buf.size, out_dir.encode(),
                                       (repo_root or "/nonexistent-reference-root").encode(), err, 1024)
    return err.value.decode() if rc else ""

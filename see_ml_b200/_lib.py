"""ctypes loader for libseeml_b200.so (the C ABI declared in include/seeml_b200.h).

The product path has no fallback: if the library has not been built, or no CUDA
device is present, calls fail with an error rather than running anything on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libseeml_b200.so")

u64, u32, i32, f32, vp, cp = C.c_uint64, C.c_uint32, C.c_int32, C.c_float, C.c_void_p, C.c_char_p
INT = C.c_int


class Scalars(C.Structure):
    _fields_ = [("lr", f32), ("beta1", f32), ("beta2", f32), ("eps", f32), ("weight_decay", f32),
                ("reserved", u32), ("step", u64)]


class FusedGemm(C.Structure):
    _fields_ = [(n, u64) for n in ("a_offset", "b_offset", "c_offset", "m", "n", "k", "a2_offset",
                                   "b2_offset", "k2", "addend_offset")]


class TrainReport(C.Structure):
    _fields_ = [("steps", u64), ("stopped_early", i32), ("initial_avg_loss", f32),
                ("final_avg_loss", f32), ("has_validation", i32), ("val_initial_loss", f32),
                ("val_final_loss", f32), ("has_val_accuracy", i32), ("val_initial_accuracy", f32),
                ("val_final_accuracy", f32), ("improved", i32)]


STOP_FN = C.CFUNCTYPE(INT, vp)


class TrainOptions(C.Structure):
    _fields_ = [("checkpoint_path", cp), ("checkpoint_every", u64), ("log_every", u64),
                ("resume", i32), ("validation", vp), ("should_stop", STOP_FN), ("user", vp),
                ("loss_curve", C.POINTER(f32))]


# name -> (restype, argtypes); every symbol include/seeml_b200.h declares
SIGNATURES = {
    "seeml_b200_abi_version": (u32, []),
    "seeml_b200_last_error": (cp, []),
    "seeml_b200_plan_self_hash": (u64, [vp, u64, u64]),
    "seeml_b200_content_hash64": (u64, [vp, u64]),
    "seeml_b200_validate_instruction": (INT, [vp, u64, u64, u32]),
    "seeml_b200_plan_verify": (INT, [vp, u64]),
    "seeml_b200_ctx_create": (INT, [INT, u64, vp, u64, vp, u64, vp, C.POINTER(vp)]),
    "seeml_b200_ctx_destroy": (None, [vp]),
    "seeml_b200_ctx_arena": (vp, [vp]),
    "seeml_b200_ctx_arena_bytes": (u64, [vp]),
    "seeml_b200_ctx_stream": (vp, [vp]),
    "seeml_b200_ctx_set_gemm": (INT, [vp, u32]),
    "seeml_b200_program_build": (INT, [vp, vp, u64, u32, u32, C.POINTER(INT)]),
    "seeml_b200_program_size": (u64, [vp, INT]),
    "seeml_b200_program_launches": (u64, [vp, INT]),
    "seeml_b200_program_run": (INT, [vp, INT, u64, u64, C.POINTER(Scalars)]),
    "seeml_b200_exec_one": (INT, [vp, vp, u32, C.POINTER(Scalars)]),
    "seeml_b200_gemm_fused": (INT, [vp, C.POINTER(FusedGemm)]),
    "seeml_b200_h2d": (INT, [vp, u64, vp, u64]),
    "seeml_b200_d2h": (INT, [vp, u64, vp, u64]),
    "seeml_b200_memset": (INT, [vp, u64, INT, u64]),
    "seeml_b200_d2d": (INT, [vp, u64, vp, u64]),
    "seeml_b200_stage_h2d": (INT, [vp, INT, vp, u64, vp, u64]),
    "seeml_b200_stage_wait": (INT, [vp, INT]),
    "seeml_b200_stage_commit": (INT, [vp, INT, u64, u64]),
    "seeml_b200_stage_io": (INT, [vp, u64, vp, u64, u64, vp, u64]),
    "seeml_b200_pinned_alloc": (vp, [u64]),
    "seeml_b200_pinned_free": (None, [vp]),
    "seeml_b200_read_f32": (INT, [vp, u64, C.POINTER(f32)]),
    "seeml_b200_sync": (INT, [vp]),
    "seeml_b200_ctx_enable_timing": (INT, [vp, INT]),
    "seeml_b200_last_run_ms": (INT, [vp, C.POINTER(f32)]),
    "seeml_b200_xent_fwd_noalloc": (INT, [vp, vp, vp, vp, u64, u64, vp]),
    "seeml_b200_grads_pack": (INT, [vp, vp, vp, u64, vp]),
    "seeml_b200_grads_unpack": (INT, [vp, vp, vp, u64, vp]),
    "seeml_b200_tree_sum": (INT, [vp, vp, u64, u64, f32]),
    "seeml_b200_comm_unique_id": (INT, [vp]),
    "seeml_b200_comm_init": (INT, [INT, vp, INT, INT, C.POINTER(vp)]),
    "seeml_b200_comm_destroy": (None, [vp]),
    "seeml_b200_comm_rank": (INT, [vp]),
    "seeml_b200_comm_world": (INT, [vp]),
    "seeml_b200_comm_allgather": (INT, [vp, vp, vp, u64, vp]),
    "seeml_b200_comm_wait": (INT, [vp, vp, C.c_double]),
    "seeml_b200_engine_dp_configure": (INT, [vp, u64, INT, INT, vp]),
    "seeml_b200_engine_dp_step_host": (INT, [vp, vp, vp, C.POINTER(f32)]),
    "seeml_b200_engine_dp_step_device": (INT, [vp, vp, vp, C.POINTER(f32)]),
    "seeml_b200_engine_dp_local_chunks": (u64, [vp]),
    "seeml_b200_dataset_load": (vp, [cp]),
    "seeml_b200_dataset_from_tokens": (vp, [vp, u64, u64]),
    "seeml_b200_dataset_from_memory": (vp, [vp, vp, u64, u64, u32, u64]),
    "seeml_b200_dataset_free": (None, [vp]),
    "seeml_b200_dataset_num_samples": (u64, [vp]),
    "seeml_b200_dataset_input_dim": (u64, [vp]),
    "seeml_b200_dataset_label_kind": (u32, [vp]),
    "seeml_b200_dataset_input_kind": (u32, [vp]),
    "seeml_b200_dataset_enable_shuffle": (None, [vp, u64]),
    "seeml_b200_dataset_rewind": (None, [vp]),
    "seeml_b200_dataset_split_validation": (vp, [vp, C.c_double]),
    "seeml_b200_dataset_fill_batch": (None, [vp, u64, vp, vp]),
    "seeml_b200_dataset_skip_served": (INT, [vp, u64]),
    "seeml_b200_dataset_validate_labels": (INT, [vp, u64]),
    "seeml_b200_dataset_save": (INT, [vp, cp]),
    "seeml_b200_dataset_label_bytes_per_sample": (u64, [vp]),
    "seeml_b200_dataset_save_pos": (None, [vp, C.POINTER(u64), C.POINTER(u64)]),
    "seeml_b200_dataset_restore_pos": (None, [vp, u64, u64]),
    "seeml_b200_engine_create": (vp, [INT, u32, u32]),
    "seeml_b200_engine_destroy": (None, [vp]),
    "seeml_b200_engine_load_memory": (INT, [vp, vp, u64]),
    "seeml_b200_engine_load_file": (INT, [vp, cp]),
    "seeml_b200_engine_train": (INT, [vp, vp, u64, C.POINTER(TrainOptions), C.POINTER(TrainReport)]),
    "seeml_b200_engine_evaluate": (INT, [vp, vp, C.POINTER(f32), C.POINTER(f32), C.POINTER(i32)]),
    "seeml_b200_engine_run_merge": (INT, [vp]),
    "seeml_b200_engine_commit": (INT, [vp, cp, cp]),
    "seeml_b200_engine_verify_source_model": (INT, [vp, cp]),
    "seeml_b200_engine_save_checkpoint": (INT, [vp, cp]),
    "seeml_b200_engine_load_checkpoint": (INT, [vp, cp]),
    "seeml_b200_engine_header": (INT, [vp, vp]),
    "seeml_b200_engine_loss": (INT, [vp, C.POINTER(f32)]),
    "seeml_b200_engine_step": (u64, [vp]),
    "seeml_b200_engine_set_step": (None, [vp, u64]),
    "seeml_b200_engine_effective_lr": (f32, [vp]),
    "seeml_b200_engine_execute_train_once": (INT, [vp]),
    "seeml_b200_engine_arena_read": (INT, [vp, u64, vp, u64]),
    "seeml_b200_engine_arena_write": (INT, [vp, u64, vp, u64]),
    "seeml_b200_engine_ctx": (vp, [vp]),
    "seeml_b200_engine_opt_begin": (u64, [vp]),
    "seeml_b200_engine_run_train_range": (INT, [vp, u64, u64]),
    "seeml_b200_engine_last_launches": (u64, [vp]),
    "seeml_b200_engine_enable_step_timing": (INT, [vp, INT]),
    "seeml_b200_engine_reset_step_timings": (INT, [vp]),
    "seeml_b200_engine_step_timings": (INT, [vp, C.POINTER(u64), C.POINTER(C.c_double),
                                             C.POINTER(C.c_double), C.POINTER(C.c_double)]),
}

_lib = None


class BackendError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise BackendError(
                f"{LIB_PATH} is missing: build it with `python -m see_ml_b200.build` "
                "(there is no CPU fallback)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def last_error() -> str:
    return lib().seeml_b200_last_error().decode(errors="replace")


def check(rc: int):
    if rc != 0:
        raise BackendError(last_error())

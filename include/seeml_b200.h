/* seeml_b200 — C ABI of the B200 (sm_100a) execution backend for SeeML update plans.
 *
 * The reference runtime has no plugin layer: its engine calls its CPU kernels
 * through plain C++ (runtime/engine/update_engine.cc:306-509). This header is the
 * seam a maintainer binds instead: the same operator contract (64-byte
 * UpdateInstruction words over an arena-offset plan), executed by CUDA kernels.
 * Every entry point cites the reference interface it stands in for.
 *
 * Conventions: every function that can fail returns 0 on success and a nonzero
 * code otherwise; the message is available from seeml_b200_last_error(). Nothing
 * throws or aborts. Host pointers are borrowed for the duration of the call
 * unless stated. Calls on one context/engine must be serialised by the caller;
 * distinct contexts are independent. All device memory is owned by the context.
 * There is no CPU fallback: without a CUDA device every device call fails.
 */
#ifndef SEEML_B200_H_
#define SEEML_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SEEML_B200_ABI_VERSION 1
uint32_t seeml_b200_abi_version(void);

/* Last error message of the calling thread (never NULL). */
const char* seeml_b200_last_error(void);

/* ---------------------------------------------------------------- integrity --
 * PlanSelfHash / ContentHash64 — source/identity/hash.h:103-161. Host code. */
uint64_t seeml_b200_plan_self_hash(const void* plan, uint64_t size, uint64_t hash_offset);
uint64_t seeml_b200_content_hash64(const void* data, uint64_t size);

/* Load-time proof of one instruction's operand extents, alignment, address
 * space, aliasing and flags — runtime/validator/plan_validator.cc:9-343
 * (ValidateInstruction). `instr` points at one 64-byte word. */
int seeml_b200_validate_instruction(const void* instr, uint64_t arena_size,
                                    uint64_t rodata_size, uint32_t plan_version);

/* Whole-plan admission: header magic/version, plan_hash, section bounds, I/O
 * slots, every instruction of the three programs, label/token bindings, emit
 * table — UpdateEngine::Initialize (runtime/engine/update_engine.cc:80-225) with
 * VerifyPlanContract / VerifyExecutorContract (runtime/engine/contract.cc:35-168). */
int seeml_b200_plan_verify(const void* plan, uint64_t size);

/* ------------------------------------------------------------ device context --
 * One context = one device arena (the plan's single allocation,
 * update_engine.cc:229-234), a device copy of the frozen rodata, and streams. */
typedef struct seeml_b200_ctx seeml_b200_ctx;

/* Per-step scalars the optimiser instructions read — the values
 * UpdateEngine::ExecuteRange passes to SgdStep/AdamWStep
 * (update_engine.cc:432-443): EffectiveLr(), header hyper-parameters, step_. */
typedef struct seeml_b200_scalars {
  float lr, beta1, beta2, eps, weight_decay;
  uint32_t reserved;
  uint64_t step; /* 1-indexed AdamW timestep */
} seeml_b200_scalars;

/* Execution modes of a program. CONTRACT runs one kernel per instruction and
 * writes every operand the instruction names. FUSED may merge instruction groups
 * into single kernels; ranges that no later instruction reads may be skipped. */
#define SEEML_B200_MODE_CONTRACT 0u
#define SEEML_B200_MODE_FUSED 1u
/* GEMM arithmetic. TF32X3: three tf32 products per step (hi.hi + lo.hi + hi.lo), f32-class
 * accuracy. F16X2: the same three-product scheme on a two-term fp16 split of power-of-two-scaled
 * operands, f32 accumulation (the same 22 significant bits at twice the tensor-core rate; taken
 * by the wide frozen-weight GEMMs, every other shape runs TF32X3). TF32: one tf32 product
 * (10-bit operands). FP32_SIMT: plain f32 FMA on the CUDA cores. */
#define SEEML_B200_GEMM_TF32X3 0u
#define SEEML_B200_GEMM_F16X2 1u
#define SEEML_B200_GEMM_FP32_SIMT 2u
#define SEEML_B200_GEMM_TF32 3u

/* rodata / persist_init may be NULL when their size is 0. The arena is zeroed,
 * then persist_init is copied to offset 0 (update_engine.cc:229-234).
 * external_arena: NULL to let the context allocate, or a device pointer to
 * arena_bytes (64-byte aligned) the caller owns. */
int seeml_b200_ctx_create(int device, uint64_t arena_bytes, const void* rodata,
                          uint64_t rodata_bytes, const void* persist_init,
                          uint64_t persist_bytes, void* external_arena,
                          seeml_b200_ctx** out);
void seeml_b200_ctx_destroy(seeml_b200_ctx* ctx);
void* seeml_b200_ctx_arena(seeml_b200_ctx* ctx);        /* device pointer */
uint64_t seeml_b200_ctx_arena_bytes(seeml_b200_ctx* ctx);
void* seeml_b200_ctx_stream(seeml_b200_ctx* ctx);       /* cudaStream_t of the compute stream */
int seeml_b200_ctx_set_gemm(seeml_b200_ctx* ctx, uint32_t gemm_kind);

/* Decode + validate + (FUSED) group an instruction stream; returns a program id.
 * Stands in for the decode in Initialize (update_engine.cc:130-137). */
int seeml_b200_program_build(seeml_b200_ctx* ctx, const void* instrs, uint64_t count,
                             uint32_t plan_version, uint32_t mode, int* program_id);
uint64_t seeml_b200_program_size(seeml_b200_ctx* ctx, int program_id);
/* Kernels launched by the most recent run of the program (a launch count, for
 * reporting). */
uint64_t seeml_b200_program_launches(seeml_b200_ctx* ctx, int program_id);

/* Enqueue instructions [begin, end) on the compute stream — ExecuteRange
 * (update_engine.cc:306-509). Asynchronous; pair with seeml_b200_sync or a read. */
int seeml_b200_program_run(seeml_b200_ctx* ctx, int program_id, uint64_t begin,
                           uint64_t end, const seeml_b200_scalars* scalars);
/* One instruction word, contract mode, synchronous. */
int seeml_b200_exec_one(seeml_b200_ctx* ctx, const void* instr, uint32_t plan_version,
                        const seeml_b200_scalars* scalars);

/* The fused GEMM the LoRA groups lower to, as one call on arena offsets:
 *   C[M,N] = (addend[M,N] +) A[M,K] . B[N,K]^T (+ A2[M,K2] . B2[N,K2]^T)
 * i.e. a forward C' = X.W + (alpha/r)(X.A).B with B = W^T, A2 = X.A, B2 = (alpha/r) B^T, or a
 * backward dX = dC'.W^T + dT.A^T. Stands in for the gemm.nn / gemm.nt + scale + add.ew
 * sequences of lora_grafter.cc:130-159 and autodiff.cc:71-91. Offsets are arena byte
 * offsets (a2/b2 ignored when k2 == 0; addend_offset == UINT64_MAX means none). Runs on the
 * tensor cores when the shape allows, else on the CUDA cores; asynchronous. */
typedef struct seeml_b200_fused_gemm {
  uint64_t a_offset, b_offset, c_offset, m, n, k;
  uint64_t a2_offset, b2_offset, k2;
  uint64_t addend_offset;
} seeml_b200_fused_gemm;
int seeml_b200_gemm_fused(seeml_b200_ctx* ctx, const seeml_b200_fused_gemm* g);

/* Arena transfers (synchronous with respect to the compute stream). */
int seeml_b200_h2d(seeml_b200_ctx* ctx, uint64_t arena_offset, const void* src, uint64_t bytes);
int seeml_b200_d2h(seeml_b200_ctx* ctx, uint64_t arena_offset, void* dst, uint64_t bytes);
int seeml_b200_memset(seeml_b200_ctx* ctx, uint64_t arena_offset, int byte, uint64_t bytes);
/* Device-to-device move into the arena, enqueued on the compute stream (asynchronous):
 * the staging step for batches that already live in HBM. */
int seeml_b200_d2d(seeml_b200_ctx* ctx, uint64_t arena_offset, const void* src_device, uint64_t bytes);
/* Batch staging — BatchPipeline::NextBatch (runtime/feeder/batch_pipeline.cc:61-79),
 * as a pinned double buffer on a copy stream. stage_h2d copies a batch from PINNED
 * host buffers into device staging slot 0 or 1 on the copy stream and returns at
 * once (it does not touch the arena, so it overlaps the running step); label may be
 * NULL. stage_wait blocks the host until that copy has finished (the pinned buffers
 * may then be refilled). stage_commit makes the compute stream wait for the slot's
 * copy and moves it into the plan's I/O slots ahead of the next program_run.
 * stage_io = stage_h2d + stage_commit on slot 0. */
int seeml_b200_stage_h2d(seeml_b200_ctx* ctx, int slot, const void* input, uint64_t input_bytes,
                         const void* label, uint64_t label_bytes);
int seeml_b200_stage_wait(seeml_b200_ctx* ctx, int slot);
int seeml_b200_stage_commit(seeml_b200_ctx* ctx, int slot, uint64_t input_offset,
                            uint64_t label_offset);
int seeml_b200_stage_io(seeml_b200_ctx* ctx, uint64_t input_offset, const void* input,
                        uint64_t input_bytes, uint64_t label_offset, const void* label,
                        uint64_t label_bytes);
void* seeml_b200_pinned_alloc(uint64_t bytes);
void seeml_b200_pinned_free(void* p);
/* The scalar loss slot — UpdateEngine::LossValue (update_engine.cc:511-513).
 * Waits for the compute stream. */
int seeml_b200_read_f32(seeml_b200_ctx* ctx, uint64_t arena_offset, float* out);
int seeml_b200_sync(seeml_b200_ctx* ctx);
/* Device time of the most recent program_run when timing is on (ms). */
int seeml_b200_ctx_enable_timing(seeml_b200_ctx* ctx, int on);
int seeml_b200_last_run_ms(seeml_b200_ctx* ctx, float* ms);

/* --------------------------------------------- allocation-free softmax cross-entropy --
 * No counterpart in the reference. For hosts that may not call the CUDA allocator (the
 * device's memory is already owned by their own pool, or an allocation's implicit
 * synchronisation is not acceptable where they call from): the same kernels as the
 * kXentFwd instruction (loss = -(1/rows) sum log softmax(logits)[label], probs cached),
 * with the reduction scratch held in a fixed array inside the library, so the call only
 * launches kernels. All pointers are DEVICE pointers the caller owns; `stream` is a
 * cudaStream_t (NULL = the default stream); the call is asynchronous on that stream.
 * Limit: rows <= 65536 per call, larger calls are refused with an error. Every GPU that
 * loads the library holds the array (about 0.5 MiB) until the process exits.
 * The first call on each device looks the array's device address up
 * (cudaGetSymbolAddress) with that device current: make that first call outside any
 * stream capture. Every call uses the same array: two calls that may overlap on the
 * GPU (different streams, no ordering between them) race on it. Nothing in the array
 * has to start at zero; each call overwrites what it reads.
 * The operands must live on the CURRENT device (the call checks `logits` and refuses
 * otherwise) and device ordinals 0..63 are supported. Every label must lie in
 * [0, classes): a label outside that range is not dereferenced, it turns the loss into NaN. */
int seeml_b200_xent_fwd_noalloc(const float* logits, const int32_t* labels, float* loss, float* probs,
                                uint64_t rows, uint64_t classes, void* stream);

/* ------------------------------------------------- data-parallel gradient sets --
 * No counterpart in the reference (single process). A gradient set is the list of
 * (arena offset, float count) pairs of the optimiser instructions' gradient
 * operands. pack/unpack gather them to/from one contiguous device buffer;
 * tree_sum adds `count` packed sets laid out back to back in a fixed binary tree
 * over the set index and scales by `scale`, writing set 0. */
int seeml_b200_grads_pack(seeml_b200_ctx* ctx, const uint64_t* offsets,
                          const uint64_t* counts, uint64_t n, void* dst_device);
int seeml_b200_grads_unpack(seeml_b200_ctx* ctx, const uint64_t* offsets,
                            const uint64_t* counts, uint64_t n, const void* src_device);
int seeml_b200_tree_sum(seeml_b200_ctx* ctx, void* sets_device, uint64_t floats_per_set,
                        uint64_t count, float scale);

/* ------------------------------------------------------------ data-parallel exchange --
 * No counterpart in the reference (single process). One communicator per GPU process (NCCL over
 * NVLink, bound at run time). Rank 0 makes a 128-byte id with comm_unique_id and hands it to
 * every rank by whatever channel the host has (a file, a socket, MPI, torch.distributed); every
 * rank then calls comm_init. allgather enqueues on `stream`; comm_wait waits for the stream on
 * the host while polling the communicator, and aborts it with an error if NCCL reports one or
 * nothing completes within timeout_s (a rank that never posted), instead of hanging. */
#define SEEML_B200_COMM_ID_BYTES 128
typedef struct seeml_b200_comm seeml_b200_comm;
int seeml_b200_comm_unique_id(void* id_out);
int seeml_b200_comm_init(int device, const void* id, int rank, int world, seeml_b200_comm** out);
void seeml_b200_comm_destroy(seeml_b200_comm* comm);
int seeml_b200_comm_rank(const seeml_b200_comm* comm);
int seeml_b200_comm_world(const seeml_b200_comm* comm);
int seeml_b200_comm_allgather(seeml_b200_comm* comm, const void* send_device, void* recv_device,
                              uint64_t floats, void* stream);
int seeml_b200_comm_wait(seeml_b200_comm* comm, void* stream, double timeout_s);

/* ------------------------------------------------------------------- datasets --
 * SDS corpora — runtime/feeder/dataset.h:43-152, dataset.cc:86-462. Host code;
 * serving order, shuffle and token label derivation are bit-exact. */
typedef struct seeml_b200_dataset seeml_b200_dataset;
seeml_b200_dataset* seeml_b200_dataset_load(const char* path);
seeml_b200_dataset* seeml_b200_dataset_from_tokens(const int32_t* tokens, uint64_t records,
                                                   uint64_t seq);
seeml_b200_dataset* seeml_b200_dataset_from_memory(const float* inputs, const void* labels,
                                                   uint64_t samples, uint64_t input_dim,
                                                   uint32_t label_kind, uint64_t label_dim);
void seeml_b200_dataset_free(seeml_b200_dataset* d);
uint64_t seeml_b200_dataset_num_samples(const seeml_b200_dataset* d);
uint64_t seeml_b200_dataset_input_dim(const seeml_b200_dataset* d);
uint32_t seeml_b200_dataset_label_kind(const seeml_b200_dataset* d);
uint32_t seeml_b200_dataset_input_kind(const seeml_b200_dataset* d);
void seeml_b200_dataset_enable_shuffle(seeml_b200_dataset* d, uint64_t seed);
void seeml_b200_dataset_rewind(seeml_b200_dataset* d);
seeml_b200_dataset* seeml_b200_dataset_split_validation(seeml_b200_dataset* d, double fraction);
void seeml_b200_dataset_fill_batch(seeml_b200_dataset* d, uint64_t batch, void* input_slot,
                                   void* label_slot);
int seeml_b200_dataset_skip_served(seeml_b200_dataset* d, uint64_t rows);
int seeml_b200_dataset_validate_labels(const seeml_b200_dataset* d, uint64_t num_classes);
int seeml_b200_dataset_save(const seeml_b200_dataset* d, const char* path);
uint64_t seeml_b200_dataset_label_bytes_per_sample(const seeml_b200_dataset* d);
/* Dataset::SaveServingPos / RestoreServingPos — runtime/feeder/dataset.h:93-106. */
void seeml_b200_dataset_save_pos(const seeml_b200_dataset* d, uint64_t* cursor, uint64_t* epoch);
void seeml_b200_dataset_restore_pos(seeml_b200_dataset* d, uint64_t cursor, uint64_t epoch);

/* --------------------------------------------------------------------- engine --
 * class UpdateEngine — runtime/engine/update_engine.h:119-190. */
typedef struct seeml_b200_engine seeml_b200_engine;

typedef struct seeml_b200_train_report { /* TrainReport, update_engine.h:91-117 */
  uint64_t steps;
  int32_t stopped_early;
  float initial_avg_loss, final_avg_loss;
  int32_t has_validation;
  float val_initial_loss, val_final_loss;
  int32_t has_val_accuracy;
  float val_initial_accuracy, val_final_accuracy;
  int32_t improved;
} seeml_b200_train_report;

typedef struct seeml_b200_train_options { /* TrainOptions, update_engine.h:43-67 */
  const char* checkpoint_path;   /* NULL/"" = none */
  uint64_t checkpoint_every;
  uint64_t log_every;            /* 0 = quiet */
  int32_t resume;
  seeml_b200_dataset* validation; /* may be NULL */
  int (*should_stop)(void* user); /* may be NULL; polled once per step */
  void* user;
  float* loss_curve;             /* may be NULL; else room for `steps` floats */
} seeml_b200_train_options;

seeml_b200_engine* seeml_b200_engine_create(int device, uint32_t mode, uint32_t gemm_kind);
void seeml_b200_engine_destroy(seeml_b200_engine* e);
/* LoadFromMemory borrows `plan` until the engine is destroyed or reloaded
 * (update_engine.h:127-130); a rejected load leaves the previous plan usable. */
int seeml_b200_engine_load_memory(seeml_b200_engine* e, const void* plan, uint64_t size);
int seeml_b200_engine_load_file(seeml_b200_engine* e, const char* path);
int seeml_b200_engine_train(seeml_b200_engine* e, seeml_b200_dataset* data, uint64_t steps,
                            const seeml_b200_train_options* options,
                            seeml_b200_train_report* report);
int seeml_b200_engine_evaluate(seeml_b200_engine* e, seeml_b200_dataset* data, float* loss,
                               float* accuracy, int32_t* has_accuracy);
int seeml_b200_engine_run_merge(seeml_b200_engine* e);
int seeml_b200_engine_commit(seeml_b200_engine* e, const char* source_model_path,
                             const char* out_path);
int seeml_b200_engine_verify_source_model(seeml_b200_engine* e, const char* source_model_path);
int seeml_b200_engine_save_checkpoint(seeml_b200_engine* e, const char* path);
int seeml_b200_engine_load_checkpoint(seeml_b200_engine* e, const char* path);
int seeml_b200_engine_header(const seeml_b200_engine* e, void* out280);
int seeml_b200_engine_loss(seeml_b200_engine* e, float* loss);
uint64_t seeml_b200_engine_step(const seeml_b200_engine* e);
void seeml_b200_engine_set_step(seeml_b200_engine* e, uint64_t step);
float seeml_b200_engine_effective_lr(const seeml_b200_engine* e);
int seeml_b200_engine_execute_train_once(seeml_b200_engine* e);
/* arena() of the reference returns a host pointer tests peek and poke through
 * (test/support/probes.cc:25-60); here the arena is device memory, so reads and
 * writes are explicit copies. */
int seeml_b200_engine_arena_read(seeml_b200_engine* e, uint64_t offset, void* dst, uint64_t bytes);
int seeml_b200_engine_arena_write(seeml_b200_engine* e, uint64_t offset, const void* src,
                                  uint64_t bytes);
seeml_b200_ctx* seeml_b200_engine_ctx(seeml_b200_engine* e);
/* Instruction index of the first clip/optimiser instruction of the train program
 * (update_engine.cc:249-261): the split point of a data-parallel step. */
uint64_t seeml_b200_engine_opt_begin(const seeml_b200_engine* e);
/* Runs train instructions [begin, end) with the engine's current step scalars. */
int seeml_b200_engine_run_train_range(seeml_b200_engine* e, uint64_t begin, uint64_t end);
/* The K-chunk data-parallel step (no counterpart in the reference; its single-process step is
 * update_engine.cc:736-771). A global step is `chunks_per_step` executions of the train stream
 * up to the first optimiser instruction, each on its own batch of the plan's compiled size;
 * rank r runs chunks [r K/world, (r+1) K/world). The per-chunk gradient sets and losses are
 * summed in one fixed binary tree over the chunk index (local subtree, NCCL all-gather, the rest
 * of the tree in rank order), scaled by 1/K, and every rank runs the optimiser instructions on
 * identical bits: 1, 2, 4 and 8 GPUs give bit-identical parameters. chunks_per_step and world
 * must be powers of two with world <= chunks_per_step; comm may be NULL when world == 1 and is
 * borrowed otherwise. dp_step_host takes this rank's chunks back to back in HOST memory (copied
 * through pinned staging on the copy stream, overlapped with the previous chunk's compute);
 * dp_step_device takes them in DEVICE memory. Each call advances the engine's step; `loss`
 * (nullable) receives the mean loss over all K chunks and makes the call synchronous. */
int seeml_b200_engine_dp_configure(seeml_b200_engine* e, uint64_t chunks_per_step, int rank, int world,
                                   seeml_b200_comm* comm);
int seeml_b200_engine_dp_step_host(seeml_b200_engine* e, const void* inputs, const void* labels, float* loss);
int seeml_b200_engine_dp_step_device(seeml_b200_engine* e, const void* inputs_device,
                                     const void* labels_device, float* loss);
uint64_t seeml_b200_engine_dp_local_chunks(const seeml_b200_engine* e);
/* Kernels launched by the most recent train-program execution. */
uint64_t seeml_b200_engine_last_launches(const seeml_b200_engine* e);
/* StepTimings (update_engine.h:84-89), from CUDA events at the same two
 * boundaries; accumulates only when enabled. */
int seeml_b200_engine_enable_step_timing(seeml_b200_engine* e, int on);
int seeml_b200_engine_step_timings(const seeml_b200_engine* e, uint64_t* steps,
                                   double* fwd_seconds, double* bwd_seconds,
                                   double* opt_seconds);
/* ResetStepTimings (update_engine.h:190). */
int seeml_b200_engine_reset_step_timings(seeml_b200_engine* e);

#ifdef __cplusplus
}
#endif
#endif /* SEEML_B200_H_ */

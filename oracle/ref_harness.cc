// TEST INFRASTRUCTURE — extern "C" shim over the UNMODIFIED reference runtime
// and compiler, so Python tests (ctypes) can drive the real thing as the
// parity checker. Linked only into oracle/_ref/libseeml_ref.so; nothing the
// product ships may load it.
//
// Every function below forwards to a public reference API; the only logic
// of our own is ref_exec(), a per-instruction switch that mirrors the operand
// conventions of UpdateEngine::ExecuteRange (runtime/engine/update_engine.cc:306-509,
// which is private) so single kernels can be checked without building a plan.
// The whole-plan path (ref_engine_*) goes through the reference's own
// dispatcher and pins those conventions.

#include <bit>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "compiler/backend/trainer/native_emitter.h"
#include "compiler/driver/update_compiler.h"
#include "compiler/frontend/ingressor/model_reader.h"
#include "runtime/engine/update_engine.h"
#include "runtime/executor/update_kernels.h"
#include "runtime/feeder/batch_pipeline.h"
#include "runtime/feeder/dataset.h"
#include "runtime/validator/plan_validator.h"
#include "source/identity/hash.h"
#include "source/parallel/parallel_for.h"

namespace up = seeml::update;
namespace rt = seeml::update_rt;
namespace k = seeml::update_rt::kernels;

namespace {

void SetErr(char* err, size_t cap, const std::string& msg) {
  if (!err || cap == 0) return;
  std::snprintf(err, cap, "%s", msg.c_str());
}

float Bits(uint64_t w) { return std::bit_cast<float>(static_cast<uint32_t>(w)); }

struct DatasetBox {
  rt::Dataset ds;
};

}  // namespace

extern "C" {

// --- substrate ---------------------------------------------------------------
void ref_set_threads(uint64_t n) { up::SetParallelThreadCount(n); }
uint64_t ref_threads() { return up::ParallelThreadCount(); }

uint64_t ref_plan_self_hash(const uint8_t* p, uint64_t n, uint64_t hash_off) {
  return up::PlanSelfHash(p, n, hash_off);
}
uint64_t ref_content_hash64(const uint8_t* p, uint64_t n) {
  return up::ContentHash64(p, n);
}
uint64_t ref_fnv1a64(const uint8_t* p, uint64_t n) { return up::Fnv1a64(p, n); }

int ref_validate_instruction(const void* ins, uint64_t arena_size,
                             uint64_t rodata_size, uint32_t version, char* err,
                             uint64_t cap) {
  up::UpdateInstruction i;
  std::memcpy(&i, ins, sizeof(i));
  auto r = rt::ValidateInstruction(i, arena_size, rodata_size, version);
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}

// --- single-instruction execution against caller buffers ---------------------
// lr/beta/eps/wd/step stand in for the engine's header fields and step counter.
void ref_exec(const void* program, uint64_t count, uint8_t* arena,
              const uint8_t* rodata, float lr, float beta1, float beta2,
              float eps, float wd, uint64_t step) {
  auto R = [&](uint64_t ref) -> const float* {
    const uint64_t off = up::RefOffset(ref);
    return reinterpret_cast<const float*>(
        (up::IsRodataRef(ref) ? rodata : arena) + off);
  };
  auto W = [&](uint64_t ref) -> float* {
    return reinterpret_cast<float*>(arena + up::RefOffset(ref));
  };
  auto I = [&](uint64_t ref) {
    return reinterpret_cast<const int32_t*>(R(ref));
  };
  auto hi = [](uint64_t w) { return w >> 32; };
  auto lo = [](uint64_t w) { return w & 0xFFFFFFFFu; };
  for (uint64_t idx = 0; idx < count; ++idx) {
    up::UpdateInstruction ins;
    std::memcpy(&ins, static_cast<const uint8_t*>(program) + idx * 64, 64);
    const uint64_t* in = ins.in;
    const uint64_t* out = ins.out;
    switch (static_cast<up::OpCode>(ins.opcode)) {
      case up::OpCode::kNop: break;
      case up::OpCode::kGemmNN:
        k::GemmNN(R(in[0]), R(in[1]), W(in[2]), out[0], out[1], out[2],
                  ins.flags & up::kFlagEpilogueBias ? R(in[3]) : nullptr,
                  up::EpilogueActOf(ins.flags));
        break;
      case up::OpCode::kGemmNT:
        k::GemmNT(R(in[0]), R(in[1]), W(in[2]), out[0], out[1], out[2]); break;
      case up::OpCode::kGemmTN:
        k::GemmTN(R(in[0]), R(in[1]), W(in[2]), out[0], out[1], out[2]); break;
      case up::OpCode::kGemmAccNN:
        k::GemmAccNN(R(in[0]), R(in[1]), W(in[2]), out[0], out[1], out[2],
                     Bits(in[3]));
        break;
      case up::OpCode::kGemmNNQ8:
        k::GemmNNQ8(R(in[0]), reinterpret_cast<const int8_t*>(R(in[1])),
                    W(in[2]), out[0], out[1], out[2], Bits(in[3]),
                    up::EpilogueActOf(ins.flags));
        break;
      case up::OpCode::kGemmNTQ8:
        k::GemmNTQ8(R(in[0]), reinterpret_cast<const int8_t*>(R(in[1])),
                    W(in[2]), out[0], out[1], out[2], Bits(in[3]));
        break;
      case up::OpCode::kAddEW: k::AddEW(R(in[0]), R(in[1]), W(in[2]), out[0]); break;
      case up::OpCode::kMulEW: k::MulEW(R(in[0]), R(in[1]), W(in[2]), out[0]); break;
      case up::OpCode::kAddBias:
        k::AddBias(R(in[0]), R(in[1]), W(in[2]), out[0], out[1]); break;
      case up::OpCode::kReluFwd: k::ReluFwd(R(in[0]), W(in[1]), out[0]); break;
      case up::OpCode::kReluBwd: k::ReluBwd(R(in[0]), R(in[1]), W(in[2]), out[0]); break;
      case up::OpCode::kGeluFwd: k::GeluFwd(R(in[0]), W(in[1]), out[0]); break;
      case up::OpCode::kGeluBwd: k::GeluBwd(R(in[0]), R(in[1]), W(in[2]), out[0]); break;
      case up::OpCode::kSiluFwd: k::SiluFwd(R(in[0]), W(in[1]), out[0]); break;
      case up::OpCode::kSiluBwd: k::SiluBwd(R(in[0]), R(in[1]), W(in[2]), out[0]); break;
      case up::OpCode::kLayerNormFwd:
        k::LayerNormFwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), W(out[1]),
                        W(out[2]), hi(out[0]), lo(out[0]));
        break;
      case up::OpCode::kLayerNormBwd:
        k::LayerNormBwd(R(in[0]), R(in[1]), R(in[2]), R(out[0]), R(out[1]),
                        W(in[3]), hi(out[2]), lo(out[2]));
        break;
      case up::OpCode::kClipNorm: k::ClipNorm(W(in[0]), out[0], Bits(in[1])); break;
      case up::OpCode::kScale: k::Scale(R(in[0]), W(in[1]), Bits(in[2]), out[0]); break;
      case up::OpCode::kReduceRows: k::ReduceRows(R(in[0]), W(in[1]), out[0], out[1]); break;
      case up::OpCode::kSoftmaxXEntFwd:
        k::SoftmaxXEntFwd(R(in[0]), I(in[1]), W(in[2]), W(in[3]), out[0], out[1]); break;
      case up::OpCode::kSoftmaxXEntBwd:
        k::SoftmaxXEntBwd(R(in[0]), I(in[1]), R(in[2]), W(in[3]), out[0], out[1]); break;
      case up::OpCode::kMseFwd: k::MseFwd(R(in[0]), R(in[1]), W(in[2]), out[0]); break;
      case up::OpCode::kMseBwd:
        k::MseBwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), out[0]); break;
      case up::OpCode::kKLDistillFwd:
        k::KLDistillFwd(R(in[0]), R(in[1]), W(in[2]), W(in[3]), W(out[0]),
                        hi(out[1]), lo(out[1]), Bits(out[2]));
        break;
      case up::OpCode::kKLDistillBwd:
        k::KLDistillBwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), hi(out[0]),
                        lo(out[0]), Bits(out[1]));
        break;
      case up::OpCode::kSgdStep: k::SgdStep(W(in[0]), R(in[1]), out[0], lr, wd); break;
      case up::OpCode::kAdamWStep:
        k::AdamWStep(W(in[0]), R(in[1]), W(in[2]), W(in[3]), out[0], lr, beta1,
                     beta2, eps, wd, step);
        break;
      case up::OpCode::kFill: k::Fill(W(in[0]), Bits(in[1]), out[0]); break;
      case up::OpCode::kCopy: k::Copy(R(in[0]), W(in[1]), out[0]); break;
      case up::OpCode::kRmsNormFwd:
        k::RmsNormFwd(R(in[0]), R(in[1]), W(in[2]), W(in[3]), hi(out[0]), lo(out[0])); break;
      case up::OpCode::kRmsNormBwd:
        k::RmsNormBwd(R(in[0]), R(in[1]), R(in[2]), R(out[0]), W(in[3]),
                      hi(out[1]), lo(out[1]));
        break;
      case up::OpCode::kRopeFwd:
        k::RopeFwd(R(in[0]), W(in[1]), hi(out[0]), lo(out[0]), hi(out[1]),
                   lo(out[1]), Bits(out[2]));
        break;
      case up::OpCode::kRopeBwd:
        k::RopeBwd(R(in[0]), W(in[1]), hi(out[0]), lo(out[0]), hi(out[1]),
                   lo(out[1]), Bits(out[2]));
        break;
      case up::OpCode::kAttnFwd:
        k::AttnFwd(R(in[0]), R(in[1]), R(in[2]), W(in[3]), W(out[0]),
                   hi(out[1]), lo(out[1]), hi(out[2]), lo(out[2]));
        break;
      case up::OpCode::kAttnDP:
        k::AttnDP(R(in[0]), R(in[1]), W(in[2]), hi(out[0]), lo(out[0]),
                  hi(out[1]), lo(out[1]));
        break;
      case up::OpCode::kAttnDV:
        k::AttnDV(R(in[0]), R(in[1]), W(in[2]), hi(out[0]), lo(out[0]),
                  hi(out[1]), lo(out[1]));
        break;
      case up::OpCode::kSoftmaxRowsBwd:
        k::SoftmaxRowsBwd(R(in[0]), R(in[1]), W(in[2]), hi(out[0]), lo(out[0])); break;
      case up::OpCode::kAttnDQ:
        k::AttnDQ(R(in[0]), R(in[1]), W(in[2]), hi(out[0]), lo(out[0]),
                  hi(out[1]), lo(out[1]));
        break;
      case up::OpCode::kAttnDK:
        k::AttnDK(R(in[0]), R(in[1]), W(in[2]), hi(out[0]), lo(out[0]),
                  hi(out[1]), lo(out[1]));
        break;
      case up::OpCode::kEmbedFwd:
        k::EmbedFwd(I(in[0]), R(in[1]), W(in[2]), out[0], lo(out[1])); break;
    }
  }
}

// --- compiler ----------------------------------------------------------------
// Compiles `smf_path` into a sealed plan written to `out_plan_path`.
// targets_csv: comma-separated LoRA target filters ("" = all).
// loss: 0 xent, 1 mse. optimizer: 0 sgd, 1 adamw. lr_schedule: 0 const, 1 cosine.
int ref_compile(const char* smf_path, const char* out_plan_path, int64_t batch,
                int64_t lora_rank, float lora_alpha, uint64_t lora_seed,
                const char* targets_csv, int loss, int optimizer, float lr,
                float weight_decay, float clip_norm, int lr_schedule,
                uint64_t warmup, float min_lr_factor, uint64_t steps,
                int fuse_epilogues, int quantize_base, int emit_optimizer,
                char* err, uint64_t cap) {
  auto model = up::LoadSmf(smf_path);
  if (!model) {
    SetErr(err, cap, model.error());
    return 1;
  }
  up::UpdateConfig cfg;
  cfg.batch = batch;
  cfg.loss = static_cast<up::LossKind>(loss);
  cfg.lora.rank = lora_rank;
  cfg.lora.alpha = lora_alpha;
  cfg.lora.seed = lora_seed;
  {
    std::stringstream ss(targets_csv ? targets_csv : "");
    std::string item;
    while (std::getline(ss, item, ','))
      if (!item.empty()) cfg.lora.target_filters.push_back(item);
  }
  cfg.optimizer.kind = static_cast<up::OptimizerKind>(optimizer);
  cfg.optimizer.lr = lr;
  cfg.optimizer.weight_decay = weight_decay;
  cfg.optimizer.clip_norm = clip_norm;
  cfg.optimizer.lr_schedule = static_cast<up::LrSchedule>(lr_schedule);
  cfg.optimizer.warmup_steps = warmup;
  cfg.optimizer.min_lr_factor = min_lr_factor;
  cfg.default_steps = steps;
  cfg.fuse_epilogues = fuse_epilogues != 0;
  cfg.quantize_base = quantize_base != 0;
  cfg.emit_optimizer = emit_optimizer != 0;
  cfg.memory_budget_bytes = 1ull << 46;  // the gate is not what is under test
  up::UpdateCompiler compiler(cfg);
  auto compiled = compiler.Compile(*model, nullptr);
  if (!compiled) {
    SetErr(err, cap, compiled.error());
    return 2;
  }
  std::ofstream f(out_plan_path, std::ios::binary | std::ios::trunc);
  f.write(reinterpret_cast<const char*>(compiled->plan.data()),
          static_cast<std::streamsize>(compiled->plan.size()));
  f.close();
  if (f.fail()) {
    SetErr(err, cap, "short write");
    return 3;
  }
  return 0;
}

// --- datasets ----------------------------------------------------------------
void* ref_dataset_load(const char* path, char* err, uint64_t cap) {
  auto d = rt::Dataset::LoadFromFile(path);
  if (!d) {
    SetErr(err, cap, d.error());
    return nullptr;
  }
  return new DatasetBox{std::move(*d)};
}
void* ref_dataset_from_tokens(const int32_t* tokens, uint64_t records,
                              uint64_t seq, char* err, uint64_t cap) {
  std::vector<int32_t> t(tokens, tokens + records * (seq + 1));
  auto d = rt::Dataset::FromTokens(std::move(t), records, seq);
  if (!d) {
    SetErr(err, cap, d.error());
    return nullptr;
  }
  return new DatasetBox{std::move(*d)};
}
void* ref_dataset_from_memory(const float* inputs, const uint8_t* labels,
                              uint64_t n, uint64_t dim, uint32_t label_kind,
                              uint64_t label_dim, char* err, uint64_t cap) {
  const uint64_t lb = label_kind == 1 ? 4 : label_kind == 2 ? 4 * label_dim : 0;
  std::vector<float> in(inputs, inputs + n * dim);
  std::vector<uint8_t> lab(labels, labels + n * lb);
  auto d = rt::Dataset::FromMemory(std::move(in), std::move(lab), n, dim,
                                   label_kind, label_dim);
  if (!d) {
    SetErr(err, cap, d.error());
    return nullptr;
  }
  return new DatasetBox{std::move(*d)};
}
void ref_dataset_free(void* d) { delete static_cast<DatasetBox*>(d); }
uint64_t ref_dataset_num_samples(void* d) {
  return static_cast<DatasetBox*>(d)->ds.num_samples();
}
void ref_dataset_enable_shuffle(void* d, uint64_t seed) {
  static_cast<DatasetBox*>(d)->ds.EnableShuffle(seed);
}
void ref_dataset_rewind(void* d) { static_cast<DatasetBox*>(d)->ds.Rewind(); }
void* ref_dataset_split_validation(void* d, double frac, char* err,
                                   uint64_t cap) {
  auto v = static_cast<DatasetBox*>(d)->ds.SplitValidation(frac);
  if (!v) {
    SetErr(err, cap, v.error());
    return nullptr;
  }
  return new DatasetBox{std::move(*v)};
}
void ref_dataset_fill_batch(void* d, uint64_t batch, float* input_slot,
                            uint8_t* label_slot) {
  static_cast<DatasetBox*>(d)->ds.FillBatch(batch, input_slot, label_slot);
}
int ref_dataset_skip_served(void* d, uint64_t rows) {
  return static_cast<DatasetBox*>(d)->ds.SkipServed(rows) ? 0 : 1;
}
int ref_dataset_save(void* d, const char* path) {
  return static_cast<DatasetBox*>(d)->ds.SaveToFile(path) ? 0 : 1;
}

// --- engine ------------------------------------------------------------------
void* ref_engine_new() { return new rt::UpdateEngine(); }
void ref_engine_free(void* e) { delete static_cast<rt::UpdateEngine*>(e); }
int ref_engine_load_file(void* e, const char* path, char* err, uint64_t cap) {
  auto r = static_cast<rt::UpdateEngine*>(e)->LoadFromFile(path);
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}
// The caller keeps `plan` alive for the engine's lifetime.
int ref_engine_load_memory(void* e, const uint8_t* plan, uint64_t n, char* err,
                           uint64_t cap) {
  auto r = static_cast<rt::UpdateEngine*>(e)->LoadFromMemory(plan, n);
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}
uint8_t* ref_engine_arena(void* e) {
  return static_cast<rt::UpdateEngine*>(e)->arena();
}
void ref_engine_header(void* e, void* out280) {
  std::memcpy(out280, &static_cast<rt::UpdateEngine*>(e)->header(), 280);
}
void ref_engine_execute_train_once(void* e) {
  static_cast<rt::UpdateEngine*>(e)->ExecuteTrainOnce();
}
float ref_engine_loss(void* e) {
  return static_cast<rt::UpdateEngine*>(e)->LossValue();
}
uint64_t ref_engine_step(void* e) {
  return static_cast<rt::UpdateEngine*>(e)->step();
}
void ref_engine_set_step(void* e, uint64_t s) {
  static_cast<rt::UpdateEngine*>(e)->SetStep(s);
}
float ref_engine_effective_lr(void* e) {
  return static_cast<rt::UpdateEngine*>(e)->EffectiveLr();
}

struct RefTrainReport {
  uint64_t steps;
  int32_t stopped_early;
  float initial_avg_loss, final_avg_loss;
  int32_t has_validation;
  float val_initial_loss, val_final_loss;
  int32_t has_val_accuracy;
  float val_initial_accuracy, val_final_accuracy;
  int32_t improved;
};

// loss_curve (may be null) receives one float per executed step.
int ref_engine_train(void* e, void* data, uint64_t steps, void* validation,
                     float* loss_curve, RefTrainReport* rep, char* err,
                     uint64_t cap) {
  rt::TrainOptions opt;
  opt.log_every = 0;
  opt.record_loss_curve = loss_curve != nullptr;
  if (validation) opt.validation = &static_cast<DatasetBox*>(validation)->ds;
  auto r = static_cast<rt::UpdateEngine*>(e)->Train(
      static_cast<DatasetBox*>(data)->ds, steps, opt);
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  if (loss_curve)
    std::memcpy(loss_curve, r->loss_curve.data(),
                r->loss_curve.size() * sizeof(float));
  if (rep) {
    rep->steps = r->steps;
    rep->stopped_early = r->stopped_early;
    rep->initial_avg_loss = r->initial_avg_loss;
    rep->final_avg_loss = r->final_avg_loss;
    rep->has_validation = r->has_validation;
    rep->val_initial_loss = r->val_initial_loss;
    rep->val_final_loss = r->val_final_loss;
    rep->has_val_accuracy = r->has_val_accuracy;
    rep->val_initial_accuracy = r->val_initial_accuracy;
    rep->val_final_accuracy = r->val_final_accuracy;
    rep->improved = r->improved();
  }
  return 0;
}

int ref_engine_evaluate(void* e, void* data, float* loss, float* accuracy,
                        int32_t* has_accuracy, char* err, uint64_t cap) {
  auto m = static_cast<rt::UpdateEngine*>(e)->EvaluateMetrics(
      static_cast<DatasetBox*>(data)->ds);
  if (!m) {
    SetErr(err, cap, m.error());
    return 1;
  }
  *loss = m->loss;
  *accuracy = m->accuracy;
  *has_accuracy = m->has_accuracy;
  return 0;
}
int ref_engine_run_merge(void* e, char* err, uint64_t cap) {
  auto r = static_cast<rt::UpdateEngine*>(e)->RunMerge();
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}
int ref_engine_commit(void* e, const char* src, const char* dst, char* err,
                      uint64_t cap) {
  auto r = static_cast<rt::UpdateEngine*>(e)->CommitToModel(src, dst);
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}
int ref_engine_save_checkpoint(void* e, const char* path, char* err,
                               uint64_t cap) {
  auto r = static_cast<rt::UpdateEngine*>(e)->SaveCheckpoint(path);
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}
int ref_engine_load_checkpoint(void* e, const char* path, char* err,
                               uint64_t cap) {
  auto r = static_cast<rt::UpdateEngine*>(e)->LoadCheckpoint(path);
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}
void ref_engine_step_timings(void* e, uint64_t* steps, double* fwd, double* bwd,
                             double* opt) {
  auto t = static_cast<rt::UpdateEngine*>(e)->step_timings();
  *steps = t.steps;
  *fwd = t.fwd_seconds;
  *bwd = t.bwd_seconds;
  *opt = t.opt_seconds;
}

// The reference compiler's native packaging step (native_emitter.cc:420-...): writes
// update_plan.seeu, update_plan_embedded.cc and the generated driver update_main.cc into
// out_dir, then vendors the runtime sources from repo_root. Returns 0 when the whole
// package was written; otherwise 1 with the emitter's message (the plan, embedded TU and
// driver are written before the vendoring step, so they exist even when repo_root does not).
int ref_emit_native_package(const uint8_t* plan, uint64_t size, const char* out_dir,
                            const char* repo_root, char* err, uint64_t cap) {
  std::vector<uint8_t> bytes(plan, plan + size);
  auto r = up::EmitNativePackage(bytes, out_dir, repo_root ? repo_root : "");
  if (!r) {
    SetErr(err, cap, r.error());
    return 1;
  }
  return 0;
}

}  // extern "C"

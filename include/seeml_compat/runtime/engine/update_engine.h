// seeml::update_rt::UpdateEngine over the seeml_b200 C ABI: the reference's public class
// (runtime/engine/update_engine.h:43-190) with the same method names, argument meaning,
// std::expected error surface ("<unit>: <message>" strings) and lifecycle, executed on a
// B200. The driver the reference's compiler generates (update_main.cc: LoadFromMemory ->
// VerifySourceModel -> Dataset::LoadFromFile -> SplitValidation -> EnableShuffle -> Train ->
// gate -> RunMerge -> CommitToModel, compiler/backend/trainer/native_emitter.cc:92-326)
// compiles against this header unchanged:
//
//   g++ -std=c++23 -I include -I include/seeml_compat update_main.cc update_plan_embedded.cc
//       -L see_ml_b200 -lseeml_b200 -Wl,-rpath,see_ml_b200 -o model_update
//
// Header-only. Differences from the reference, all forced by the arena living in device
// memory: arena() is replaced by ArenaRead / ArenaWrite (explicit copies), and the engine is
// created on the device named by SEEML_B200_DEVICE (default 0) in the execution mode named by
// SEEML_B200_MODE ("fused", the default, or "contract") with the GEMM arithmetic named by
// SEEML_B200_GEMM ("f16x2" default, "tf32x3", "tf32", "simt").
#ifndef SEEML_COMPAT_RUNTIME_ENGINE_UPDATE_ENGINE_H_
#define SEEML_COMPAT_RUNTIME_ENGINE_UPDATE_ENGINE_H_

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <expected>
#include <functional>
#include <string>
#include <vector>

#include "runtime/feeder/dataset.h"
#include "seeml_b200.h"
#include "source/plan/update_types.h"

namespace seeml::update_rt {

struct TrainOptions {
  std::string checkpoint_path;
  uint64_t checkpoint_every = 0;
  uint64_t log_every = 100;
  bool resume = false;
  Dataset* validation = nullptr;
  std::function<bool()> should_stop;
  bool record_loss_curve = false;
};

struct EvalMetrics {
  float loss = 0.0f;
  float accuracy = 0.0f;
  bool has_accuracy = false;
};

struct StepTimings {   // measured with CUDA events at the reference's two phase boundaries
  uint64_t steps = 0;
  double fwd_seconds = 0.0;
  double bwd_seconds = 0.0;
  double opt_seconds = 0.0;
};

struct TrainReport {
  uint64_t steps = 0;
  bool stopped_early = false;
  float initial_avg_loss = 0.0f;
  float final_avg_loss = 0.0f;
  bool has_validation = false;
  float val_initial_loss = 0.0f;
  float val_final_loss = 0.0f;
  bool has_val_accuracy = false;
  float val_initial_accuracy = 0.0f;
  float val_final_accuracy = 0.0f;
  std::vector<float> loss_curve;
  bool improved() const {
    return has_validation ? val_final_loss < val_initial_loss : final_avg_loss < initial_avg_loss;
  }
};

class UpdateEngine {
 public:
  UpdateEngine() = default;
  ~UpdateEngine() { seeml_b200_engine_destroy(e_); }
  UpdateEngine(const UpdateEngine&) = delete;
  UpdateEngine& operator=(const UpdateEngine&) = delete;

  [[nodiscard]] std::expected<void, std::string> LoadFromMemory(const uint8_t* plan, size_t size) {
    if (auto r = Ensure(); !r) return r;
    return Loaded(seeml_b200_engine_load_memory(e_, plan, size));
  }
  [[nodiscard]] std::expected<void, std::string> LoadFromFile(const std::string& path) {
    if (auto r = Ensure(); !r) return r;
    return Loaded(seeml_b200_engine_load_file(e_, path.c_str()));
  }

  [[nodiscard]] std::expected<TrainReport, std::string> Train(Dataset& data, uint64_t steps,
                                                              const TrainOptions& options = {}) {
    if (!e_) return std::unexpected("UpdateEngine: no plan loaded");
    seeml_b200_train_options o{};
    o.checkpoint_path = options.checkpoint_path.empty() ? nullptr : options.checkpoint_path.c_str();
    o.checkpoint_every = options.checkpoint_every;
    o.log_every = options.log_every;
    o.resume = options.resume ? 1 : 0;
    o.validation = options.validation ? options.validation->handle() : nullptr;
    if (options.should_stop) {
      o.should_stop = [](void* user) -> int { return (*static_cast<const std::function<bool()>*>(user))() ? 1 : 0; };
      o.user = const_cast<std::function<bool()>*>(&options.should_stop);
    }
    TrainReport rep;
    const uint64_t n = steps ? steps : header_.default_steps;
    if (options.record_loss_curve) rep.loss_curve.assign(n, 0.0f);
    o.loss_curve = options.record_loss_curve && n ? rep.loss_curve.data() : nullptr;
    seeml_b200_train_report r{};
    if (seeml_b200_engine_train(e_, data.handle(), steps, &o, &r) != 0) return std::unexpected(Err());
    rep.steps = r.steps;
    rep.stopped_early = r.stopped_early != 0;
    rep.initial_avg_loss = r.initial_avg_loss;
    rep.final_avg_loss = r.final_avg_loss;
    rep.has_validation = r.has_validation != 0;
    rep.val_initial_loss = r.val_initial_loss;
    rep.val_final_loss = r.val_final_loss;
    rep.has_val_accuracy = r.has_val_accuracy != 0;
    rep.val_initial_accuracy = r.val_initial_accuracy;
    rep.val_final_accuracy = r.val_final_accuracy;
    if (options.record_loss_curve) rep.loss_curve.resize(r.steps);
    return rep;
  }

  [[nodiscard]] std::expected<float, std::string> Evaluate(Dataset& data) {
    auto m = EvaluateMetrics(data);
    if (!m) return std::unexpected(m.error());
    return m->loss;
  }
  [[nodiscard]] std::expected<EvalMetrics, std::string> EvaluateMetrics(Dataset& data) {
    if (!e_) return std::unexpected("UpdateEngine: no plan loaded");
    EvalMetrics m;
    int32_t has = 0;
    if (seeml_b200_engine_evaluate(e_, data.handle(), &m.loss, &m.accuracy, &has) != 0) return std::unexpected(Err());
    m.has_accuracy = has != 0;
    return m;
  }

  [[nodiscard]] std::expected<void, std::string> RunMerge() { return Status(e_ ? seeml_b200_engine_run_merge(e_) : NoPlan()); }
  [[nodiscard]] std::expected<void, std::string> CommitToModel(const std::string& source_model_path,
                                                               const std::string& out_path) const {
    return Status(e_ ? seeml_b200_engine_commit(e_, source_model_path.c_str(), out_path.c_str()) : NoPlan());
  }
  [[nodiscard]] std::expected<void, std::string> VerifySourceModel(const std::string& source_model_path) const {
    return Status(e_ ? seeml_b200_engine_verify_source_model(e_, source_model_path.c_str()) : NoPlan());
  }
  [[nodiscard]] std::expected<void, std::string> SaveCheckpoint(const std::string& path) const {
    return Status(e_ ? seeml_b200_engine_save_checkpoint(e_, path.c_str()) : NoPlan());
  }
  [[nodiscard]] std::expected<void, std::string> LoadCheckpoint(const std::string& path) {
    return Status(e_ ? seeml_b200_engine_load_checkpoint(e_, path.c_str()) : NoPlan());
  }

  const seeml::update::PlanHeader& header() const { return header_; }
  float LossValue() const {
    float v = 0.0f;
    if (e_) seeml_b200_engine_loss(e_, &v);
    return v;
  }
  uint64_t step() const { return e_ ? seeml_b200_engine_step(e_) : 0; }
  void SetStep(uint64_t s) { if (e_) seeml_b200_engine_set_step(e_, s); }
  float EffectiveLr() const { return e_ ? seeml_b200_engine_effective_lr(e_) : 0.0f; }
  void ExecuteTrainOnce() { if (e_) seeml_b200_engine_execute_train_once(e_); }

  StepTimings step_timings() const {
    StepTimings t;
    if (e_) seeml_b200_engine_step_timings(e_, &t.steps, &t.fwd_seconds, &t.bwd_seconds, &t.opt_seconds);
    return t;
  }
  void ResetStepTimings() { if (e_) seeml_b200_engine_reset_step_timings(e_); }
  /// Turns the phase timing on or off (the reference compiles it in with -DSEEML_STEP_TIMING;
  /// here it is a run-time switch because it costs a device synchronisation per step).
  void EnableStepTiming(bool on) { if (e_) seeml_b200_engine_enable_step_timing(e_, on ? 1 : 0); }

  /// The arena is device memory: tests that peek and poke through arena() in the reference use
  /// these explicit copies instead.
  [[nodiscard]] std::expected<void, std::string> ArenaRead(uint64_t offset, void* dst, uint64_t bytes) {
    return Status(e_ ? seeml_b200_engine_arena_read(e_, offset, dst, bytes) : NoPlan());
  }
  [[nodiscard]] std::expected<void, std::string> ArenaWrite(uint64_t offset, const void* src, uint64_t bytes) {
    return Status(e_ ? seeml_b200_engine_arena_write(e_, offset, src, bytes) : NoPlan());
  }
  seeml_b200_engine* handle() const { return e_; }

 private:
  static std::string Err() { return std::string(seeml_b200_last_error()); }
  static int NoPlan() { return -1; }
  static std::expected<void, std::string> Status(int rc) {
    if (rc == -1) return std::unexpected("UpdateEngine: no plan loaded");
    if (rc != 0) return std::unexpected(Err());
    return {};
  }
  static uint32_t EnvChoice(const char* name, std::initializer_list<const char*> names, uint32_t dflt) {
    const char* v = std::getenv(name);
    if (!v) return dflt;
    uint32_t i = 0;
    for (const char* n : names) {
      if (std::strcmp(v, n) == 0) return i;
      ++i;
    }
    return dflt;
  }
  std::expected<void, std::string> Ensure() {
    if (e_) return {};
    const char* dev = std::getenv("SEEML_B200_DEVICE");
    e_ = seeml_b200_engine_create(dev ? std::atoi(dev) : 0, EnvChoice("SEEML_B200_MODE", {"contract", "fused"}, 1),
                                  EnvChoice("SEEML_B200_GEMM", {"tf32x3", "f16x2", "simt", "tf32"}, 1));
    if (!e_) return std::unexpected(Err());
    return {};
  }
  std::expected<void, std::string> Loaded(int rc) {
    if (rc != 0) return std::unexpected(Err());
    seeml_b200_engine_header(e_, &header_);
    return {};
  }
  seeml_b200_engine* e_ = nullptr;
  seeml::update::PlanHeader header_{};
};

}  // namespace seeml::update_rt

#endif  // SEEML_COMPAT_RUNTIME_ENGINE_UPDATE_ENGINE_H_

// UpdateEngine on a B200: plan admission, the device arena, the train / evaluate /
// merge loops and the checkpoint / commit hand-off, with the lifecycle and error
// behaviour of the reference engine (runtime/engine/update_engine.cc:80-911) and
// every tensor operation on the GPU. The feeder stages batches through pinned host
// double buffers and a copy stream while the previous step computes; the batch
// sequence is exactly the serial FillBatch sequence
// (runtime/feeder/batch_pipeline.cc:9-79).
#include <fcntl.h>
#include <sys/file.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>

#include "backend.h"
#include "dataset.h"

using namespace seeml_b200;

namespace {

// Pinned double buffer + one staging thread. At most two batches are staged ahead;
// at teardown the dataset position is put back to "exactly the batches consumed".
class Feeder {
 public:
  Feeder(seeml_b200_dataset& d, uint64_t batch, uint64_t in_bytes, uint64_t lab_bytes)
      : d_(d), batch_(batch), in_bytes_(in_bytes), lab_bytes_(lab_bytes) {
    for (auto& b : buf_) {
      b.in = static_cast<uint8_t*>(seeml_b200_pinned_alloc(in_bytes));
      b.lab = lab_bytes ? static_cast<uint8_t*>(seeml_b200_pinned_alloc(lab_bytes)) : nullptr;
    }
    thread_ = std::thread([this] { loop(); });
  }
  ~Feeder() {
    {
      std::lock_guard<std::mutex> lk(m_);
      stop_ = true;
    }
    cv_.notify_all();
    thread_.join();
    // un-consume whatever was staged (or handed out) but never executed
    bool have = false;
    seeml_b200_dataset::Pos earliest{0, 0};
    if (handed_unconsumed_) { earliest = handed_pos_; have = true; }
    for (int k = 0; k < 2 && !have; ++k) {
      const Buf& b = buf_[(head_ + k) % 2];
      if (b.full) { earliest = b.before; have = true; }
    }
    if (have) d_.restore_pos(earliest);
    for (auto& b : buf_) {
      seeml_b200_pinned_free(b.in);
      seeml_b200_pinned_free(b.lab);
    }
  }
  // Next staged batch, in serving order. The buffer stays owned by the caller until release().
  int acquire(const uint8_t** in, const uint8_t** lab) {
    std::unique_lock<std::mutex> lk(m_);
    cv_.wait(lk, [&] { return buf_[head_].full; });
    const int idx = head_;
    *in = buf_[idx].in;
    *lab = buf_[idx].lab;
    handed_pos_ = buf_[idx].before;
    handed_unconsumed_ = true;
    return idx;
  }
  void consumed() { handed_unconsumed_ = false; }   // the handed batch was executed
  void release(int idx) {
    {
      std::lock_guard<std::mutex> lk(m_);
      buf_[idx].full = false;
      head_ = (idx + 1) % 2;
    }
    cv_.notify_all();
  }

 private:
  struct Buf {
    uint8_t* in = nullptr;
    uint8_t* lab = nullptr;
    bool full = false;
    seeml_b200_dataset::Pos before{0, 0};
  };
  void loop() {
    int tail = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lk(m_);
        cv_.wait(lk, [&] { return !buf_[tail].full || stop_; });
        if (stop_) return;
      }
      buf_[tail].before = d_.save_pos();
      d_.fill_batch(batch_, buf_[tail].in, buf_[tail].lab);
      {
        std::lock_guard<std::mutex> lk(m_);
        buf_[tail].full = true;
      }
      cv_.notify_all();
      tail = (tail + 1) % 2;
    }
  }
  seeml_b200_dataset& d_;
  uint64_t batch_, in_bytes_, lab_bytes_;
  Buf buf_[2];
  int head_ = 0;
  bool stop_ = false, handed_unconsumed_ = false;
  seeml_b200_dataset::Pos handed_pos_{0, 0};
  std::mutex m_;
  std::condition_variable cv_;
  std::thread thread_;
};

struct Loaded {
  PlanHeader h{};
  seeml_b200_ctx* ctx = nullptr;
  int train = -1, eval = -1, merge = -1;
  std::vector<EmitEntry> emit;
  std::vector<Instr> train_instrs;
  uint64_t num_classes = 0, vocab_bound = 0;
  uint64_t eval_probs_ref = kNullRef, eval_rows = 0, eval_cols = 0;
  uint64_t bwd_begin = 0, opt_begin = 0;
  std::vector<uint8_t> owned;
};

}  // namespace

// K-chunk data-parallel step (configured by seeml_b200_engine_dp_configure).
struct DpState {
  uint64_t K = 0, local = 0, fps = 0;           // chunks per step, chunks on this rank, floats per packed set
  int rank = 0, world = 1;
  seeml_b200_comm* comm = nullptr;              // borrowed; null when world == 1
  float* sets = nullptr;                        // [local][fps]: one packed gradient set (+ loss) per chunk
  float* gathered = nullptr;                    // [world][fps]
  k::Span* spans = nullptr;                     // device span table: gradient operands, then the loss slot
  uint64_t nspans = 0;
  uint8_t* pin_in[2] = {nullptr, nullptr};
  uint8_t* pin_lab[2] = {nullptr, nullptr};
  uint64_t launches = 0;
  double timeout_s = 120.0;
};

struct seeml_b200_engine {
  int device = 0;
  uint32_t mode = SEEML_B200_MODE_CONTRACT, gemm = SEEML_B200_GEMM_TF32X3;
  Loaded L;
  bool loaded = false;
  uint64_t step = 0;
  bool merged = false;
  uint64_t last_launches = 0;
  bool timing = false;
  uint64_t t_steps = 0;
  double t_fwd = 0, t_bwd = 0, t_opt = 0;
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  unsigned long long* counter_dev = nullptr;
  DpState dp;
};

namespace {

void free_dp(DpState& d) {
  cudaFree(d.sets);
  cudaFree(d.gathered);
  cudaFree(d.spans);
  for (int i = 0; i < 2; ++i) {
    seeml_b200_pinned_free(d.pin_in[i]);
    seeml_b200_pinned_free(d.pin_lab[i]);
  }
  d = DpState{};
}

void free_loaded(Loaded& L) {
  if (L.ctx) seeml_b200_ctx_destroy(L.ctx);
  L = Loaded{};
}

float effective_lr(const PlanHeader& h, uint64_t step) {  // update_engine.cc:515-534
  const float base = h.lr;
  if (h.lr_schedule != 1) return base;
  if (h.warmup_steps > 0 && step <= h.warmup_steps)
    return base * static_cast<float>(step) / static_cast<float>(h.warmup_steps);
  const uint64_t horizon = h.default_steps > h.warmup_steps ? h.default_steps - h.warmup_steps : 0;
  const float floor_lr = base * h.min_lr_factor;
  if (horizon == 0 || step - h.warmup_steps >= horizon) return floor_lr;
  const float t = static_cast<float>(step - h.warmup_steps) / static_cast<float>(horizon);
  constexpr float kPi = 3.14159265358979323846f;
  return floor_lr + (base - floor_lr) * 0.5f * (1.0f + std::cos(kPi * t));
}

seeml_b200_scalars scalars_of(const seeml_b200_engine* e) {
  const PlanHeader& h = e->L.h;
  seeml_b200_scalars s{};
  s.lr = effective_lr(h, e->step);
  s.beta1 = h.beta1; s.beta2 = h.beta2; s.eps = h.eps; s.weight_decay = h.weight_decay;
  s.step = e->step;
  return s;
}

int initialize(seeml_b200_engine* e, const uint8_t* plan, uint64_t size, std::vector<uint8_t>&& owned) {
  Loaded L;
  const std::string err = verify_plan(plan, size, &L.h);
  if (!err.empty()) return fail(err);
  const PlanHeader& h = L.h;
  std::vector<Instr> train(h.train_instr_count), merge(h.merge_instr_count), eval(h.eval_instr_count);
  if (!train.empty()) std::memcpy(train.data(), plan + h.train_instr_offset, train.size() * 64);
  if (!merge.empty()) std::memcpy(merge.data(), plan + h.merge_instr_offset, merge.size() * 64);
  if (!eval.empty()) std::memcpy(eval.data(), plan + h.eval_instr_offset, eval.size() * 64);
  L.emit.resize(h.emit_count);
  if (h.emit_count) std::memcpy(L.emit.data(), plan + h.emit_table_offset, h.emit_count * 24);
  // narrowest softmax width / embedding table anywhere: the runtime bound on staged ids
  for (const auto* prog : {&train, &merge, &eval})
    for (const Instr& ins : *prog) {
      if (ins.opcode == kXentFwd || ins.opcode == kXentBwd) {
        const uint64_t cls = ins.out[1];
        if (cls != 0 && (L.num_classes == 0 || cls < L.num_classes)) L.num_classes = cls;
      }
      if (ins.opcode == kEmbedFwd) {
        const uint64_t v = ins.out[1] >> 32;
        if (v != 0 && (L.vocab_bound == 0 || v < L.vocab_bound)) L.vocab_bound = v;
      }
    }
  for (const Instr& ins : eval)
    if (ins.opcode == kXentFwd) {
      L.eval_probs_ref = ins.in[3];
      L.eval_rows = ins.out[0];
      L.eval_cols = ins.out[1];
    }
  // phase boundaries: forward ends after the last loss-forward; the optimiser phase starts
  // at the first clip/step instruction (update_engine.cc:243-263)
  L.bwd_begin = L.opt_begin = train.size();
  for (size_t i = 0; i < train.size(); ++i) {
    const uint16_t op = train[i].opcode;
    if (op == kXentFwd || op == kMseFwd || op == kKlFwd) L.bwd_begin = i + 1;
    if ((op == kClipNorm || op == kSgd || op == kAdamW) && L.opt_begin == train.size()) L.opt_begin = i;
  }
  if (L.opt_begin < L.bwd_begin) L.opt_begin = L.bwd_begin;

  if (int r = seeml_b200_ctx_create(e->device, h.arena_size, plan + h.rodata_offset, h.rodata_size,
                                    plan + h.persist_init_offset, h.persist_init_size, nullptr, &L.ctx))
    return r;
  seeml_b200_ctx_set_gemm(L.ctx, e->gemm);
  int rc = seeml_b200_program_build(L.ctx, train.data(), train.size(), h.version, e->mode, &L.train);
  if (!rc) rc = seeml_b200_program_build(L.ctx, eval.data(), eval.size(), h.version, e->mode, &L.eval);
  if (!rc) rc = seeml_b200_program_build(L.ctx, merge.data(), merge.size(), h.version,
                                         SEEML_B200_MODE_CONTRACT, &L.merge);
  if (rc) {
    seeml_b200_ctx_destroy(L.ctx);
    return rc;
  }
  L.train_instrs = std::move(train);
  L.owned = std::move(owned);
  // commit: nothing below can fail
  free_dp(e->dp);
  free_loaded(e->L);
  e->L = std::move(L);
  e->loaded = true;
  e->step = 0;
  e->merged = false;
  e->t_steps = 0;
  e->t_fwd = e->t_bwd = e->t_opt = 0;
  return 0;
}

// runtime/engine/contract.cc:170-235
int verify_feeder(const seeml_b200_engine* e, const seeml_b200_dataset& d) {
  const PlanHeader& h = e->L.h;
  if (h.input_kind == 1) {
    if (d.input_kind != 1)
      return fail("UpdateEngine: the compiled plan takes token ids, but the dataset carries feature rows");
    if (d.input_dim != h.seq_len)
      return fail("UpdateEngine: dataset sequence length does not match the compiled plan");
    if (h.input_floats != h.batch)
      return fail("UpdateEngine: token plan input slot does not hold one id per batch row");
    if (h.label_kind == 1) {
      if (h.batch > UINT64_MAX / 4 || h.batch * 4 != h.label_bytes)
        return fail("UpdateEngine: token plan label slot does not hold one id per batch row");
    } else if (h.label_kind != 0) {
      return fail("UpdateEngine: token plans take class labels or none, not dense labels");
    }
    uint64_t bound = e->L.vocab_bound;
    if (e->L.num_classes != 0 && (bound == 0 || e->L.num_classes < bound)) bound = e->L.num_classes;
    const std::string err = d.validate_labels(bound);
    return err.empty() ? 0 : fail(err);
  }
  if (d.input_kind != 0)
    return fail("UpdateEngine: the compiled plan takes feature rows, but the dataset carries token ids");
  if (d.input_dim != 0 && h.batch > UINT64_MAX / d.input_dim)
    return fail("UpdateEngine: dataset input width does not match the compiled plan");
  if (h.batch * d.input_dim != h.input_floats)
    return fail("UpdateEngine: dataset input width does not match the compiled plan");
  if (h.label_kind != 0) {
    if (d.label_kind != h.label_kind)
      return fail("UpdateEngine: dataset label kind does not match the compiled plan");
    if (h.batch * d.label_bytes_per_sample() != h.label_bytes)
      return fail("UpdateEngine: dataset label width does not match the compiled plan");
  }
  if (h.label_kind == 1) {
    const std::string err = d.validate_labels(e->L.num_classes);
    if (!err.empty()) return fail(err);
  }
  return 0;
}

// One execution of the train stream (optionally split at the phase boundaries for timing).
int run_train(seeml_b200_engine* e) {
  Loaded& L = e->L;
  const seeml_b200_scalars sc = scalars_of(e);
  const uint64_t n = L.train_instrs.size();
  if (!e->timing) {
    if (int r = seeml_b200_program_run(L.ctx, L.train, 0, n, &sc)) return r;
    e->last_launches = seeml_b200_program_launches(L.ctx, L.train);
    return 0;
  }
  cudaStream_t st = static_cast<cudaStream_t>(seeml_b200_ctx_stream(L.ctx));
  uint64_t launches = 0;
  cudaEventRecord(e->ev[0], st);
  if (int r = seeml_b200_program_run(L.ctx, L.train, 0, L.bwd_begin, &sc)) return r;
  launches += seeml_b200_program_launches(L.ctx, L.train);
  cudaEventRecord(e->ev[1], st);
  if (int r = seeml_b200_program_run(L.ctx, L.train, L.bwd_begin, L.opt_begin, &sc)) return r;
  launches += seeml_b200_program_launches(L.ctx, L.train);
  cudaEventRecord(e->ev[2], st);
  if (int r = seeml_b200_program_run(L.ctx, L.train, L.opt_begin, n, &sc)) return r;
  launches += seeml_b200_program_launches(L.ctx, L.train);
  cudaEventRecord(e->ev[3], st);
  cudaEventSynchronize(e->ev[3]);
  float a = 0, b = 0, c = 0;
  cudaEventElapsedTime(&a, e->ev[0], e->ev[1]);
  cudaEventElapsedTime(&b, e->ev[1], e->ev[2]);
  cudaEventElapsedTime(&c, e->ev[2], e->ev[3]);
  ++e->t_steps;
  e->t_fwd += a * 1e-3;
  e->t_bwd += b * 1e-3;
  e->t_opt += c * 1e-3;
  e->last_launches = launches;
  return 0;
}

struct EvalOut { float loss = 0, acc = 0; bool has_acc = false; };

// update_engine.cc:557-650
int evaluate(seeml_b200_engine* e, seeml_b200_dataset& data, EvalOut* out) {
  Loaded& L = e->L;
  const PlanHeader& h = L.h;
  if (!e->loaded) return fail("UpdateEngine: no plan loaded");
  if (h.eval_instr_count == 0) return fail("UpdateEngine: plan carries no eval program");
  if (int r = verify_feeder(e, data)) return r;
  const seeml_b200_dataset::Pos entry = data.save_pos();
  data.cursor = 0;
  const bool track = h.label_kind == 1 && L.eval_probs_ref != kNullRef && L.eval_cols > 0 &&
                     L.eval_rows >= h.batch;
  const uint64_t rows_per_sample = h.input_kind == 1 ? h.seq_len : 1;
  const uint64_t per_step = h.batch / rows_per_sample;
  const uint64_t batches = std::max<uint64_t>(1, (data.samples + per_step - 1) / per_step);
  double total = 0.0;
  uint64_t counted = 0;
  cudaStream_t st = static_cast<cudaStream_t>(seeml_b200_ctx_stream(L.ctx));
  if (track) cudaMemsetAsync(e->counter_dev, 0, sizeof(unsigned long long), st);
  int rc = 0;
  {
    Feeder feeder(data, h.batch, h.input_floats * 4, h.label_kind == 0 ? 0 : h.label_bytes);
    const seeml_b200_scalars sc = scalars_of(e);
    for (uint64_t b = 0; b < batches && !rc; ++b) {
      const uint8_t *in, *lab;
      const int idx = feeder.acquire(&in, &lab);
      rc = seeml_b200_stage_h2d(L.ctx, (int)(b & 1), in, h.input_floats * 4, lab,
                                h.label_kind == 0 ? 0 : h.label_bytes);
      if (!rc) rc = seeml_b200_stage_commit(L.ctx, (int)(b & 1), ref_off(h.input_ref), ref_off(h.label_ref));
      if (!rc) rc = seeml_b200_stage_wait(L.ctx, (int)(b & 1));
      feeder.consumed();
      feeder.release(idx);
      if (!rc) rc = seeml_b200_program_run(L.ctx, L.eval, 0, h.eval_instr_count, &sc);
      if (rc) break;
      if (track) {
        const uint64_t served = b * per_step;
        const uint64_t real_samples =
            std::min<uint64_t>(per_step, data.samples > served ? data.samples - served : 0);
        const uint64_t real = real_samples * rows_per_sample;
        k::count_correct(reinterpret_cast<const float*>(static_cast<uint8_t*>(seeml_b200_ctx_arena(L.ctx)) +
                                                        ref_off(L.eval_probs_ref)),
                         reinterpret_cast<const int32_t*>(static_cast<uint8_t*>(seeml_b200_ctx_arena(L.ctx)) +
                                                          ref_off(h.label_ref)),
                         real, L.eval_cols, e->counter_dev, st);
        counted += real;
      }
      float loss = 0;
      rc = seeml_b200_read_f32(L.ctx, ref_off(h.loss_ref), &loss);
      total += loss;
    }
  }
  data.restore_pos(entry);
  if (rc) return rc;
  out->loss = static_cast<float>(total / static_cast<double>(batches));
  if (track && counted > 0) {
    unsigned long long correct = 0;
    cudaMemcpyAsync(&correct, e->counter_dev, sizeof(correct), cudaMemcpyDeviceToHost, st);
    cudaStreamSynchronize(st);
    out->acc = static_cast<float>(static_cast<double>(correct) / static_cast<double>(counted));
    out->has_acc = true;
  }
  return 0;
}

int write_all(int fd, const void* p, size_t n) {
  const auto* b = static_cast<const uint8_t*>(p);
  while (n) {
    const ssize_t w = ::write(fd, b, n);
    if (w <= 0) return 1;
    b += w;
    n -= static_cast<size_t>(w);
  }
  return 0;
}
// write to a sidecar, fsync, rename into place (runtime/custodian/durable_io.cc:47-80)
int write_file_durable(const std::string& path, const void* a, size_t an, const void* b, size_t bn) {
  const std::string tmp = path + ".tmp." + std::to_string(::getpid());
  const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return fail("DurableIO: cannot write '" + tmp + "'");
  int bad = write_all(fd, a, an) || (bn && write_all(fd, b, bn));
  if (!bad && ::fsync(fd) != 0) bad = 1;
  ::close(fd);
  if (bad) {
    ::unlink(tmp.c_str());
    return fail("DurableIO: short write to '" + tmp + "'");
  }
  if (std::rename(tmp.c_str(), path.c_str()) != 0) {
    ::unlink(tmp.c_str());
    return fail("DurableIO: cannot rename '" + tmp + "' into place");
  }
  return 0;
}

#pragma pack(push, 1)
struct CkptHeader {  // SEKP v3, runtime/custodian/checkpoint.cc:17-35
  uint32_t magic = 0x504B4553, version = 3;
  uint64_t plan_hash = 0, step = 0, persistent_size = 0, payload_hash = 0;
};
#pragma pack(pop)

}  // namespace

extern "C" {

seeml_b200_engine* seeml_b200_engine_create(int device, uint32_t mode, uint32_t gemm_kind) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    fail("UpdateEngine: no CUDA device available — this backend has no CPU fallback");
    return nullptr;
  }
  if (device < 0 || device >= count) {
    fail("UpdateEngine: device ordinal out of range");
    return nullptr;
  }
  if (mode > SEEML_B200_MODE_FUSED || gemm_kind > SEEML_B200_GEMM_TF32) {
    fail("UpdateEngine: unknown execution mode");
    return nullptr;
  }
  auto* e = new seeml_b200_engine();
  e->device = device;
  e->mode = mode;
  e->gemm = gemm_kind;
  cudaSetDevice(device);
  for (auto& ev : e->ev) cudaEventCreate(&ev);
  cudaMalloc(&e->counter_dev, 64);
  return e;
}
void seeml_b200_engine_destroy(seeml_b200_engine* e) {
  if (!e) return;
  cudaSetDevice(e->device);
  free_dp(e->dp);
  free_loaded(e->L);
  for (auto& ev : e->ev) cudaEventDestroy(ev);
  cudaFree(e->counter_dev);
  delete e;
}
int seeml_b200_engine_load_memory(seeml_b200_engine* e, const void* plan, uint64_t size) {
  if (!e) return fail("UpdateEngine: null engine");
  return initialize(e, static_cast<const uint8_t*>(plan), size, {});
}
int seeml_b200_engine_load_file(seeml_b200_engine* e, const char* path) {
  if (!e || !path) return fail("UpdateEngine: null argument");
  std::FILE* f = std::fopen(path, "rb");
  if (!f) return fail(std::string("UpdateEngine: cannot open '") + path + "'");
  std::fseek(f, 0, SEEK_END);
  const long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<uint8_t> bytes(n > 0 ? static_cast<size_t>(n) : 0);
  const size_t got = bytes.empty() ? 0 : std::fread(bytes.data(), 1, bytes.size(), f);
  std::fclose(f);
  if (got != bytes.size()) return fail(std::string("UpdateEngine: cannot read '") + path + "'");
  const uint8_t* p = bytes.data();
  const uint64_t sz = bytes.size();
  return initialize(e, p, sz, std::move(bytes));
}

int seeml_b200_engine_header(const seeml_b200_engine* e, void* out280) {
  if (!e || !e->loaded || !out280) return fail("UpdateEngine: no plan loaded");
  std::memcpy(out280, &e->L.h, 280);
  return 0;
}
int seeml_b200_engine_loss(seeml_b200_engine* e, float* loss) {
  if (!e || !e->loaded) return fail("UpdateEngine: no plan loaded");
  return seeml_b200_read_f32(e->L.ctx, ref_off(e->L.h.loss_ref), loss);
}
uint64_t seeml_b200_engine_step(const seeml_b200_engine* e) { return e ? e->step : 0; }
void seeml_b200_engine_set_step(seeml_b200_engine* e, uint64_t s) { if (e) e->step = s; }
float seeml_b200_engine_effective_lr(const seeml_b200_engine* e) {
  return e && e->loaded ? effective_lr(e->L.h, e->step) : 0.0f;
}
int seeml_b200_engine_execute_train_once(seeml_b200_engine* e) {  // update_engine.cc:536-544
  if (!e || !e->loaded) return fail("UpdateEngine: no plan loaded");
  if (e->step == 0) e->step = 1;
  e->merged = false;
  if (int r = run_train(e)) return r;
  return seeml_b200_sync(e->L.ctx);
}
int seeml_b200_engine_arena_read(seeml_b200_engine* e, uint64_t off, void* dst, uint64_t bytes) {
  if (!e || !e->loaded) return fail("UpdateEngine: no plan loaded");
  return seeml_b200_d2h(e->L.ctx, off, dst, bytes);
}
int seeml_b200_engine_arena_write(seeml_b200_engine* e, uint64_t off, const void* src, uint64_t bytes) {
  if (!e || !e->loaded) return fail("UpdateEngine: no plan loaded");
  return seeml_b200_h2d(e->L.ctx, off, src, bytes);
}
seeml_b200_ctx* seeml_b200_engine_ctx(seeml_b200_engine* e) { return e && e->loaded ? e->L.ctx : nullptr; }
uint64_t seeml_b200_engine_opt_begin(const seeml_b200_engine* e) { return e && e->loaded ? e->L.opt_begin : 0; }
int seeml_b200_engine_run_train_range(seeml_b200_engine* e, uint64_t begin, uint64_t end) {
  if (!e || !e->loaded) return fail("UpdateEngine: no plan loaded");
  const seeml_b200_scalars sc = scalars_of(e);
  if (int r = seeml_b200_program_run(e->L.ctx, e->L.train, begin, end, &sc)) return r;
  e->last_launches = seeml_b200_program_launches(e->L.ctx, e->L.train);
  if (end > e->L.opt_begin) e->merged = false;
  return 0;
}
uint64_t seeml_b200_engine_last_launches(const seeml_b200_engine* e) { return e ? e->last_launches : 0; }
int seeml_b200_engine_enable_step_timing(seeml_b200_engine* e, int on) {
  if (!e) return fail("UpdateEngine: null engine");
  e->timing = on != 0;
  return 0;
}
int seeml_b200_engine_step_timings(const seeml_b200_engine* e, uint64_t* steps, double* fwd, double* bwd,
                                   double* opt) {
  if (!e) return fail("UpdateEngine: null engine");
  if (steps) *steps = e->t_steps;
  if (fwd) *fwd = e->t_fwd;
  if (bwd) *bwd = e->t_bwd;
  if (opt) *opt = e->t_opt;
  return 0;
}

int seeml_b200_engine_reset_step_timings(seeml_b200_engine* e) {
  if (!e) return fail("UpdateEngine: null engine");
  e->t_steps = 0;
  e->t_fwd = e->t_bwd = e->t_opt = 0;
  return 0;
}

int seeml_b200_engine_evaluate(seeml_b200_engine* e, seeml_b200_dataset* data, float* loss,
                               float* accuracy, int32_t* has_accuracy) {
  if (!e || !data) return fail("UpdateEngine: null argument");
  EvalOut o;
  if (int r = evaluate(e, *data, &o)) return r;
  if (loss) *loss = o.loss;
  if (accuracy) *accuracy = o.acc;
  if (has_accuracy) *has_accuracy = o.has_acc;
  return 0;
}

// update_engine.cc:664-787
int seeml_b200_engine_train(seeml_b200_engine* e, seeml_b200_dataset* data, uint64_t steps,
                            const seeml_b200_train_options* options, seeml_b200_train_report* report) {
  if (!e || !data) return fail("UpdateEngine: null argument");
  if (!e->loaded) return fail("UpdateEngine: no plan loaded");
  seeml_b200_train_options opt{};
  opt.log_every = 100;
  if (options) opt = *options;
  Loaded& L = e->L;
  const PlanHeader& h = L.h;
  if (steps == 0) steps = h.default_steps;
  if (steps == 0) return fail("UpdateEngine: no steps requested and the plan has no default");
  if (int r = verify_feeder(e, *data)) return r;
  if (opt.validation) if (int r = verify_feeder(e, *opt.validation)) return r;
  const bool have_ckpt = opt.checkpoint_path && opt.checkpoint_path[0];
  if (opt.resume && have_ckpt) {
    if (seeml_b200_engine_load_checkpoint(e, opt.checkpoint_path)) {
      std::fprintf(stderr, "seeml-update: no checkpoint resumed (%s)\n", seeml_b200_last_error());
    } else if (e->step > 0) {
      if (h.batch != 0 && e->step > UINT64_MAX / h.batch)
        return fail("UpdateEngine: resumed step count overflows the feeder position");
      const std::string err = data->skip_served(e->step * h.batch);
      if (!err.empty()) return fail(err);
    }
  }
  seeml_b200_train_report rep{};
  if (opt.validation) {
    EvalOut v;
    if (int r = evaluate(e, *opt.validation, &v)) return r;
    rep.has_validation = 1;
    rep.val_initial_loss = v.loss;
    rep.has_val_accuracy = v.has_acc;
    rep.val_initial_accuracy = v.acc;
  }
  const uint64_t window = std::max<uint64_t>(1, std::min<uint64_t>(20, steps / 5));
  double first_sum = 0, last_sum = 0;
  uint64_t first_n = 0, last_n = 0, executed = 0;
  const uint64_t start = e->step;
  e->merged = false;
  const uint64_t in_bytes = h.input_floats * 4, lab_bytes = h.label_kind == 0 ? 0 : h.label_bytes;
  int rc = 0;
  {
    Feeder feeder(*data, h.batch, in_bytes, lab_bytes);
    // batch s rides staging slot s%2: its H2D is issued while step s-1 computes
    int held = -1;
    auto prefetch = [&](uint64_t s) -> int {
      const uint8_t *in, *lab;
      held = feeder.acquire(&in, &lab);
      return seeml_b200_stage_h2d(L.ctx, (int)((s - start) & 1), in, in_bytes, lab, lab_bytes);
    };
    bool prefetched = false;
    for (uint64_t s = start; s < start + steps; ++s) {
      if (opt.should_stop && opt.should_stop(opt.user)) {
        rep.stopped_early = 1;
        break;
      }
      e->step = s + 1;
      const int slot = (int)((s - start) & 1);
      if (!prefetched) if ((rc = prefetch(s))) break;
      if ((rc = seeml_b200_stage_commit(L.ctx, slot, ref_off(h.input_ref), ref_off(h.label_ref)))) break;
      if ((rc = seeml_b200_stage_wait(L.ctx, slot))) break;
      feeder.consumed();
      feeder.release(held);
      held = -1;
      prefetched = false;
      if ((rc = run_train(e))) break;
      ++executed;
      if (s + 1 < start + steps) {  // overlap the next batch's copy with this step
        if ((rc = prefetch(s + 1))) break;
        prefetched = true;
      }
      float loss = 0;
      if ((rc = seeml_b200_read_f32(L.ctx, ref_off(h.loss_ref), &loss))) break;
      if (!std::isfinite(loss)) {
        rc = fail("UpdateEngine: loss became non-finite at step " + std::to_string(e->step) +
                  " — aborting the update");
        break;
      }
      if (opt.loss_curve) opt.loss_curve[s - start] = loss;
      if (s - start < window) { first_sum += loss; ++first_n; }
      if (s - start >= steps - window) { last_sum += loss; ++last_n; }
      if (opt.log_every && (s - start) % opt.log_every == 0)
        std::fprintf(stderr, "seeml-update: step %llu  loss %.6f\n", (unsigned long long)e->step, loss);
      if (opt.checkpoint_every && have_ckpt && e->step % opt.checkpoint_every == 0)
        if ((rc = seeml_b200_engine_save_checkpoint(e, opt.checkpoint_path))) break;
    }
    if (prefetched) seeml_b200_stage_wait(L.ctx, 0), seeml_b200_stage_wait(L.ctx, 1);
  }
  if (rc) return rc;
  rep.steps = executed;
  rep.initial_avg_loss = first_n ? static_cast<float>(first_sum / first_n) : 0.0f;
  rep.final_avg_loss = last_n ? static_cast<float>(last_sum / last_n) : rep.initial_avg_loss;
  if (opt.validation) {
    EvalOut v;
    if (int r = evaluate(e, *opt.validation, &v)) return r;
    rep.val_final_loss = v.loss;
    rep.val_final_accuracy = v.acc;
  }
  rep.improved = rep.has_validation ? rep.val_final_loss < rep.val_initial_loss
                                    : rep.final_avg_loss < rep.initial_avg_loss;
  if (report) *report = rep;
  return 0;
}

// ---- K-chunk data-parallel step -------------------------------------------------------------
// A global step is K executions ("chunks") of the train stream up to the first optimiser
// instruction (update_engine.cc:249-261), each on its own batch; rank r of `world` runs chunks
// [r K/world, (r+1) K/world). Every chunk's gradient operands (in[1] of the optimiser
// instructions) and its loss are packed into one set; the sets are summed in ONE fixed binary
// tree over the chunk index - the local subtree on this GPU, then an NCCL all-gather of the
// world's partial sums and the rest of the tree in rank order - scaled by 1/K, unpacked into the
// gradient slots, and every rank runs the optimiser instructions on identical bits. K and world
// are powers of two, so 1, 2, 4 and 8 GPUs give bit-identical parameters.
static bool pow2(uint64_t v) { return v && !(v & (v - 1)); }

int seeml_b200_engine_dp_configure(seeml_b200_engine* e, uint64_t chunks_per_step, int rank, int world,
                                   seeml_b200_comm* comm) {
  if (!e || !e->loaded) return fail("UpdateEngine: no plan loaded");
  if (!pow2(chunks_per_step) || world < 1 || !pow2((uint64_t)world) || (uint64_t)world > chunks_per_step)
    return fail("UpdateEngine: chunks per step and world size must be powers of two with world <= chunks");
  if (rank < 0 || rank >= world) return fail("UpdateEngine: rank out of range");
  if (world > 1 && !comm) return fail("UpdateEngine: a communicator is required when world > 1");
  if (cudaError_t ce = cudaSetDevice(e->device); ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
  free_dp(e->dp);
  DpState d;
  d.K = chunks_per_step;
  d.rank = rank;
  d.world = world;
  d.local = chunks_per_step / (uint64_t)world;
  d.comm = world > 1 ? comm : nullptr;
  if (const char* t = std::getenv("SEEML_B200_COMM_TIMEOUT_S")) d.timeout_s = std::atof(t);
  const Loaded& L = e->L;
  std::vector<k::Span> spans;
  uint64_t at = 0;
  for (const Instr& ins : L.train_instrs)
    if (ins.opcode == kSgd || ins.opcode == kAdamW) {
      spans.push_back({ref_off(ins.in[1]), ins.out[0], at});
      at += ins.out[0];
    }
  spans.push_back({ref_off(L.h.loss_ref), 1, at});      // the chunk loss rides the set as one more span
  d.fps = at + 1;
  d.nspans = spans.size();
  const uint64_t in_bytes = L.h.input_floats * 4, lab_bytes = L.h.label_kind == 0 ? 0 : L.h.label_bytes;
  bool ok = cudaMalloc(&d.sets, d.local * d.fps * sizeof(float)) == cudaSuccess &&
            cudaMalloc(&d.gathered, (uint64_t)world * d.fps * sizeof(float)) == cudaSuccess &&
            cudaMalloc(&d.spans, spans.size() * sizeof(k::Span)) == cudaSuccess &&
            cudaMemcpy(d.spans, spans.data(), spans.size() * sizeof(k::Span), cudaMemcpyHostToDevice) == cudaSuccess;
  for (int i = 0; i < 2 && ok; ++i) {
    d.pin_in[i] = static_cast<uint8_t*>(seeml_b200_pinned_alloc(in_bytes));
    d.pin_lab[i] = static_cast<uint8_t*>(seeml_b200_pinned_alloc(lab_bytes ? lab_bytes : 4));
    ok = d.pin_in[i] && d.pin_lab[i];
  }
  if (!ok) {
    cudaGetLastError();
    free_dp(d);
    return fail("UpdateEngine: data-parallel buffers could not be allocated");
  }
  e->dp = d;
  return 0;
}

namespace {

int dp_chunk(seeml_b200_engine* e, uint64_t c) {      // stream up to the optimiser, then pack set c
  Loaded& L = e->L;
  DpState& d = e->dp;
  const seeml_b200_scalars sc = scalars_of(e);
  if (int r = seeml_b200_program_run(L.ctx, L.train, 0, L.opt_begin, &sc)) return r;
  d.launches += seeml_b200_program_launches(L.ctx, L.train);
  cudaStream_t st = static_cast<cudaStream_t>(seeml_b200_ctx_stream(L.ctx));
  d.launches += k::pack_spans(static_cast<uint8_t*>(seeml_b200_ctx_arena(L.ctx)), d.spans, d.nspans, d.sets + c * d.fps,
                              0, d.fps, st);
  return 0;
}

int dp_finish(seeml_b200_engine* e, float* loss) {    // tree, exchange, optimiser
  Loaded& L = e->L;
  DpState& d = e->dp;
  cudaStream_t st = static_cast<cudaStream_t>(seeml_b200_ctx_stream(L.ctx));
  uint8_t* arena = static_cast<uint8_t*>(seeml_b200_ctx_arena(L.ctx));
  float* total = d.sets;
  const float inv_k = 1.0f / static_cast<float>(d.K);
  if (d.world > 1) {
    d.launches += k::tree_sum(d.sets, d.fps, d.local, 1.0f, st);
    if (int r = seeml_b200_comm_allgather(d.comm, d.sets, d.gathered, d.fps, st)) return r;
    d.launches += 1;
    total = d.gathered;
    d.launches += k::tree_sum(total, d.fps, (uint64_t)d.world, inv_k, st);
  } else {
    d.launches += k::tree_sum(total, d.fps, d.local, inv_k, st);
  }
  d.launches += k::pack_spans(arena, d.spans, d.nspans, total, 1, d.fps, st);
  const seeml_b200_scalars sc = scalars_of(e);
  if (int r = seeml_b200_program_run(L.ctx, L.train, L.opt_begin, L.train_instrs.size(), &sc)) return r;
  d.launches += seeml_b200_program_launches(L.ctx, L.train);
  e->merged = false;
  e->last_launches = d.launches;
  if (d.world > 1 && loss)                       // never block on a collective without a deadline
    if (int r = seeml_b200_comm_wait(d.comm, st, d.timeout_s)) return r;
  if (loss) return seeml_b200_read_f32(L.ctx, ref_off(L.h.loss_ref), loss);
  return 0;
}

}  // namespace

int seeml_b200_engine_dp_step_device(seeml_b200_engine* e, const void* inputs_device, const void* labels_device,
                                     float* loss) {
  if (!e || !e->loaded || e->dp.K == 0) return fail("UpdateEngine: data-parallel step is not configured");
  if (!inputs_device) return fail("UpdateEngine: null argument");
  Loaded& L = e->L;
  DpState& d = e->dp;
  const uint64_t in_bytes = L.h.input_floats * 4, lab_bytes = L.h.label_kind == 0 ? 0 : L.h.label_bytes;
  ++e->step;
  d.launches = 0;
  for (uint64_t c = 0; c < d.local; ++c) {
    if (int r = seeml_b200_d2d(L.ctx, ref_off(L.h.input_ref), static_cast<const uint8_t*>(inputs_device) + c * in_bytes,
                               in_bytes))
      return r;
    if (lab_bytes && labels_device)
      if (int r = seeml_b200_d2d(L.ctx, ref_off(L.h.label_ref),
                                 static_cast<const uint8_t*>(labels_device) + c * lab_bytes, lab_bytes))
        return r;
    d.launches += 2;
    if (int r = dp_chunk(e, c)) return r;
  }
  return dp_finish(e, loss);
}

int seeml_b200_engine_dp_step_host(seeml_b200_engine* e, const void* inputs, const void* labels, float* loss) {
  if (!e || !e->loaded || e->dp.K == 0) return fail("UpdateEngine: data-parallel step is not configured");
  if (!inputs) return fail("UpdateEngine: null argument");
  Loaded& L = e->L;
  DpState& d = e->dp;
  const uint64_t in_bytes = L.h.input_floats * 4, lab_bytes = L.h.label_kind == 0 ? 0 : L.h.label_bytes;
  const bool has_lab = lab_bytes && labels;
  ++e->step;
  d.launches = 0;
  auto stage = [&](uint64_t c) -> int {           // pinned staging + H2D on the copy stream
    const int s = (int)(c & 1);
    if (int r = seeml_b200_stage_wait(L.ctx, s)) return r;      // the slot's previous copy has left the pinned buffer
    std::memcpy(d.pin_in[s], static_cast<const uint8_t*>(inputs) + c * in_bytes, in_bytes);
    if (has_lab) std::memcpy(d.pin_lab[s], static_cast<const uint8_t*>(labels) + c * lab_bytes, lab_bytes);
    return seeml_b200_stage_h2d(L.ctx, s, d.pin_in[s], in_bytes, has_lab ? d.pin_lab[s] : nullptr, lab_bytes);
  };
  if (int r = stage(0)) return r;
  for (uint64_t c = 0; c < d.local; ++c) {
    const int s = (int)(c & 1);
    if (int r = seeml_b200_stage_commit(L.ctx, s, ref_off(L.h.input_ref), ref_off(L.h.label_ref))) return r;
    d.launches += 2;
    if (int r = dp_chunk(e, c)) return r;
    if (c + 1 < d.local)                          // the next chunk's copy overlaps this chunk's compute
      if (int r = stage(c + 1)) return r;
  }
  return dp_finish(e, loss);
}

uint64_t seeml_b200_engine_dp_local_chunks(const seeml_b200_engine* e) { return e ? e->dp.local : 0; }

// update_engine.cc:789-811 — the finiteness scan of the deltas runs on the device.
int seeml_b200_engine_run_merge(seeml_b200_engine* e) {
  if (!e || !e->loaded) return fail("UpdateEngine: no plan loaded");
  Loaded& L = e->L;
  const seeml_b200_scalars sc = scalars_of(e);
  if (int r = seeml_b200_program_run(L.ctx, L.merge, 0, L.h.merge_instr_count, &sc)) return r;
  cudaStream_t st = static_cast<cudaStream_t>(seeml_b200_ctx_stream(L.ctx));
  cudaMemsetAsync(e->counter_dev, 0, sizeof(unsigned long long), st);
  auto* arena = static_cast<uint8_t*>(seeml_b200_ctx_arena(L.ctx));
  for (const EmitEntry& en : L.emit)
    k::count_nonfinite(reinterpret_cast<const float*>(arena + en.arena_offset), en.byte_size / 4,
                       e->counter_dev, st);
  unsigned long long bad = 0;
  cudaMemcpyAsync(&bad, e->counter_dev, sizeof(bad), cudaMemcpyDeviceToHost, st);
  if (int r = seeml_b200_sync(L.ctx)) return r;
  if (bad)
    return fail("UpdateEngine: merged delta contains a non-finite value — the adapters are numerically "
                "poisoned; refusing to stage a commit");
  e->merged = true;
  return 0;
}

int seeml_b200_engine_verify_source_model(seeml_b200_engine* e, const char* path) {
  if (!e || !e->loaded || !path) return fail("UpdateEngine: no plan loaded");
  if (e->L.h.source_model_hash == 0) return 0;
  std::FILE* f = std::fopen(path, "rb");
  if (!f) return fail(std::string("DurableIO: cannot open '") + path + "'");
  std::fseek(f, 0, SEEK_END);
  const long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<uint8_t> bytes(n > 0 ? (size_t)n : 0);
  const size_t got = bytes.empty() ? 0 : std::fread(bytes.data(), 1, bytes.size(), f);
  std::fclose(f);
  if (got != bytes.size()) return fail(std::string("DurableIO: cannot read '") + path + "'");
  if (content_hash64(bytes.data(), bytes.size()) != e->L.h.source_model_hash)
    return fail(std::string("UpdateEngine: source model does not match the plan's source_model_hash — "
                            "refusing to run against '") + path + "'");
  return 0;
}

// update_engine.cc:826-892: lock, copy, verify the copy, patch W' = W + delta, fsync + rename.
int seeml_b200_engine_commit(seeml_b200_engine* e, const char* src, const char* dst) {
  if (!e || !e->loaded || !src || !dst) return fail("UpdateEngine: no plan loaded");
  if (!e->merged) return fail("UpdateEngine: RunMerge() must precede commit");
  Loaded& L = e->L;
  const std::string lock_path = std::string(dst) + ".lock";
  const int lock_fd = ::open(lock_path.c_str(), O_RDWR | O_CREAT, 0644);
  if (lock_fd < 0) return fail("DurableIO: cannot open commit lock '" + lock_path + "'");
  if (::flock(lock_fd, LOCK_EX) != 0) {
    ::close(lock_fd);
    return fail("DurableIO: cannot take commit lock '" + lock_path + "'");
  }
  int rc = 0;
  std::vector<uint8_t> bytes;
  {
    std::FILE* f = std::fopen(src, "rb");
    if (!f) rc = fail(std::string("DurableIO: cannot open '") + src + "'");
    if (!rc) {
      std::fseek(f, 0, SEEK_END);
      const long n = std::ftell(f);
      std::fseek(f, 0, SEEK_SET);
      bytes.resize(n > 0 ? (size_t)n : 0);
      if (!bytes.empty() && std::fread(bytes.data(), 1, bytes.size(), f) != bytes.size())
        rc = fail(std::string("DurableIO: cannot read '") + src + "'");
      std::fclose(f);
    }
  }
  if (!rc && L.h.source_model_hash != 0 &&
      content_hash64(bytes.data(), bytes.size()) != L.h.source_model_hash)
    rc = fail(std::string("UpdateEngine: source model does not match the plan's source_model_hash — "
                          "refusing to patch '") + src + "'");
  std::vector<float> delta;
  for (size_t i = 0; !rc && i < L.emit.size(); ++i) {
    const EmitEntry& en = L.emit[i];
    if (en.smf_data_offset > bytes.size() || en.byte_size > bytes.size() - en.smf_data_offset ||
        en.byte_size % 4 != 0) {
      rc = fail("UpdateEngine: emit entry exceeds the source model file — plan and model are out of sync");
      break;
    }
    delta.resize(en.byte_size / 4);
    rc = seeml_b200_d2h(L.ctx, en.arena_offset, delta.data(), en.byte_size);
    if (rc) break;
    for (size_t j = 0; j < delta.size(); ++j) {
      float w;
      std::memcpy(&w, bytes.data() + en.smf_data_offset + j * 4, 4);
      w += delta[j];
      std::memcpy(bytes.data() + en.smf_data_offset + j * 4, &w, 4);
    }
  }
  if (!rc) rc = write_file_durable(dst, bytes.data(), bytes.size(), nullptr, 0);
  ::flock(lock_fd, LOCK_UN);
  ::close(lock_fd);
  return rc;
}

int seeml_b200_engine_save_checkpoint(seeml_b200_engine* e, const char* path) {
  if (!e || !e->loaded || !path) return fail("UpdateEngine: no plan loaded");
  std::vector<uint8_t> persistent(e->L.h.persistent_size);
  if (int r = seeml_b200_d2h(e->L.ctx, 0, persistent.data(), persistent.size())) return r;
  CkptHeader h;
  h.plan_hash = e->L.h.plan_hash;
  h.step = e->step;
  h.persistent_size = persistent.size();
  h.payload_hash = content_hash64(persistent.data(), persistent.size());
  return write_file_durable(path, &h, sizeof(h), persistent.data(), persistent.size());
}
int seeml_b200_engine_load_checkpoint(seeml_b200_engine* e, const char* path) {
  if (!e || !e->loaded || !path) return fail("UpdateEngine: no plan loaded");
  std::FILE* f = std::fopen(path, "rb");
  if (!f) return fail(std::string("Checkpoint: no checkpoint at '") + path + "'");
  CkptHeader h;
  const bool ok = std::fread(&h, sizeof(h), 1, f) == 1;
  if (!ok || h.magic != 0x504B4553 || h.version != 3) {
    std::fclose(f);
    return fail(std::string("Checkpoint: not a v3 checkpoint: '") + path + "'");
  }
  if (h.plan_hash != e->L.h.plan_hash) {
    std::fclose(f);
    return fail("Checkpoint: checkpoint belongs to a different plan");
  }
  if (h.persistent_size != e->L.h.persistent_size) {
    std::fclose(f);
    return fail("Checkpoint: checkpoint incompatible with plan");
  }
  std::vector<uint8_t> payload(h.persistent_size);
  const bool got = payload.empty() || std::fread(payload.data(), 1, payload.size(), f) == payload.size();
  std::fclose(f);
  if (!got) return fail("Checkpoint: truncated checkpoint");
  if (content_hash64(payload.data(), payload.size()) != h.payload_hash)
    return fail("Checkpoint: checkpoint payload is corrupt");
  if (int r = seeml_b200_h2d(e->L.ctx, 0, payload.data(), payload.size())) return r;
  e->step = h.step;
  e->merged = false;
  return 0;
}

}  // extern "C"

// seeml::update_rt::Dataset over the seeml_b200 C ABI: the reference's public interface
// (runtime/feeder/dataset.h:43-152), same method names, argument meaning and error
// strings, so a program written against the reference's header compiles and links
// against libseeml_b200.so unchanged. Header-only; move-only (the reference's class
// is movable too, it sits inside std::expected / std::optional in the generated driver).
#ifndef SEEML_COMPAT_RUNTIME_FEEDER_DATASET_H_
#define SEEML_COMPAT_RUNTIME_FEEDER_DATASET_H_

#include <cstdint>
#include <expected>
#include <string>
#include <utility>
#include <vector>

#include "seeml_b200.h"

namespace seeml::update_rt {

inline constexpr uint32_t kSdsMagic = 0x31534453;  // "SDS1"

class Dataset {
 public:
  [[nodiscard]] static std::expected<Dataset, std::string> LoadFromFile(const std::string& path) {
    return Wrap(seeml_b200_dataset_load(path.c_str()));
  }
  [[nodiscard]] static std::expected<Dataset, std::string> FromMemory(std::vector<float> inputs,
                                                                      std::vector<uint8_t> labels,
                                                                      uint64_t num_samples, uint64_t input_dim,
                                                                      uint32_t label_kind, uint64_t label_dim) {
    if (inputs.size() != num_samples * input_dim) return std::unexpected("Dataset: input size mismatch");
    return Wrap(seeml_b200_dataset_from_memory(inputs.data(), labels.empty() ? nullptr : labels.data(), num_samples,
                                               input_dim, label_kind, label_dim));
  }
  [[nodiscard]] static std::expected<Dataset, std::string> FromTokens(std::vector<int32_t> tokens,
                                                                      uint64_t num_records, uint64_t seq) {
    if (tokens.size() != num_records * (seq + 1)) return std::unexpected("Dataset: token store size mismatch");
    return Wrap(seeml_b200_dataset_from_tokens(tokens.data(), num_records, seq));
  }

  Dataset(Dataset&& o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
  Dataset& operator=(Dataset&& o) noexcept {
    if (this != &o) {
      seeml_b200_dataset_free(h_);
      h_ = std::exchange(o.h_, nullptr);
    }
    return *this;
  }
  Dataset(const Dataset&) = delete;
  Dataset& operator=(const Dataset&) = delete;
  ~Dataset() { seeml_b200_dataset_free(h_); }

  uint64_t num_samples() const { return seeml_b200_dataset_num_samples(h_); }
  uint64_t input_dim() const { return seeml_b200_dataset_input_dim(h_); }
  uint32_t label_kind() const { return seeml_b200_dataset_label_kind(h_); }
  uint32_t input_kind() const { return seeml_b200_dataset_input_kind(h_); }
  uint64_t label_bytes_per_sample() const { return seeml_b200_dataset_label_bytes_per_sample(h_); }

  [[nodiscard]] std::expected<void, std::string> ValidateClassLabels(uint64_t num_classes) const {
    return Status(seeml_b200_dataset_validate_labels(h_, num_classes));
  }
  void FillBatch(uint64_t batch, float* input_slot, uint8_t* label_slot) {
    seeml_b200_dataset_fill_batch(h_, batch, input_slot, label_slot);
  }
  void Rewind() { seeml_b200_dataset_rewind(h_); }
  void EnableShuffle(uint64_t seed) { seeml_b200_dataset_enable_shuffle(h_, seed); }

  struct ServingPos {
    uint64_t cursor = 0;
    uint64_t epoch = 0;
  };
  ServingPos SaveServingPos() const {
    ServingPos p;
    seeml_b200_dataset_save_pos(h_, &p.cursor, &p.epoch);
    return p;
  }
  void RestoreServingPos(ServingPos pos) { seeml_b200_dataset_restore_pos(h_, pos.cursor, pos.epoch); }

  [[nodiscard]] std::expected<void, std::string> SkipServed(uint64_t rows) {
    return Status(seeml_b200_dataset_skip_served(h_, rows));
  }
  [[nodiscard]] std::expected<Dataset, std::string> SplitValidation(double fraction) {
    return Wrap(seeml_b200_dataset_split_validation(h_, fraction));
  }
  [[nodiscard]] std::expected<void, std::string> SaveToFile(const std::string& path) const {
    return Status(seeml_b200_dataset_save(h_, path.c_str()));
  }

  /// The C handle (for UpdateEngine; not part of the reference's interface).
  seeml_b200_dataset* handle() const { return h_; }

 private:
  explicit Dataset(seeml_b200_dataset* h) : h_(h) {}
  static std::expected<Dataset, std::string> Wrap(seeml_b200_dataset* h) {
    if (!h) return std::unexpected(std::string(seeml_b200_last_error()));
    return Dataset(h);
  }
  static std::expected<void, std::string> Status(int rc) {
    if (rc != 0) return std::unexpected(std::string(seeml_b200_last_error()));
    return {};
  }
  seeml_b200_dataset* h_ = nullptr;
};

}  // namespace seeml::update_rt

#endif  // SEEML_COMPAT_RUNTIME_FEEDER_DATASET_H_

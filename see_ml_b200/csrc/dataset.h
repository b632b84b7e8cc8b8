// SDS corpora and batch serving on the host. Serving order (sequential with
// wraparound, or a seeded per-epoch Fisher-Yates permutation driven by SplitMix64),
// the tail validation split and the token -> (inputs, shifted labels) view are
// bit-exact restatements of the reference feeder (runtime/feeder/dataset.cc:86-462):
// the same corpus, seed and call sequence produce the same bytes in the I/O slots.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

struct seeml_b200_dataset {
  std::vector<float> inputs;      // samples * input_dim            (input_kind 0)
  std::vector<uint8_t> labels;    // samples * label_bytes_per_sample
  std::vector<int32_t> tokens;    // samples * (input_dim + 1)      (input_kind 1)
  uint64_t samples = 0, input_dim = 0, label_dim = 0;
  uint32_t label_kind = 0, input_kind = 0;
  uint64_t cursor = 0;
  std::vector<uint64_t> order;    // empty = sequential serving
  uint64_t shuffle_state = 0, shuffle_origin = 0, epoch = 0;

  struct Pos { uint64_t cursor, epoch; };
  uint64_t label_bytes_per_sample() const;
  void fill_batch(uint64_t batch, void* input_slot, void* label_slot);
  void enable_shuffle(uint64_t seed);
  void reshuffle();
  Pos save_pos() const { return {cursor, epoch}; }
  void restore_pos(Pos p);
  std::string skip_served(uint64_t rows);
  std::string validate_labels(uint64_t num_classes) const;
  std::string split_validation(double fraction, seeml_b200_dataset* out);
  std::string save(const std::string& path) const;
  static std::string load(const std::string& path, seeml_b200_dataset* out);
};

#include "dataset.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <memory>

#include "backend.h"

namespace {

constexpr uint32_t kSdsMagic = 0x31534453;  // "SDS1"
constexpr uint64_t kHeaderBytes = 40;

bool mul_u64(uint64_t a, uint64_t b, uint64_t* out) {
  if (b != 0 && a > UINT64_MAX / b) return false;
  *out = a * b;
  return true;
}
uint64_t splitmix64(uint64_t* s) {
  uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
struct File {
  std::FILE* f = nullptr;
  ~File() { if (f) std::fclose(f); }
};

}  // namespace

uint64_t seeml_b200_dataset::label_bytes_per_sample() const {
  if (input_kind == 1) return input_dim * 4;  // one derived next-token id per position
  return label_kind == 1 ? 4 : label_kind == 2 ? label_dim * 4 : 0;
}

// dataset.cc:86-203 — header, bounds against the real file size, then the payload.
std::string seeml_b200_dataset::load(const std::string& path, seeml_b200_dataset* out) {
  File fh;
  fh.f = std::fopen(path.c_str(), "rb");
  if (!fh.f) return "Dataset: cannot open '" + path + "'";
  std::fseek(fh.f, 0, SEEK_END);
  const long end = std::ftell(fh.f);
  if (end < 0) return "Dataset: cannot stat '" + path + "'";
  const uint64_t file_size = static_cast<uint64_t>(end);
  std::fseek(fh.f, 0, SEEK_SET);
  uint8_t hdr[kHeaderBytes];
  if (file_size < 4 || std::fread(hdr, 1, 4, fh.f) != 4) return "Dataset: bad magic in '" + path + "'";
  uint32_t magic;
  std::memcpy(&magic, hdr, 4);
  if (magic != kSdsMagic) return "Dataset: bad magic in '" + path + "'";
  uint32_t version = 0;
  if (std::fread(&version, 1, 4, fh.f) != 4 || version < 1 || version > 2)
    return "Dataset: unsupported version";
  if (std::fread(hdr, 1, 32, fh.f) != 32) return "Dataset: truncated header";
  seeml_b200_dataset d;
  std::memcpy(&d.samples, hdr, 8);
  std::memcpy(&d.input_dim, hdr + 8, 8);
  std::memcpy(&d.label_kind, hdr + 16, 4);
  std::memcpy(&d.input_kind, hdr + 20, 4);
  std::memcpy(&d.label_dim, hdr + 24, 8);
  if (d.samples == 0 || d.input_dim == 0) return "Dataset: empty dataset";
  if (d.label_kind > 2) return "Dataset: unknown label kind";
  if (d.label_kind == 2 && (d.label_dim == 0 || d.label_dim > UINT64_MAX / 4))
    return "Dataset: label dim out of range";
  if (d.input_kind > 1 || (version < 2 && d.input_kind != 0)) return "Dataset: unknown input kind";
  if (d.input_kind == 1) {
    if (d.label_kind != 1 || d.label_dim != 0)
      return "Dataset: token corpora derive next-token class labels (label_kind 1, label_dim 0)";
    uint64_t rec = 0, payload = 0;
    if (d.input_dim >= UINT64_MAX || !mul_u64(d.input_dim + 1, 4, &rec) ||
        !mul_u64(d.samples, rec, &payload) || payload > file_size - kHeaderBytes)
      return "Dataset: sample section exceeds file size";
    d.tokens.resize(d.samples * (d.input_dim + 1));
    if (std::fread(d.tokens.data(), 1, payload, fh.f) != payload) return "Dataset: truncated inputs";
    for (int32_t t : d.tokens)
      if (t < 0) return "Dataset: negative token id";
    *out = std::move(d);
    return {};
  }
  const uint64_t lb = d.label_bytes_per_sample();
  uint64_t in_bytes = 0, payload = 0;
  if (!mul_u64(d.input_dim, 4, &in_bytes) || in_bytes > UINT64_MAX - lb ||
      !mul_u64(d.samples, in_bytes + lb, &payload) || payload > file_size - kHeaderBytes)
    return "Dataset: sample section exceeds file size";
  d.inputs.resize(d.samples * d.input_dim);
  d.labels.resize(d.samples * lb);
  if (lb == 0) {
    if (std::fread(d.inputs.data(), 1, d.samples * in_bytes, fh.f) != d.samples * in_bytes)
      return "Dataset: truncated inputs";
  } else {
    // records interleave input and label: read whole records in bounded chunks
    const uint64_t rec = in_bytes + lb;
    const uint64_t per = std::max<uint64_t>(1, (256 * 1024) / rec);
    std::vector<uint8_t> buf(per * rec);
    for (uint64_t i = 0; i < d.samples;) {
      const uint64_t n = std::min(per, d.samples - i);
      if (std::fread(buf.data(), 1, n * rec, fh.f) != n * rec) return "Dataset: truncated inputs";
      for (uint64_t s = 0; s < n; ++s) {
        std::memcpy(d.inputs.data() + (i + s) * d.input_dim, buf.data() + s * rec, in_bytes);
        std::memcpy(d.labels.data() + (i + s) * lb, buf.data() + s * rec + in_bytes, lb);
      }
      i += n;
    }
  }
  *out = std::move(d);
  return {};
}

std::string seeml_b200_dataset::save(const std::string& path) const {
  File fh;
  fh.f = std::fopen(path.c_str(), "wb");
  if (!fh.f) return "Dataset: cannot write '" + path + "'";
  const uint32_t version = input_kind == 1 ? 2 : 1;
  bool ok = std::fwrite(&kSdsMagic, 4, 1, fh.f) == 1 && std::fwrite(&version, 4, 1, fh.f) == 1 &&
            std::fwrite(&samples, 8, 1, fh.f) == 1 && std::fwrite(&input_dim, 8, 1, fh.f) == 1 &&
            std::fwrite(&label_kind, 4, 1, fh.f) == 1 && std::fwrite(&input_kind, 4, 1, fh.f) == 1 &&
            std::fwrite(&label_dim, 8, 1, fh.f) == 1;
  if (input_kind == 1) {
    ok = ok && std::fwrite(tokens.data(), 4, tokens.size(), fh.f) == tokens.size();
  } else {
    const uint64_t lb = label_bytes_per_sample(), in_bytes = input_dim * 4;
    for (uint64_t i = 0; ok && i < samples; ++i) {
      ok = std::fwrite(inputs.data() + i * input_dim, 1, in_bytes, fh.f) == in_bytes;
      if (ok && lb) ok = std::fwrite(labels.data() + i * lb, 1, lb, fh.f) == lb;
    }
  }
  const int rc = std::fclose(fh.f);
  fh.f = nullptr;
  if (!ok || rc != 0) return "Dataset: short write to '" + path + "'";
  return {};
}

std::string seeml_b200_dataset::validate_labels(uint64_t num_classes) const {
  if (label_kind != 1 || num_classes == 0) return {};
  if (input_kind == 1) {
    for (uint64_t i = 0; i < tokens.size(); ++i)
      if (tokens[i] < 0 || static_cast<uint64_t>(tokens[i]) >= num_classes)
        return "Dataset: token id " + std::to_string(tokens[i]) + " at position " + std::to_string(i) +
               " outside [0, " + std::to_string(num_classes) + ")";
    return {};
  }
  const auto* lab = reinterpret_cast<const int32_t*>(labels.data());
  for (uint64_t i = 0; i < samples; ++i)
    if (lab[i] < 0 || static_cast<uint64_t>(lab[i]) >= num_classes)
      return "Dataset: class label " + std::to_string(lab[i]) + " at sample " + std::to_string(i) +
             " outside [0, " + std::to_string(num_classes) + ")";
  return {};
}

// dataset.cc:288-349. `batch` counts rows; a token corpus serves batch/input_dim records.
void seeml_b200_dataset::fill_batch(uint64_t batch, void* input_slot, void* label_slot) {
  auto advance = [&] {
    if (++cursor == samples) {
      cursor = 0;
      if (!order.empty()) {
        reshuffle();  // a fresh permutation every epoch
        ++epoch;
      }
    }
  };
  if (input_kind == 1) {
    const uint64_t S = input_dim, records = batch / S;
    auto* in = static_cast<int32_t*>(input_slot);
    auto* lab = static_cast<int32_t*>(label_slot);
    for (uint64_t r = 0; r < records; ++r) {
      const uint64_t i = order.empty() ? cursor : order[cursor];
      const int32_t* rec = tokens.data() + i * (S + 1);
      std::memcpy(in + r * S, rec, S * 4);
      if (lab) std::memcpy(lab + r * S, rec + 1, S * 4);  // labels = the view shifted by one
      advance();
    }
    return;
  }
  const uint64_t lb = label_bytes_per_sample();
  auto* in = static_cast<float*>(input_slot);
  auto* lab = static_cast<uint8_t*>(label_slot);
  for (uint64_t b = 0; b < batch; ++b) {
    const uint64_t i = order.empty() ? cursor : order[cursor];
    std::memcpy(in + b * input_dim, inputs.data() + i * input_dim, input_dim * 4);
    if (lab && lb) std::memcpy(lab + b * lb, labels.data() + i * lb, lb);
    advance();
  }
}

void seeml_b200_dataset::reshuffle() {  // dataset.cc:410-417
  for (uint64_t i = 0; i < samples; ++i) order[i] = i;
  for (uint64_t i = samples - 1; i > 0; --i) {
    const uint64_t j = splitmix64(&shuffle_state) % (i + 1);
    std::swap(order[i], order[j]);
  }
}
void seeml_b200_dataset::enable_shuffle(uint64_t seed) {  // dataset.cc:365-375
  shuffle_state = seed;
  shuffle_state = splitmix64(&shuffle_state) | 1ull;
  shuffle_origin = shuffle_state;
  epoch = 0;
  order.resize(samples);
  reshuffle();
  cursor = 0;
}
void seeml_b200_dataset::restore_pos(Pos p) {  // dataset.cc:377-391
  cursor = p.cursor;
  if (order.empty() || epoch == p.epoch) return;
  shuffle_state = shuffle_origin;
  epoch = 0;
  reshuffle();
  while (epoch < p.epoch) {
    reshuffle();
    ++epoch;
  }
}
std::string seeml_b200_dataset::skip_served(uint64_t rows) {  // dataset.cc:393-408
  uint64_t records = rows;
  if (input_kind == 1) {
    if (rows % input_dim != 0)
      return "Dataset: served rows are not a whole number of token records — cannot replay the "
             "serving position";
    records = rows / input_dim;
  }
  restore_pos({records % samples, records / samples});
  return {};
}
std::string seeml_b200_dataset::split_validation(double fraction, seeml_b200_dataset* out) {
  if (!(fraction > 0.0) || fraction >= 1.0) return "Dataset: validation fraction must be in (0, 1)";
  if (samples < 2) return "Dataset: too few samples to split";
  if (!order.empty()) return "Dataset: split before enabling shuffle";
  uint64_t val_n = static_cast<uint64_t>(static_cast<double>(samples) * fraction);
  if (val_n == 0) val_n = 1;
  if (val_n >= samples) val_n = samples - 1;
  const uint64_t train_n = samples - val_n;
  seeml_b200_dataset v;
  v.samples = val_n;
  v.input_dim = input_dim;
  v.label_kind = label_kind;
  v.label_dim = label_dim;
  v.input_kind = input_kind;
  if (input_kind == 1) {
    const uint64_t rec = input_dim + 1;
    v.tokens.assign(tokens.begin() + static_cast<ptrdiff_t>(train_n * rec), tokens.end());
    tokens.resize(train_n * rec);
  } else {
    const uint64_t lb = label_bytes_per_sample();
    v.inputs.assign(inputs.begin() + static_cast<ptrdiff_t>(train_n * input_dim), inputs.end());
    v.labels.assign(labels.begin() + static_cast<ptrdiff_t>(train_n * lb), labels.end());
    inputs.resize(train_n * input_dim);
    labels.resize(train_n * lb);
  }
  samples = train_n;
  cursor = 0;
  *out = std::move(v);
  return {};
}

using seeml_b200::fail;
extern "C" {

seeml_b200_dataset* seeml_b200_dataset_load(const char* path) {
  auto d = std::make_unique<seeml_b200_dataset>();
  const std::string err = seeml_b200_dataset::load(path ? path : "", d.get());
  if (!err.empty()) {
    fail(err);
    return nullptr;
  }
  return d.release();
}
seeml_b200_dataset* seeml_b200_dataset_from_tokens(const int32_t* tokens, uint64_t records, uint64_t seq) {
  if (records == 0) { fail("Dataset: zero samples"); return nullptr; }
  if (seq == 0) { fail("Dataset: zero input dim"); return nullptr; }
  uint64_t want = 0;
  if (!tokens || seq >= UINT64_MAX || !mul_u64(records, seq + 1, &want)) {
    fail("Dataset: token buffer size mismatch");
    return nullptr;
  }
  for (uint64_t i = 0; i < want; ++i)
    if (tokens[i] < 0) {
      fail("Dataset: negative token id at position " + std::to_string(i));
      return nullptr;
    }
  auto d = std::make_unique<seeml_b200_dataset>();
  d->input_kind = 1;
  d->label_kind = 1;
  d->samples = records;
  d->input_dim = seq;
  d->tokens.assign(tokens, tokens + want);
  return d.release();
}
seeml_b200_dataset* seeml_b200_dataset_from_memory(const float* inputs, const void* labels,
                                                   uint64_t samples, uint64_t input_dim,
                                                   uint32_t label_kind, uint64_t label_dim) {
  if (samples == 0) { fail("Dataset: zero samples"); return nullptr; }
  if (input_dim == 0) { fail("Dataset: zero input dim"); return nullptr; }
  if (label_kind > 2) { fail("Dataset: unknown label kind"); return nullptr; }
  if (label_kind == 2 && (label_dim == 0 || label_dim > UINT64_MAX / 4)) {
    fail("Dataset: label dim out of range");
    return nullptr;
  }
  uint64_t want = 0;
  if (!inputs || !mul_u64(samples, input_dim, &want)) {
    fail("Dataset: input buffer size mismatch");
    return nullptr;
  }
  auto d = std::make_unique<seeml_b200_dataset>();
  d->samples = samples;
  d->input_dim = input_dim;
  d->label_kind = label_kind;
  d->label_dim = label_dim;
  d->inputs.assign(inputs, inputs + want);
  const uint64_t lb = d->label_bytes_per_sample();
  if (lb) {
    if (!labels) { fail("Dataset: label buffer size mismatch"); return nullptr; }
    const auto* p = static_cast<const uint8_t*>(labels);
    d->labels.assign(p, p + samples * lb);
  }
  return d.release();
}
void seeml_b200_dataset_free(seeml_b200_dataset* d) { delete d; }
uint64_t seeml_b200_dataset_num_samples(const seeml_b200_dataset* d) { return d ? d->samples : 0; }
uint64_t seeml_b200_dataset_input_dim(const seeml_b200_dataset* d) { return d ? d->input_dim : 0; }
uint32_t seeml_b200_dataset_label_kind(const seeml_b200_dataset* d) { return d ? d->label_kind : 0; }
uint32_t seeml_b200_dataset_input_kind(const seeml_b200_dataset* d) { return d ? d->input_kind : 0; }
void seeml_b200_dataset_enable_shuffle(seeml_b200_dataset* d, uint64_t seed) { if (d) d->enable_shuffle(seed); }
void seeml_b200_dataset_rewind(seeml_b200_dataset* d) { if (d) d->cursor = 0; }
seeml_b200_dataset* seeml_b200_dataset_split_validation(seeml_b200_dataset* d, double fraction) {
  if (!d) { fail("Dataset: null dataset"); return nullptr; }
  auto v = std::make_unique<seeml_b200_dataset>();
  const std::string err = d->split_validation(fraction, v.get());
  if (!err.empty()) { fail(err); return nullptr; }
  return v.release();
}
void seeml_b200_dataset_fill_batch(seeml_b200_dataset* d, uint64_t batch, void* input_slot,
                                   void* label_slot) {
  if (d) d->fill_batch(batch, input_slot, label_slot);
}
int seeml_b200_dataset_skip_served(seeml_b200_dataset* d, uint64_t rows) {
  if (!d) return fail("Dataset: null dataset");
  const std::string err = d->skip_served(rows);
  return err.empty() ? 0 : fail(err);
}
int seeml_b200_dataset_validate_labels(const seeml_b200_dataset* d, uint64_t num_classes) {
  if (!d) return fail("Dataset: null dataset");
  const std::string err = d->validate_labels(num_classes);
  return err.empty() ? 0 : fail(err);
}
int seeml_b200_dataset_save(const seeml_b200_dataset* d, const char* path) {
  if (!d || !path) return fail("Dataset: null argument");
  const std::string err = d->save(path);
  return err.empty() ? 0 : fail(err);
}

/* Dataset::label_bytes_per_sample, SaveServingPos / RestoreServingPos (dataset.h:57, 93-106). */
uint64_t seeml_b200_dataset_label_bytes_per_sample(const seeml_b200_dataset* d) {
  return d ? d->label_bytes_per_sample() : 0;
}
void seeml_b200_dataset_save_pos(const seeml_b200_dataset* d, uint64_t* cursor, uint64_t* epoch) {
  if (!d) return;
  const seeml_b200_dataset::Pos p = d->save_pos();
  if (cursor) *cursor = p.cursor;
  if (epoch) *epoch = p.epoch;
}
void seeml_b200_dataset_restore_pos(seeml_b200_dataset* d, uint64_t cursor, uint64_t epoch) {
  if (d) d->restore_pos({cursor, epoch});
}

}  // extern "C"

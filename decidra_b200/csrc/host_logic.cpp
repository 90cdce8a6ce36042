// Host-side integer logic of the state-once path. Plain C++, no CUDA.
#include "host_logic.h"

#include <algorithm>
#include <cmath>
#include <numeric>
#include <vector>

#include "../../include/decidra_b200.h"

// Engine::state_once_batch_rows chunking (native/src/engine.rs:4893-4918 in juanqui/decidra):
// indices are stably sorted by question length, then appended greedily; a chunk is closed when
// adding the next question would exceed rows, rows*(state+maxlen) keys or
// rows*maxlen*(state+maxlen) scores. The extra max_tokens cap (sum of lengths) bounds the
// workspace of this implementation.
int plan_chunks_host(const size_t* lens, size_t B, size_t state_len, size_t max_rows, size_t max_keys, size_t max_scores,
                     size_t max_tokens, int32_t* order, int32_t* chunk_of, int32_t* n_chunks) {
  if (B == 0) return -3;
  std::vector<size_t> ord(B);
  std::iota(ord.begin(), ord.end(), (size_t)0);
  std::stable_sort(ord.begin(), ord.end(), [&](size_t a, size_t b) { return lens[a] < lens[b]; });
  int chunks = 0;
  size_t cur = 0, max_q = 0, tokens = 0;
  for (size_t n = 0; n < B; ++n) {
    const size_t index = ord[n], len = lens[index];
    const size_t next_max = std::max(max_q, len);
    const size_t rows = cur + 1;
    const unsigned __int128 keys = (unsigned __int128)rows * (state_len + next_max);
    const unsigned __int128 scores = keys * next_max;
    const bool over_tokens = max_tokens != 0 && tokens + len > max_tokens;
    if (rows == 1 && (keys > max_keys || scores > max_scores || (max_tokens != 0 && len > max_tokens))) return -5;
    if (cur != 0 && (rows > max_rows || keys > max_keys || scores > max_scores || over_tokens)) {
      ++chunks;
      cur = 0;
      max_q = 0;
      tokens = 0;
      if (max_tokens != 0 && len > max_tokens) return -5;
    }
    order[n] = (int32_t)index;
    chunk_of[index] = chunks;
    ++cur;
    tokens += len;
    max_q = std::max(max_q, len);
  }
  *n_chunks = chunks + 1;
  return 0;
}

extern "C" {

int dcd_plan_chunks(const size_t* lens, size_t B, size_t state_len, size_t max_rows, size_t max_keys, size_t max_scores,
                    int32_t* order, int32_t* chunk_of, int32_t* n_chunks) {
  if (!lens || !order || !chunk_of || !n_chunks) return DCD_E_INVALID;
  if (max_rows == 0 || max_keys == 0 || max_scores == 0) return DCD_E_INVALID;  // "state-once caps must be positive"
  return plan_chunks_host(lens, B, state_len, max_rows, max_keys, max_scores, 0, order, chunk_of, n_chunks) == 0 ? DCD_OK : DCD_E_INVALID;
}

// block_cascade_mask, native/src/engine.rs:490-504.
int dcd_block_cascade_mask(size_t seq, size_t split, uint8_t* mask) {
  if (!mask || split == 0 || split >= seq) return DCD_E_INVALID;
  for (size_t q = 0; q < seq; ++q) {
    const size_t end = q < split ? split : seq;
    for (size_t k = 0; k < end; ++k) {
      const size_t bit = q * seq + k;
      mask[bit >> 3] |= (uint8_t)(1u << (bit & 7));
    }
  }
  return DCD_OK;
}

// NativeBackend::answers probabilities (src/native_backend.rs:611-619) followed by d3::to_answer
// (src/d3.rs:373-438), choice_confidence (:443-453) and score_confidence (:457-478). All sums
// run left to right in f32 like the iterator sums they replace.
int dcd_decode_answer(const float* logits, int count, float temperature, int kind, float* shares, float* out2) {
  if (!logits || !shares || !out2 || count <= 0 || kind < 0 || kind > 2) return DCD_E_INVALID;
  if (kind == 1 && count < 2) return DCD_E_INVALID;
  std::vector<float> p((size_t)count);
  float total = 0.f;
  for (int i = 0; i < count; ++i) {
    p[i] = expf(logits[i] / temperature);
    total += p[i];
  }
  if (!std::isfinite(total) || total <= 0.f) return DCD_E_INVALID;  // "non-finite d3 logits"
  for (int i = 0; i < count; ++i) p[i] = p[i] / total;
  float t2 = 0.f;
  for (int i = 0; i < count; ++i) t2 += p[i];
  if (!std::isfinite(t2) || t2 <= 0.f) return DCD_E_INVALID;
  for (int i = 0; i < count; ++i) {
    if (!std::isfinite(p[i]) || p[i] < 0.f) return DCD_E_INVALID;
    shares[i] = p[i] / t2;
  }
  out2[0] = 0.f;
  out2[1] = 0.f;
  if (kind == 2) {
    float score = 0.f;
    for (int i = 0; i < count; ++i) score += (float)i * shares[i];
    float conf = 1.0f;
    if (count > 1) {
      int mode = 0;
      for (int l = 1; l < count; ++l)
        if (shares[l] > shares[mode]) mode = l;
      float spread = 0.f;
      for (int l = 0; l < count; ++l) spread += shares[l] * fabsf((float)l - (float)mode);
      float even = 0.f;
      for (int l = 0; l < count; ++l) even += fabsf((float)l - (float)(count - 1) / 2.0f);
      even /= (float)count;
      conf = std::min(std::max(1.0f - spread / even, 0.0f), 1.0f);
    }
    out2[0] = score;
    out2[1] = conf;
    return DCD_OK;
  }
  if (kind == 1) {
    out2[0] = shares[1];
    return DCD_OK;
  }
  int best = 0;
  for (int i = 1; i < count; ++i)
    if (shares[i] > shares[best]) best = i;
  float conf = 1.0f;
  if (count > 1) {
    float top = -INFINITY;
    for (int i = 0; i < count; ++i) top = std::max(top, shares[i]);
    conf = (top - 1.0f / (float)count) / (1.0f - 1.0f / (float)count);
    conf = std::min(std::max(conf, 0.0f), 1.0f);
  }
  out2[0] = (float)best;
  out2[1] = conf;
  return DCD_OK;
}

}  // extern "C"

// Host-side integer logic of the path (bit-exact parts): chunk planner, block-cascade mask,
// answer decoding.
#pragma once
#include <stddef.h>
#include <stdint.h>

// Greedy chunk planner. Returns 0, -3 (empty) or -5 (one question alone exceeds a cap).
// max_tokens == 0 disables the workspace-row cap (the reference has none).
int plan_chunks_host(const size_t* lens, size_t B, size_t state_len, size_t max_rows, size_t max_keys, size_t max_scores,
                     size_t max_tokens, int32_t* order, int32_t* chunk_of, int32_t* n_chunks);

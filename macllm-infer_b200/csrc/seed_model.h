// Seed-model tensor generator (see seed_model.cpp).
#pragma once
#include <cstdint>

namespace mk {
int64_t seed_row_bytes(int type, int64_t cols);
void seed_tensor(uint64_t seed, uint64_t stream, float std_dev, int type, int64_t rows, int64_t cols, void* out);
}  // namespace mk

// Host sampler pieces that stay on the CPU: penalties and the first-index argmax
// (src/sampling.rs:392-433 of the reference).
#pragma once
#include <cstdint>
#include <cstring>
#include <cmath>
#include <vector>
#include <algorithm>

namespace mk {

inline int32_t float_total_key(float f) {
    int32_t b;
    memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

inline int64_t argmax_first(const float* v, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; ++i)
        if (float_total_key(v[i]) > float_total_key(v[best])) best = i;
    return best;
}

inline void apply_penalties(float* logits, int64_t vocab, const uint32_t* history, int64_t nh, float rep, const uint32_t* generated,
                            int64_t ng, float presence, float frequency) {
    if (rep > 0.f && std::fabs(rep - 1.0f) >= 1.1920929e-07f && nh > 0) {
        std::vector<uint32_t> seen(history, history + nh);
        std::sort(seen.begin(), seen.end());
        seen.erase(std::unique(seen.begin(), seen.end()), seen.end());
        for (uint32_t t : seen)
            if ((int64_t)t < vocab) logits[t] = logits[t] < 0.f ? logits[t] * rep : logits[t] / rep;
    }
    if ((presence != 0.f || frequency != 0.f) && ng > 0) {
        std::vector<uint32_t> g(generated, generated + ng);
        std::sort(g.begin(), g.end());
        for (size_t i = 0; i < g.size();) {
            size_t j = i;
            while (j < g.size() && g[j] == g[i]) ++j;
            if ((int64_t)g[i] < vocab) logits[g[i]] -= frequency * (float)(j - i) + presence;
            i = j;
        }
    }
}

}  // namespace mk

// The host sampler: penalties, the first-index argmax and the temperature / top-k / top-p draw
// (src/sampling.rs:95-169,337-433 of the reference).
#pragma once
#include "sampling_math.h"
#include <cstdint>
#include <cstring>
#include <cmath>
#include <stdexcept>
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

// Sampler::sample_stochastic + nucleus_probabilities + sample_from_probabilities (src/sampling.rs:145-169,337-390) as a
// function of one uniform draw u in [0, 1): scale by 1 / temperature, rank by (value descending, index ascending), keep
// the top_k best (0 = all), softmax over the kept, rank by (probability descending, index ascending), keep the shortest
// head whose probabilities add up to top_p, then walk the kept probabilities in index order until the running sum
// passes u times their total.  Sums run in the reference's order (index order for the totals, rank order for the
// nucleus); the exponential is det_expf, which the device kernel shares, so both give the same token for the same u.
inline uint32_t sample_top_k_top_p(const float* row, int64_t vocab, float temperature, int top_k, float top_p, float u) {
    std::vector<float> values(row, row + vocab);
    for (float& v : values) v /= temperature;
    std::vector<uint64_t> ranked((size_t)vocab);
    for (int64_t i = 0; i < vocab; ++i) ranked[(size_t)i] = rank_key(values[(size_t)i], (uint32_t)i);
    const bool cut = top_k > 0 && top_k < vocab;
    if (cut) {
        std::nth_element(ranked.begin(), ranked.begin() + top_k, ranked.end(), std::greater<uint64_t>());
        for (size_t i = (size_t)top_k; i < ranked.size(); ++i) values[rank_key_index(ranked[i])] = -INFINITY;
        ranked.resize((size_t)top_k);
    }
    float mx = -INFINITY;
    for (uint64_t k : ranked) { float v = values[rank_key_index(k)]; if (f32_order_key(v) > f32_order_key(mx)) mx = v; }
    std::vector<float> prob((size_t)vocab, 0.f);
    std::vector<uint32_t> kept;
    kept.reserve(ranked.size());
    for (uint64_t k : ranked) kept.push_back(rank_key_index(k));
    std::sort(kept.begin(), kept.end());                      // index order
    float sum = 0.f;
    for (uint32_t i : kept) { prob[i] = det_expf(values[i] - mx); sum += prob[i]; }
    if (!(sum > 0.f) || !std::isfinite(sum)) throw std::runtime_error("sampling distribution is empty");
    for (uint32_t i : kept) prob[i] /= sum;
    for (size_t j = 0; j < kept.size(); ++j) ranked[j] = rank_key(prob[kept[j]], kept[j]);
    std::sort(ranked.begin(), ranked.end(), std::greater<uint64_t>());
    if (top_p >= 0.f && top_p < 1.f) {
        float cumulative = 0.f;
        size_t keep = 0;
        for (uint64_t k : ranked) {
            cumulative += prob[rank_key_index(k)];
            ++keep;
            if (cumulative >= top_p) break;
        }
        for (size_t j = keep; j < ranked.size(); ++j) prob[rank_key_index(ranked[j])] = 0.f;
    }
    float total = 0.f;
    for (uint32_t i : kept) total += prob[i];
    const float target = u * total;
    float cumulative = 0.f;
    for (uint32_t i : kept) {
        if (prob[i] <= 0.f) continue;
        cumulative += prob[i];
        if (target < cumulative) return i;
    }
    return rank_key_index(ranked[0]);  // argmax of the probabilities: the best rank
}

}  // namespace mk

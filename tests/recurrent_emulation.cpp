// Host walk of the recurrent kernels' threads over the per-thread steps of recurrent_core.cuh (the same header the sm_100a
// kernels compile): every (lane, head, column / position) "thread" runs its rows in order, with the state indexing of the
// kernels.  Built by tests/test_recurrent_core.py with a plain C++ compiler; test infrastructure only.
#include "recurrent_core.cuh"
#include <cstdint>
#include <vector>

using namespace mk::recurrent;

extern "C" {

void emu_gated_delta_decay(const float* alpha, const float* time_bias, const float* state_decay, int64_t tokens, int heads, float* out) {
    for (int64_t i = 0; i < tokens * heads; ++i) out[i] = gated_delta_decay(alpha[i], time_bias[i % heads], state_decay[i % heads]);
}

// variant 0: the column lives in the output state and is updated in place (the kernel for any key_dim);
// variant 1: the column is held in a local array of KD floats (the register kernels), KD = 4 or 8 here
void emu_gated_delta(int variant, const float* query, const float* key, const float* value, const float* decay, const float* beta,
                     const int32_t* cu, int lanes, int heads, int key_dim, int value_dim, const float* state_in, float* state_out, float* out) {
    for (int lane = 0; lane < lanes; ++lane)
        for (int head = 0; head < heads; ++head)
            for (int v = 0; v < value_dim; ++v) {
                const int64_t sb = ((int64_t)lane * heads + head) * key_dim * value_dim;
                float s4[4], s8[8];
                if (variant == 0) {
                    for (int k = 0; k < key_dim; ++k) state_out[sb + (int64_t)k * value_dim + v] = state_in[sb + (int64_t)k * value_dim + v];
                } else {
                    for (int k = 0; k < key_dim; ++k) (key_dim == 4 ? s4[k] : s8[k]) = state_in[sb + (int64_t)k * value_dim + v];
                }
                for (int r = cu[lane]; r < cu[lane + 1]; ++r) {
                    const int64_t th = (int64_t)r * heads + head;
                    const float* ks = key + th * key_dim;
                    const float* qs = query + th * key_dim;
                    float o;
                    if (variant == 0) o = gated_delta_step(state_out + sb + v, value_dim, key_dim, ks, qs, decay[th], beta[th], value[th * value_dim + v]);
                    else if (key_dim == 4) o = gated_delta_step_reg<4>(s4, ks, qs, decay[th], beta[th], value[th * value_dim + v]);
                    else o = gated_delta_step_reg<8>(s8, ks, qs, decay[th], beta[th], value[th * value_dim + v]);
                    out[th * value_dim + v] = o;
                }
                if (variant != 0)
                    for (int k = 0; k < key_dim; ++k) state_out[sb + (int64_t)k * value_dim + v] = key_dim == 4 ? s4[k] : s8[k];
            }
}

void emu_mamba2(int variant, const float* xbc, const float* raw_dt, const float* dt_bias, const float* a, const float* d, const int32_t* cu,
                int lanes, int heads, int head_dim, int state_size, int groups, const float* state_in, float* state_out, float* out) {
    const int64_t inner = (int64_t)heads * head_dim, gsw = (int64_t)groups * state_size, width = inner + 2 * gsw;
    for (int lane = 0; lane < lanes; ++lane)
        for (int head = 0; head < heads; ++head)
            for (int p = 0; p < head_dim; ++p) {
                const int group = head / (heads / groups);
                const int64_t lane_i = (int64_t)head * head_dim + p;
                const int64_t sb = ((int64_t)lane * inner + lane_i) * state_size;
                float s3[3];
                if (variant == 0) for (int n = 0; n < state_size; ++n) state_out[sb + n] = state_in[sb + n];
                else for (int n = 0; n < 3; ++n) s3[n] = state_in[sb + n];
                for (int r = cu[lane]; r < cu[lane + 1]; ++r) {
                    const float* row = xbc + (int64_t)r * width;
                    const float* Bs = row + inner + (int64_t)group * state_size;
                    const float* Cs = row + inner + gsw + (int64_t)group * state_size;
                    float delta, decay;
                    mamba2_controls(raw_dt[(int64_t)r * heads + head], dt_bias[head], a[head], &delta, &decay);
                    out[(int64_t)r * inner + lane_i] = variant == 0 ? mamba2_step(state_out + sb, state_size, Bs, Cs, decay, delta, row[lane_i], d[head])
                                                                    : mamba2_step_reg<3>(s3, Bs, Cs, decay, delta, row[lane_i], d[head]);
                }
                if (variant != 0) for (int n = 0; n < 3; ++n) state_out[sb + n] = s3[n];
            }
}

static float window_value(const float* bcx, const float* tail_in, int hidden, int K, int lane, int first, int w, int c) {
    const int hist = K - 1;
    if (w < hist) return tail_in[((int64_t)lane * hist + w) * hidden + c];
    const float* row = bcx + (int64_t)(first + w - hist) * 3 * hidden;
    return mul(row[c], row[2 * hidden + c]);
}

void emu_short_conv(const float* bcx, const float* kernel, const int32_t* cu, int lanes, int hidden, int K, const float* tail_in, float* tail_out,
                    float* out) {
    const int rows = cu[lanes];
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < hidden; ++c) {
            int lo = 0, hi = lanes - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (cu[mid] <= r) lo = mid; else hi = mid - 1;
            }
            const int lane = lo, first = cu[lane];
            float window[8], taps[8];
            for (int j = 0; j < K; ++j) {
                window[j] = window_value(bcx, tail_in, hidden, K, lane, first, r - first + j, c);
                taps[j] = kernel[(int64_t)c * K + j];
            }
            out[(int64_t)r * hidden + c] = short_conv_tap_sum(window, taps, K, bcx[(int64_t)r * 3 * hidden + hidden + c]);
        }
    for (int lane = 0; lane < lanes; ++lane)
        for (int j = 0; j < K - 1; ++j)
            for (int c = 0; c < hidden; ++c)
                tail_out[((int64_t)lane * (K - 1) + j) * hidden + c] = window_value(bcx, tail_in, hidden, K, lane, cu[lane], cu[lane + 1] - cu[lane] + j, c);
}

}  // extern "C"

// Recurrent sequence mixers over ragged lanes: Gated DeltaNet (decay controls and the delta-rule recurrence), the Mamba2
// selective scan and the short convolution.  They restate crates/macllm-kernels/src/gated_delta.rs, crates/macllm-kernels/
// src/mamba2.rs and ShortConvolution::forward_lane (src/decoder.rs:1430-1492) of the reference as sm_100a kernels.
//
// Rows of lane l are cu[l] .. cu[l+1] of the packed batch.  Every kernel reads the lane's state from `*_in` and writes the
// next state to `*_out` (two buffers: the input stays valid, so a forward that fails in a later layer can fall back to it,
// the rule the reference states at gated_delta.rs:131-137).  The state of a lane is read from HBM once and written once per
// launch whatever the number of its rows: it lives in registers while the lane's tokens go by.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace mk {

// out[t][h] = exp(softplus(alpha[t][h] + time_bias[h]) * state_decay[h])
void launch_gated_delta_decay(const float* alpha, const float* time_bias, const float* state_decay, int64_t tokens, int heads, float* out,
                              cudaStream_t stream);

struct GatedDeltaArgs {
    const float* query = nullptr;   // [rows][heads][key_dim], normalised and scaled
    const float* key = nullptr;     // [rows][heads][key_dim], normalised
    const float* value = nullptr;   // [rows][heads][value_dim]
    const float* decay = nullptr;   // [rows][heads]
    const float* beta = nullptr;    // [rows][heads]
    const int32_t* cu = nullptr;    // [lanes + 1], device memory
    const float* state_in = nullptr;  // [lanes][heads][key_dim][value_dim]
    float* state_out = nullptr;
    float* out = nullptr;           // [rows][heads][value_dim]
    int lanes = 0, heads = 0, key_dim = 0, value_dim = 0;
};
void launch_gated_delta_recurrence(const GatedDeltaArgs& a, cudaStream_t stream);

struct Mamba2Args {
    const float* xbc = nullptr;     // [rows][heads*head_dim + 2*groups*state_size], laid out [x | B | C]
    const float* raw_dt = nullptr;  // [rows][heads]
    const float* dt_bias = nullptr; // [heads]
    const float* a = nullptr;       // [heads], negative
    const float* d = nullptr;       // [heads]
    const int32_t* cu = nullptr;    // [lanes + 1], device memory
    const float* state_in = nullptr;  // [lanes][heads][head_dim][state_size]
    float* state_out = nullptr;
    float* out = nullptr;           // [rows][heads][head_dim]
    int lanes = 0, heads = 0, head_dim = 0, state_size = 0, groups = 0;
};
// The group count a projection width implies, with the refusals of ScanGeometry::validate (mamba2.rs:64-150).
int mamba2_groups(int64_t xbc_width, int heads, int head_dim, int state_size);
void launch_mamba2_scan(const Mamba2Args& a, cudaStream_t stream);

struct ShortConvArgs {
    const float* bcx = nullptr;     // [rows][3*hidden], laid out [B | C | x]
    const float* kernel = nullptr;  // [hidden][K], oldest tap first
    const int32_t* cu = nullptr;    // [lanes + 1], device memory
    const float* tail_in = nullptr; // [lanes][K-1][hidden]: the lane's last K-1 rows of B*x (zeros for a fresh lane)
    float* tail_out = nullptr;
    float* out = nullptr;           // [rows][hidden]
    int rows = 0, lanes = 0, hidden = 0, K = 0;
};
constexpr int kShortConvMaxTaps = 8;
void launch_short_conv(const ShortConvArgs& a, cudaStream_t stream);

}  // namespace mk

// See recurrent.h.  The arithmetic of each thread is in recurrent_core.cuh.
#include "recurrent.h"
#include "recurrent_core.cuh"
#include "device_util.h"
#include <stdexcept>
#include <string>

namespace mk {

namespace {

using namespace recurrent;

__global__ void gated_delta_decay_kernel(const float* __restrict__ alpha, const float* __restrict__ time_bias,
                                         const float* __restrict__ state_decay, int64_t count, int heads, float* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        const int h = (int)(i % heads);
        out[i] = gated_delta_decay(alpha[i], time_bias[h], state_decay[h]);
    }
}

constexpr int kGdColumns = 64;  // value columns (threads) per CTA

// One CTA: 64 value columns of one (lane, head).  A thread keeps its column of the state - key_dim floats - in registers
// while the lane's rows go by; the row's key and query vectors are staged in shared memory for all columns.
template <int KD>
__global__ void __launch_bounds__(kGdColumns) gated_delta_reg_kernel(GatedDeltaArgs a) {
    __shared__ float ks[KD], qs[KD];
    const int v = blockIdx.x * kGdColumns + threadIdx.x, head = blockIdx.y, lane = blockIdx.z;
    const bool live = v < a.value_dim;
    const int64_t sb = ((int64_t)lane * a.heads + head) * KD * a.value_dim;
    float S[KD];
#pragma unroll
    for (int k = 0; k < KD; ++k) S[k] = live ? a.state_in[sb + (int64_t)k * a.value_dim + v] : 0.f;
    const int first = a.cu[lane], last = a.cu[lane + 1];
    for (int r = first; r < last; ++r) {
        const int64_t th = (int64_t)r * a.heads + head;
        for (int i = threadIdx.x; i < KD; i += kGdColumns) {
            ks[i] = a.key[th * KD + i];
            qs[i] = a.query[th * KD + i];
        }
        __syncthreads();
        if (live) a.out[th * a.value_dim + v] = gated_delta_step_reg<KD>(S, ks, qs, a.decay[th], a.beta[th], a.value[th * a.value_dim + v]);
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int k = 0; k < KD; ++k) a.state_out[sb + (int64_t)k * a.value_dim + v] = S[k];
    }
}

constexpr int kGdGenericMaxKey = 1024;

// Any key_dim up to 1024: the column lives in the output state (copied there first) and is updated in place.
__global__ void __launch_bounds__(kGdColumns) gated_delta_generic_kernel(GatedDeltaArgs a) {
    __shared__ float ks[kGdGenericMaxKey], qs[kGdGenericMaxKey];
    const int v = blockIdx.x * kGdColumns + threadIdx.x, head = blockIdx.y, lane = blockIdx.z;
    const bool live = v < a.value_dim;
    const int KD = a.key_dim;
    const int64_t sb = ((int64_t)lane * a.heads + head) * KD * a.value_dim;
    if (live)
        for (int k = 0; k < KD; ++k) a.state_out[sb + (int64_t)k * a.value_dim + v] = a.state_in[sb + (int64_t)k * a.value_dim + v];
    const int first = a.cu[lane], last = a.cu[lane + 1];
    for (int r = first; r < last; ++r) {
        const int64_t th = (int64_t)r * a.heads + head;
        for (int i = threadIdx.x; i < KD; i += kGdColumns) {
            ks[i] = a.key[th * KD + i];
            qs[i] = a.query[th * KD + i];
        }
        __syncthreads();
        if (live)
            a.out[th * a.value_dim + v] =
                gated_delta_step(a.state_out + sb + v, a.value_dim, KD, ks, qs, a.decay[th], a.beta[th], a.value[th * a.value_dim + v]);
        __syncthreads();
    }
}

constexpr int kMambaMaxPositions = 256;  // head_dim (threads) of one CTA
constexpr int kMambaMaxState = 1024;

// One CTA: the head_dim positions of one (lane, head); a thread keeps its position's state_size floats in registers.  The
// row's B and C vectors of the head's group are staged in shared memory; every thread derives the head's controls itself.
template <int N>
__global__ void __launch_bounds__(kMambaMaxPositions) mamba2_reg_kernel(Mamba2Args a) {
    __shared__ float Bs[N], Cs[N];
    const int p = threadIdx.x, head = blockIdx.x, lane = blockIdx.y;
    const bool live = p < a.head_dim;
    const int64_t inner = (int64_t)a.heads * a.head_dim, gsw = (int64_t)a.groups * N, width = inner + 2 * gsw;
    const int group = head / (a.heads / a.groups);
    const int64_t lane_i = (int64_t)head * a.head_dim + p;
    const int64_t sb = ((int64_t)lane * inner + lane_i) * N;
    float S[N];
#pragma unroll
    for (int n = 0; n < N; ++n) S[n] = live ? a.state_in[sb + n] : 0.f;
    const float dt_bias = a.dt_bias[head], av = a.a[head], skip = a.d[head];
    const int first = a.cu[lane], last = a.cu[lane + 1];
    for (int r = first; r < last; ++r) {
        const float* row = a.xbc + (int64_t)r * width;
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            Bs[i] = row[inner + (int64_t)group * N + i];
            Cs[i] = row[inner + gsw + (int64_t)group * N + i];
        }
        __syncthreads();
        if (live) {
            float delta, decay;
            mamba2_controls(a.raw_dt[(int64_t)r * a.heads + head], dt_bias, av, &delta, &decay);
            a.out[(int64_t)r * inner + lane_i] = mamba2_step_reg<N>(S, Bs, Cs, decay, delta, row[lane_i], skip);
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < N; ++n) a.state_out[sb + n] = S[n];
    }
}

__global__ void __launch_bounds__(kMambaMaxPositions) mamba2_generic_kernel(Mamba2Args a) {
    __shared__ float Bs[kMambaMaxState], Cs[kMambaMaxState];
    const int p = threadIdx.x, head = blockIdx.x, lane = blockIdx.y;
    const bool live = p < a.head_dim;
    const int N = a.state_size;
    const int64_t inner = (int64_t)a.heads * a.head_dim, gsw = (int64_t)a.groups * N, width = inner + 2 * gsw;
    const int group = head / (a.heads / a.groups);
    const int64_t lane_i = (int64_t)head * a.head_dim + p;
    const int64_t sb = ((int64_t)lane * inner + lane_i) * N;
    if (live)
        for (int n = 0; n < N; ++n) a.state_out[sb + n] = a.state_in[sb + n];
    const float dt_bias = a.dt_bias[head], av = a.a[head], skip = a.d[head];
    const int first = a.cu[lane], last = a.cu[lane + 1];
    for (int r = first; r < last; ++r) {
        const float* row = a.xbc + (int64_t)r * width;
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            Bs[i] = row[inner + (int64_t)group * N + i];
            Cs[i] = row[inner + gsw + (int64_t)group * N + i];
        }
        __syncthreads();
        if (live) {
            float delta, decay;
            mamba2_controls(a.raw_dt[(int64_t)r * a.heads + head], dt_bias, av, &delta, &decay);
            a.out[(int64_t)r * inner + lane_i] = mamba2_step(a.state_out + sb, N, Bs, Cs, decay, delta, row[lane_i], skip);
        }
        __syncthreads();
    }
}

// The lane a packed row belongs to: the last l with cu[l] <= row.
__device__ __forceinline__ int lane_of_row(const int32_t* cu, int lanes, int row) {
    int lo = 0, hi = lanes - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cu[mid] <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// B*x of window entry `w` (0 .. hist + n) of a lane: its tail for w < hist, its own rows after that.
__device__ __forceinline__ float window_value(const ShortConvArgs& a, int lane, int first, int w, int c) {
    const int hist = a.K - 1;
    if (w < hist) return a.tail_in[((int64_t)lane * hist + w) * a.hidden + c];
    const float* row = a.bcx + (int64_t)(first + w - hist) * 3 * a.hidden;
    return mul(row[c], row[2 * a.hidden + c]);
}

// One thread per (row, channel): the K window values are rebuilt from the rows themselves (one product each, the same
// rounding as the stored ones), so rows are independent of one another.
__global__ void short_conv_kernel(ShortConvArgs a) {
    const int64_t total = (int64_t)a.rows * a.hidden;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / a.hidden), c = (int)(i % a.hidden);
        const int lane = lane_of_row(a.cu, a.lanes, r);
        const int first = a.cu[lane];
        float window[kShortConvMaxTaps], taps[kShortConvMaxTaps];
        for (int j = 0; j < a.K; ++j) {
            window[j] = window_value(a, lane, first, r - first + j, c);
            taps[j] = a.kernel[(int64_t)c * a.K + j];
        }
        a.out[i] = short_conv_tap_sum(window, taps, a.K, a.bcx[(int64_t)r * 3 * a.hidden + a.hidden + c]);
    }
}

// The new tail of every lane: the last K-1 entries of its window.
__global__ void short_conv_tail_kernel(ShortConvArgs a) {
    const int hist = a.K - 1;
    const int64_t total = (int64_t)a.lanes * hist * a.hidden;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % a.hidden), j = (int)(i / a.hidden % hist), lane = (int)(i / a.hidden / hist);
        const int first = a.cu[lane], n = a.cu[lane + 1] - first;
        a.tail_out[i] = window_value(a, lane, first, n + j, c);
    }
}

int grid_for(int64_t work, int threads) {
    const int64_t blocks = (work + threads - 1) / threads;
    const int64_t cap = (int64_t)device_sm_count() * 8;
    return (int)std::max<int64_t>(1, std::min(blocks, cap));
}

}  // namespace

void launch_gated_delta_decay(const float* alpha, const float* time_bias, const float* state_decay, int64_t tokens, int heads, float* out,
                              cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0) throw std::runtime_error("Gated DeltaNet decay requires non-empty token and head dimensions");
    gated_delta_decay_kernel<<<grid_for(tokens * heads, 256), 256, 0, stream>>>(alpha, time_bias, state_decay, tokens * heads, heads, out);
    MK_CUDA(cudaGetLastError());
}

void launch_gated_delta_recurrence(const GatedDeltaArgs& a, cudaStream_t stream) {
    if (a.lanes <= 0 || a.heads <= 0 || a.key_dim <= 0 || a.value_dim <= 0)
        throw std::runtime_error("Gated DeltaNet decode has incompatible query/key geometry");
    if (a.key_dim > kGdGenericMaxKey) throw std::runtime_error("Gated DeltaNet key dimension " + std::to_string(a.key_dim) + " exceeds 1024");
    if (a.heads > 65535 || a.lanes > 65535) throw std::runtime_error("Gated DeltaNet recurrence: at most 65535 heads and 65535 lanes per launch");
    const dim3 grid((unsigned)((a.value_dim + kGdColumns - 1) / kGdColumns), (unsigned)a.heads, (unsigned)a.lanes);
    if (a.key_dim == 128) gated_delta_reg_kernel<128><<<grid, kGdColumns, 0, stream>>>(a);
    else if (a.key_dim == 64) gated_delta_reg_kernel<64><<<grid, kGdColumns, 0, stream>>>(a);
    else gated_delta_generic_kernel<<<grid, kGdColumns, 0, stream>>>(a);
    MK_CUDA(cudaGetLastError());
}

int mamba2_groups(int64_t xbc_width, int heads, int head_dim, int state_size) {
    if (heads <= 0 || head_dim <= 0 || state_size <= 0) throw std::runtime_error("Mamba2 scan requires non-empty dimensions");
    const int64_t inner = (int64_t)heads * head_dim;
    if (xbc_width < inner)
        throw std::runtime_error("Mamba2 xBC width " + std::to_string(xbc_width) + " is smaller than inner size " + std::to_string(inner));
    const int64_t bc = xbc_width - inner;
    if (bc == 0 || bc % (2 * (int64_t)state_size) != 0)
        throw std::runtime_error("Mamba2 xBC width " + std::to_string(xbc_width) + " cannot encode paired B/C states of width " +
                                 std::to_string(state_size));
    const int64_t groups = bc / (2 * (int64_t)state_size);
    if (heads % groups != 0)
        throw std::runtime_error("Mamba2 scan head count " + std::to_string(heads) + " is not divisible by inferred group count " +
                                 std::to_string(groups));
    return (int)groups;
}

void launch_mamba2_scan(const Mamba2Args& a, cudaStream_t stream) {
    if (a.lanes <= 0 || a.heads <= 0 || a.head_dim <= 0 || a.state_size <= 0 || a.groups <= 0 || a.heads % a.groups != 0)
        throw std::runtime_error("Mamba2 scan requires non-empty dimensions");
    if (a.head_dim > kMambaMaxPositions) throw std::runtime_error("Mamba2 head dimension " + std::to_string(a.head_dim) + " exceeds 256");
    if (a.state_size > kMambaMaxState) throw std::runtime_error("Mamba2 state size " + std::to_string(a.state_size) + " exceeds 1024");
    if (a.lanes > 65535) throw std::runtime_error("Mamba2 scan: at most 65535 lanes per launch");
    const dim3 grid((unsigned)a.heads, (unsigned)a.lanes);
    const int threads = (a.head_dim + 31) / 32 * 32;
    if (a.state_size == 128) mamba2_reg_kernel<128><<<grid, threads, 0, stream>>>(a);
    else if (a.state_size == 64) mamba2_reg_kernel<64><<<grid, threads, 0, stream>>>(a);
    else if (a.state_size == 16) mamba2_reg_kernel<16><<<grid, threads, 0, stream>>>(a);
    else mamba2_generic_kernel<<<grid, threads, 0, stream>>>(a);
    MK_CUDA(cudaGetLastError());
}

void launch_short_conv(const ShortConvArgs& a, cudaStream_t stream) {
    if (a.rows <= 0 || a.lanes <= 0 || a.hidden <= 0 || a.K < 1) throw std::runtime_error("short-convolution state geometry does not match its layer");
    if (a.K > kShortConvMaxTaps) throw std::runtime_error("short-convolution kernel size " + std::to_string(a.K) + " exceeds 8");
    short_conv_kernel<<<grid_for((int64_t)a.rows * a.hidden, 256), 256, 0, stream>>>(a);
    MK_CUDA(cudaGetLastError());
    if (a.K > 1) {
        short_conv_tail_kernel<<<grid_for((int64_t)a.lanes * (a.K - 1) * a.hidden, 256), 256, 0, stream>>>(a);
        MK_CUDA(cudaGetLastError());
    }
}

}  // namespace mk

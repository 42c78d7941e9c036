// Device-side construction of the ragged batch descriptor of one scheduler tick.
//
// The reference assembles these arrays on the host and uploads each of them every tick
// (packed ids / start positions / lane lengths in src/decoder.rs:4203-4269, the page table and lane
// offsets in crates/macllm-kv/src/cache.rs:2707-2851, last-row indices in src/decoder.rs:3333-3341).
// Here the host uploads one small header per lane plus the lanes' block tables, and this kernel
// expands them into cu_seqlens, per-token positions, the slot mapping of the paged KV write
// (token at absolute position p -> block p / block_tokens, row p % block_tokens,
// cache.rs:2613-2638), last-token indices and the attention query-tile work list.
#include "kernels.h"

namespace mk {

namespace {

__global__ void __launch_bounds__(1024) build_batch_kernel(BatchDesc b, int block_tokens, int q_tile) {
    __shared__ int s_total_tiles;
    if (threadIdx.x == 0) {
        int acc = 0, tiles = 0;
        b.cu_seqlens[0] = 0;
        for (int l = 0; l < b.lanes; ++l) {
            LaneHeader h = b.hdr[l];
            int first_tile = tiles;
            int nt = (h.n_tokens + q_tile - 1) / q_tile;
            for (int i = 0; i < nt && first_tile + i < b.max_tiles; ++i) {
                b.tile_lane[first_tile + i] = l;
                b.tile_row0[first_tile + i] = i * q_tile;
            }
            tiles += nt;
            acc += h.n_tokens;
            b.cu_seqlens[l + 1] = acc;
            b.last_index[l] = acc - 1;
        }
        if (tiles > b.max_tiles || acc != b.T) atomicExch(b.error_flag, 1);
        *b.n_tiles = min(tiles, b.max_tiles);
        s_total_tiles = tiles;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < b.T; t += blockDim.x) {
        int lo = 0, hi = b.lanes;  // largest lane with cu[lane] <= t
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (b.cu_seqlens[mid] <= t) lo = mid; else hi = mid;
        }
        LaneHeader h = b.hdr[lo];
        int pos = h.start_pos + (t - b.cu_seqlens[lo]);
        int blk = pos / block_tokens;
        int64_t slot = 0;
        if (blk >= h.n_blocks || pos < 0) {
            atomicExch(b.error_flag, 2);
        } else {
            slot = (int64_t)b.tables[h.table_off + blk] * block_tokens + pos % block_tokens;
        }
        b.positions[t] = pos;
        b.token_lane[t] = lo;
        b.slots[t] = slot;
    }
}

}  // namespace

void launch_build_batch(const BatchDesc& b, int block_tokens, int q_tile, cudaStream_t s) {
    build_batch_kernel<<<1, 1024, 0, s>>>(b, block_tokens, q_tile);
    MK_LAUNCH_CHECK();
}

}  // namespace mk

// Flat scatter-add without atomics: output[:] = 0, then output[index[i]] += update[i] for every valid i.
//
// Replaces prepareFlatScatterAdd / runFlatScatterAdd (Utilities/Expression/FlatScatterAddKernel.h:16-74;
// FlatScatterAddKernel.cu:46-64 materialise, :120-200 CUB sort + reduce-by-key, :330-376 cuSPARSE axpby), the step behind
// arg scans in min / max scan backward (StampedEquation.cpp:3134-3137).  The reference canonicalises duplicates with
// cub::DeviceRadixSort::SortPairs + cub::DeviceReduce::ReduceByKey and applies the unique updates with cusparseAxpby;
// here the same three steps are this library's own kernels and no vendor library is involved:
//
//   1. a stable least-significant-digit radix sort of (destination, update) pairs, 8 bits per pass, over only as many
//      bits as the output size needs (an output of 2^20 elements sorts in three passes, one of 65536 in two, one of
//      200 in one).  The first pass reads the caller's tensors directly and turns invalid destinations (the sentinel
//      0xFFFFFFFF or anything past the output) into the pair (destination 0, update +0), which changes no sum.
//      Per pass: digit histogram per tile (shared-memory counters) -> one exclusive scan of the [digit][tile] table ->
//      stable scatter (each warp ranks its 32 consecutive elements per round with one ballot per digit bit; warps of a tile are ordered
//      by a per-digit prefix over the warps' counters).
//   2. one kernel that walks the sorted pairs and adds every run of equal destinations IN THE ORIGINAL ORDER of its
//      updates (the sort is stable), starting from +0: the result equals the sequential loop of the definition bit for
//      bit, which a tree-shaped reduce-by-key does not promise.  Every thread walks eight consecutive pairs; a run that
//      spans threads hands its running sum from lane to lane, one that leaves a warp's window is finished by that warp.
//   3. the store of each run's sum into the zero-filled output is part of step 2.
//
// Indices known to be unique and valid skip the sort: zero fill + one scatter kernel.
// fp32 updates and output, uint32 indices (what the reference supports).
#include "common.cuh"

namespace tb {
namespace {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kItems = 16;                           // elements per thread and tile
constexpr int kTile = kSortThreads * kItems;          // 4096 elements per CTA
constexpr int kRadix = 256;

struct PassArgs {
    const uint32_t* keys_in;   // nullptr in the first pass: keys come from `indices`
    const float* vals_in;
    uint32_t* keys_out;
    float* vals_out;
    const uint32_t* indices;   // first pass only
    uint32_t* table;           // [kRadix][tiles]
    uint32_t* totals;          // [kRadix] of this pass, zero before the histogram kernel
    uint64_t n;
    uint64_t output_numel;
    uint32_t tiles;
    uint32_t shift;
};

// An invalid destination (the sentinel or anything past the output) becomes the pair (destination 0, update +0): adding
// +0 leaves every running sum as it is -- a sum that starts from +0 is never -0 -- so no compaction pass and no extra
// key bit are needed (the reference's materialise kernel makes the same substitution, FlatScatterAddKernel.cu:55-63).
__device__ __forceinline__ bool invalidDestination(const PassArgs& a, uint32_t dst) {
    return dst == 0xFFFFFFFFu || static_cast<uint64_t>(dst) >= a.output_numel;
}
// FIRST = the pass that reads the caller's tensors; later passes read the ping-pong arrays.  A template parameter, not
// a run-time test, so that the loads of a thread carry no branches between them and are all in flight together.
template <bool FIRST>
__device__ __forceinline__ uint32_t loadKey(const PassArgs& a, uint64_t i) {
    if constexpr (!FIRST) return a.keys_in[i];
    const uint32_t dst = a.indices[i];
    return invalidDestination(a, dst) ? 0u : dst;
}
template <bool FIRST>
__device__ __forceinline__ void loadPair(const PassArgs& a, uint64_t i, uint32_t& key, float& value) {
    value = a.vals_in[i];
    if constexpr (FIRST) {
        const uint32_t dst = a.indices[i];
        const bool invalid = invalidDestination(a, dst);
        key = invalid ? 0u : dst;
        value = invalid ? 0.0f : value;
    } else {
        key = a.keys_in[i];
    }
}

// One CTA counts kHistTiles consecutive tiles: a table column per tile, and ONE addition per digit and CTA to the
// per-digit totals (4096 CTAs adding to the same 256 words cost 26 us of the 45 us this kernel took with a tile per CTA).
constexpr int kHistTiles = 4;

template <bool FIRST>
__global__ void __launch_bounds__(kSortThreads) digitHistogramKernel(PassArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ uint32_t counts[kRadix];
    uint32_t total = 0;
    for (uint32_t tile = blockIdx.x * kHistTiles; tile < min(a.tiles, (blockIdx.x + 1) * kHistTiles); ++tile) {
        counts[threadIdx.x] = 0;
        __syncthreads();
        const uint64_t base = static_cast<uint64_t>(tile) * kTile;
        uint32_t digit[kItems];  // all loads first, then the counters: the loads of a thread are in flight together
        if (base + kTile <= a.n) {  // a full tile: unconditional loads
#pragma unroll
            for (int r = 0; r < kItems; ++r) digit[r] = (loadKey<FIRST>(a, base + static_cast<uint64_t>(r) * kSortThreads + threadIdx.x) >> a.shift) & 0xFFu;
        } else {
#pragma unroll
            for (int r = 0; r < kItems; ++r) {
                const uint64_t i = base + static_cast<uint64_t>(r) * kSortThreads + threadIdx.x;
                digit[r] = i < a.n ? (loadKey<FIRST>(a, i) >> a.shift) & 0xFFu : 0x100u;
            }
        }
#pragma unroll
        for (int r = 0; r < kItems; ++r)
            if (digit[r] < 0x100u) atomicAdd(&counts[digit[r]], 1u);  // integer counters: the order is irrelevant
        __syncthreads();
        const uint32_t c = counts[threadIdx.x];
        a.table[static_cast<uint64_t>(threadIdx.x) * a.tiles + tile] = c;
        total += c;
        __syncthreads();  // the counters are cleared for the next tile only after everybody has read them
    }
    if (total) atomicAdd(&a.totals[threadIdx.x], total);  // integer sum: the same value whatever the order
}

// Exclusive prefix sum of the [digit][tile] table in digit-major order, in place.  CTA d owns row d: it starts from the
// number of elements with a smaller digit (the per-digit totals the histogram kernel accumulated) and scans its row in
// chunks of 1024 tiles with a running carry.
__global__ void __launch_bounds__(1024) tableScanKernel(uint32_t* table, const uint32_t* totals, uint32_t tiles) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t carry;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, digit = blockIdx.x;
    if (warp == 0) {
        uint32_t below = 0;
        for (uint32_t d = lane; d < digit; d += 32) below += totals[d];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) below += __shfl_xor_sync(0xFFFFFFFFu, below, o);
        if (lane == 0) carry = below;
    }
    __syncthreads();
    uint32_t* row = table + static_cast<uint64_t>(digit) * tiles;
    for (uint32_t t0 = 0; t0 < tiles; t0 += 1024) {
        const uint32_t t = t0 + threadIdx.x;
        const uint32_t v = t < tiles ? row[t] : 0u;
        uint32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t u = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= static_cast<uint32_t>(d)) incl += u;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            uint32_t w = warp_sums[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t u = __shfl_up_sync(0xFFFFFFFFu, w, d);
                if (lane >= static_cast<uint32_t>(d)) w += u;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const uint32_t before = carry + (warp ? warp_sums[warp - 1] : 0u) + incl - v;
        if (t < tiles) row[t] = before;
        __syncthreads();  // everybody has read carry and warp_sums
        if (threadIdx.x == 1023) carry = before + v;
        __syncthreads();
    }
}

// Stable scatter of one tile.  Warp w owns elements [w * 32 * kItems, (w + 1) * 32 * kItems) of the tile, in kItems rounds
// of 32 consecutive elements, so "earlier in the input" means (lower warp, lower round, lower lane).  The tile is first
// put into digit order in shared memory (position = elements of the tile with a smaller digit + elements with the same
// digit in earlier warps + rank inside the warp) and then written out by consecutive threads, so that every run of
// equal digits leaves the CTA as consecutive, coalesced stores.
template <bool FIRST>
__global__ void __launch_bounds__(kSortThreads, 3) digitScatterKernel(PassArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ uint32_t warp_counts[kSortWarps][kRadix];
    __shared__ uint32_t digit_start[kRadix];   // first position of the digit inside the sorted tile
    __shared__ uint32_t global_shift[kRadix];  // (position in the output) - (position in the sorted tile), modulo 2^32
    __shared__ uint32_t scan_sums[kSortWarps];
    __shared__ uint32_t tile_keys[kTile];
    __shared__ float tile_vals[kTile];
    for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&warp_counts[0][0])[i] = 0;
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint64_t tile_base = static_cast<uint64_t>(blockIdx.x) * kTile;
    const uint64_t base = tile_base + static_cast<uint64_t>(warp) * (32 * kItems);
    uint32_t key[kItems], rank[kItems];
    float val[kItems];
    if (tile_base + kTile <= a.n) {  // a full tile: unconditional loads
#pragma unroll
        for (int r = 0; r < kItems; ++r) loadPair<FIRST>(a, base + static_cast<uint64_t>(r) * 32 + lane, key[r], val[r]);
    } else {
#pragma unroll
        for (int r = 0; r < kItems; ++r) {
            const uint64_t i = base + static_cast<uint64_t>(r) * 32 + lane;
            key[r] = 0xFFFFFFFFu;
            val[r] = 0.0f;
            if (i < a.n) loadPair<FIRST>(a, i, key[r], val[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < kItems; ++r) {
        const uint64_t i = base + static_cast<uint64_t>(r) * 32 + lane;
        const bool live = i < a.n;
        const uint32_t digit = (key[r] >> a.shift) & 0xFFu;
        // lanes past the end take no part; they sit at the end of the last tile so the ranks of live lanes are unaffected
        const uint32_t live_mask = __ballot_sync(0xFFFFFFFFu, live);
        // lanes with the same digit: one ballot per digit bit (the match instruction runs on a pipe eight times slower)
        uint32_t peers = live_mask;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const bool set = (digit >> b) & 1u;
            const uint32_t with_bit = __ballot_sync(0xFFFFFFFFu, set);
            peers &= set ? with_bit : ~with_bit;
        }
        uint32_t before = 0;
        if (live) {
            const uint32_t leader = __ffs(peers) - 1u;
            uint32_t start = 0;
            if (lane == leader) {
                start = warp_counts[warp][digit];
                warp_counts[warp][digit] = start + __popc(peers);
            }
            start = __shfl_sync(peers, start, leader);
            before = start + __popc(peers & ((1u << lane) - 1u));
        }
        rank[r] = before;
        __syncwarp();
    }
    __syncthreads();
    {   // thread d: exclusive prefix of digit d over the warps, the digit's total, then an exclusive scan over the digits
        const uint32_t d = threadIdx.x;
        uint32_t total = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const uint32_t c = warp_counts[w][d];
            warp_counts[w][d] = total;
            total += c;
        }
        uint32_t incl = total;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t u = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= static_cast<uint32_t>(o)) incl += u;
        }
        if (lane == 31) scan_sums[warp] = incl;
        __syncthreads();
        uint32_t warps_before = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) warps_before += static_cast<uint32_t>(w) < warp ? scan_sums[w] : 0u;
        const uint32_t first = warps_before + incl - total;
        digit_start[d] = first;
        global_shift[d] = a.table[static_cast<uint64_t>(d) * a.tiles + blockIdx.x] - first;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kItems; ++r) {
        const uint64_t i = base + static_cast<uint64_t>(r) * 32 + lane;
        if (i < a.n) {
            const uint32_t d = (key[r] >> a.shift) & 0xFFu;
            const uint32_t pos = digit_start[d] + warp_counts[warp][d] + rank[r];
            tile_keys[pos] = key[r];
            tile_vals[pos] = val[r];
        }
    }
    __syncthreads();
    const uint32_t live_in_tile = static_cast<uint32_t>(min(static_cast<uint64_t>(kTile), a.n - tile_base));
#pragma unroll
    for (int r = 0; r < kItems; ++r) {
        const uint32_t idx = static_cast<uint32_t>(r) * kSortThreads + threadIdx.x;
        if (idx < live_in_tile) {
            const uint32_t k = tile_keys[idx];
            const uint32_t pos = global_shift[(k >> a.shift) & 0xFFu] + idx;
            a.keys_out[pos] = k;
            a.vals_out[pos] = tile_vals[idx];
        }
    }
}

// Sorted pairs -> output.  Every thread takes kApplyItems consecutive sorted positions (vector loads) and walks them in
// order, so all lanes add: runs that begin inside a thread's chunk start from +0 there; a chunk whose first elements
// continue the previous thread's last run waits for that run's sum (a shuffle from the lane below, repeated until no lane
// waits -- as many rounds as a run spans threads) and goes on adding to it, which keeps the order of the definition.
// A run belongs to the warp that holds its head: the run that is still open at the end of a warp's 32 x kApplyItems
// window is finished by that warp with global loads (32 at a time, added one after another), and the next warp skips
// the elements that continue it.
constexpr int kApplyItems = 8;
constexpr int kApplyThreads = 256;

__global__ void __launch_bounds__(kApplyThreads) applyRunsKernel(const uint32_t* __restrict__ keys, const float* __restrict__ vals, float* __restrict__ output,
                                                                 uint64_t n, uint64_t output_numel) {
    gridDependencyWait();
    gridLaunchDependents();
    constexpr uint32_t FULL = 0xFFFFFFFFu;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t i0 = (static_cast<uint64_t>(blockIdx.x) * kApplyThreads + threadIdx.x) * kApplyItems;
    const uint64_t window_end = i0 - static_cast<uint64_t>(lane) * kApplyItems + 32ull * kApplyItems;
    uint32_t k[kApplyItems];
    float v[kApplyItems];
    if (i0 + kApplyItems <= n) {
        const uint4 ka = *reinterpret_cast<const uint4*>(keys + i0), kb = *reinterpret_cast<const uint4*>(keys + i0 + 4);
        const float4 va = *reinterpret_cast<const float4*>(vals + i0), vb = *reinterpret_cast<const float4*>(vals + i0 + 4);
        k[0] = ka.x, k[1] = ka.y, k[2] = ka.z, k[3] = ka.w, k[4] = kb.x, k[5] = kb.y, k[6] = kb.z, k[7] = kb.w;
        v[0] = va.x, v[1] = va.y, v[2] = va.z, v[3] = va.w, v[4] = vb.x, v[5] = vb.y, v[6] = vb.z, v[7] = vb.w;
    } else {
#pragma unroll
        for (int e = 0; e < kApplyItems; ++e) {
            const bool live = i0 + e < n;
            k[e] = live ? keys[i0 + e] : 0xFFFFFFFFu;  // never a valid destination (valid ones are below output_numel <= 2^32 - 1)
            v[e] = live ? vals[i0 + e] : 0.0f;
        }
    }
    auto valid = [&](uint32_t key) { return static_cast<uint64_t>(key) < output_numel; };

    // does this chunk begin inside a run that started earlier?
    uint32_t below = __shfl_up_sync(FULL, k[kApplyItems - 1], 1);
    if (lane == 0) below = (i0 > 0 && i0 <= n) ? keys[i0 - 1] : ~k[0];
    const bool continues = i0 > 0 && i0 < n && below == k[0];

    // first segment: the leading elements equal to k[0]
    int first_len = 1;
    {
        bool same = true;
#pragma unroll
        for (int e = 1; e < kApplyItems; ++e) {
            same = same && k[e] == k[0];
            first_len += same ? 1 : 0;
        }
    }
    // runs that begin after the first segment: closed ones are stored at once, the last one stays open as the tail
    float tail_sum = 0.0f;
    uint32_t tail_key = k[kApplyItems - 1];
    bool tail_ready = false, tail_owned = true;
#pragma unroll
    for (int e = 1; e < kApplyItems; ++e) {
        if (e >= first_len) {
            if (k[e] != k[e - 1]) {
                if (tail_ready && valid(k[e - 1])) output[k[e - 1]] = tail_sum;
                tail_sum = 0.0f;
                tail_ready = true;
            }
            tail_sum += v[e];
        }
    }
    // the first segment: a head starts from +0 at once; a continuation waits for the sum of the lane below
    const bool whole_chunk = first_len == kApplyItems;
    bool waiting = continues && lane != 0;
    if (!continues || lane == 0) {
        // lane 0 of a warp never adds to a run that began in an earlier warp: that warp finishes it
        const bool owned = !continues;
        float sum = 0.0f;
#pragma unroll
        for (int e = 0; e < kApplyItems; ++e)
            if (e < first_len) sum += v[e];
        if (whole_chunk) {
            tail_sum = sum, tail_owned = owned, tail_ready = true;
        } else if (owned && valid(k[0])) {
            output[k[0]] = sum;
        }
    }
    while (__ballot_sync(FULL, waiting) != 0) {
        const float c_sum = __shfl_up_sync(FULL, tail_sum, 1);
        const bool c_owned = __shfl_up_sync(FULL, tail_owned ? 1 : 0, 1) != 0;
        const bool c_ready = __shfl_up_sync(FULL, tail_ready ? 1 : 0, 1) != 0;
        if (waiting && c_ready) {
            float sum = c_sum;
#pragma unroll
            for (int e = 0; e < kApplyItems; ++e)
                if (e < first_len) sum += v[e];
            if (whole_chunk) {
                tail_sum = sum, tail_owned = c_owned, tail_ready = true;
            } else if (c_owned && valid(k[0])) {
                output[k[0]] = sum;
            }
            waiting = false;
        }
    }
    // the tail: complete unless the next lane continues it; lane 31's may run on past the warp's window
    const bool next_continues = __shfl_down_sync(FULL, continues ? 1 : 0, 1) != 0;
    const bool mine_to_store = tail_owned && valid(tail_key) && i0 < n;
    if (lane != 31 && !next_continues && mine_to_store) output[tail_key] = tail_sum;
    const bool runs_on = lane == 31 && mine_to_store && window_end < n && keys[window_end] == tail_key;
    if (lane == 31 && mine_to_store && !runs_on) output[tail_key] = tail_sum;
    if (__ballot_sync(FULL, runs_on) != 0) {
        const uint32_t rk = __shfl_sync(FULL, tail_key, 31);
        float rs = __shfl_sync(FULL, tail_sum, 31);
        // batches of 128 pairs (four coalesced loads per lane), the next batch in flight while this one is added
        constexpr int kBatch = 4;
        uint64_t rj = window_end;
        uint32_t bk[kBatch], nk[kBatch];
        float bx[kBatch], nx[kBatch];
        auto load = [&](uint64_t from, uint32_t (&kk)[kBatch], float (&xx)[kBatch]) {
#pragma unroll
            for (int t = 0; t < kBatch; ++t) {
                const uint64_t p = from + static_cast<uint64_t>(t) * 32 + lane;
                const bool live = p < n;
                kk[t] = live ? keys[p] : ~rk;  // anything but the run's destination
                xx[t] = live ? vals[p] : 0.0f;
            }
        };
        load(rj, bk, bx);
        bool more = true;
        while (more) {
            load(rj + 32ull * kBatch, nk, nx);
#pragma unroll
            for (int t = 0; t < kBatch; ++t) {
                if (more) {
                    const uint32_t in_run = __ballot_sync(FULL, bk[t] == rk);
                    const uint32_t len = in_run == FULL ? 32u : static_cast<uint32_t>(__ffs(~in_run) - 1);  // the leading set bits
                    if (len == 32u) {
#pragma unroll
                        for (int u = 0; u < 32; ++u) rs += __shfl_sync(FULL, bx[t], u);  // unrolled: the shuffles run ahead of the adds
                    } else {
                        for (uint32_t u = 0; u < len; ++u) rs += __shfl_sync(FULL, bx[t], u);
                    }
                    more = len == 32u;
                }
            }
            rj += 32ull * kBatch;
#pragma unroll
            for (int t = 0; t < kBatch; ++t) bk[t] = nk[t], bx[t] = nx[t];
        }
        if (lane == 31) output[rk] = rs;
    }
}

__global__ void __launch_bounds__(256) scatterUniqueKernel(const float* updates, const uint32_t* indices, float* output, uint64_t n) {
    gridDependencyWait();
    gridLaunchDependents();
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) output[indices[i]] = 0.0f + updates[i];
}

uint32_t sortPasses(uint64_t output_numel) {
    uint32_t bits = 0;
    while (bits < 32 && ((output_numel - 1) >> bits) != 0) ++bits;  // the largest destination is output_numel - 1
    return bits == 0 ? 1 : (bits + 7) / 8;
}

size_t alignUp(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
constexpr size_t kTotalsBytes = 4 * kRadix * sizeof(uint32_t);  // per-digit totals of up to four passes

}  // namespace
}  // namespace tb

extern "C" {

int thor_b200_scatter_add_workspace_bytes(const thor_b200_scatter_add_desc* desc, size_t* bytes) {
    using namespace tb;
    TB_REQUIRE(desc != nullptr && bytes != nullptr, "scatter_add_workspace_bytes: null argument");
    TB_REQUIRE(desc->value_dtype == THOR_B200_FP32, "scatter_add: only fp32 updates and outputs are supported (as in the reference), got %s",
               dtypeName(desc->value_dtype));
    TB_REQUIRE(desc->index_policy == THOR_B200_SCATTER_CANONICALIZE || desc->index_policy == THOR_B200_SCATTER_UNIQUE_VALID,
               "scatter_add: unknown index policy %d", desc->index_policy);
    TB_REQUIRE(desc->num_updates < (1ull << 31), "scatter_add: at most 2^31 - 1 updates");
    TB_REQUIRE(desc->output_numel < (1ull << 32), "scatter_add: 32-bit destinations address at most 2^32 - 1 output elements");
    if (desc->index_policy == THOR_B200_SCATTER_UNIQUE_VALID || desc->num_updates == 0) {
        *bytes = 1;  // the reference's "at least one byte" workspace convention
        return THOR_B200_OK;
    }
    const size_t n = static_cast<size_t>(desc->num_updates);
    const size_t tiles = (n + kTile - 1) / kTile;
    *bytes = 4 * alignUp(n * 4) + alignUp(tiles * kRadix * 4) + kTotalsBytes;
    return THOR_B200_OK;
}

int thor_b200_scatter_add_launch(const thor_b200_scatter_add_desc* desc, const void* updates, const void* indices, void* output, void* workspace,
                                 size_t workspace_bytes, void* stream_) {
    using namespace tb;
    size_t need = 0;
    if (int st = thor_b200_scatter_add_workspace_bytes(desc, &need)) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const uint64_t n = desc->num_updates, out_n = desc->output_numel;
    TB_REQUIRE(out_n == 0 || output != nullptr, "scatter_add: null output");
    if (out_n) TB_CUDA(cudaMemsetAsync(output, 0, out_n * sizeof(float), stream));
    if (n == 0 || out_n == 0) return THOR_B200_OK;
    TB_REQUIRE(updates != nullptr && indices != nullptr, "scatter_add: null updates or indices");
    const uint32_t blocks = static_cast<uint32_t>((n + 255) / 256);
    if (desc->index_policy == THOR_B200_SCATTER_UNIQUE_VALID) {
        TB_CUDA(launchDependent(scatterUniqueKernel, dim3(blocks), dim3(256), 0, stream, static_cast<const float*>(updates),
                                static_cast<const uint32_t*>(indices), static_cast<float*>(output), n));
        countLaunch();
        return THOR_B200_OK;
    }
    TB_REQUIRE(workspace != nullptr && workspace_bytes >= need, "scatter_add: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    TB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15u) == 0, "scatter_add: workspace must be 16-byte aligned");
    const size_t part = alignUp(static_cast<size_t>(n) * 4);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    uint32_t* keys[2] = {reinterpret_cast<uint32_t*>(ws), reinterpret_cast<uint32_t*>(ws + part)};
    float* vals[2] = {reinterpret_cast<float*>(ws + 2 * part), reinterpret_cast<float*>(ws + 3 * part)};
    const uint32_t tiles = static_cast<uint32_t>((n + kTile - 1) / kTile);
    PassArgs a = {};
    a.table = reinterpret_cast<uint32_t*>(ws + 4 * part);
    a.n = n;
    a.output_numel = out_n;
    a.tiles = tiles;
    a.indices = static_cast<const uint32_t*>(indices);
    const uint32_t passes = sortPasses(out_n);
    uint32_t* totals = reinterpret_cast<uint32_t*>(ws + 4 * part + alignUp(static_cast<size_t>(tiles) * kRadix * 4));
    TB_CUDA(cudaMemsetAsync(totals, 0, kTotalsBytes, stream));
    for (uint32_t p = 0; p < passes; ++p) {
        a.keys_in = p == 0 ? nullptr : keys[(p - 1) & 1];
        a.vals_in = p == 0 ? static_cast<const float*>(updates) : vals[(p - 1) & 1];
        a.keys_out = keys[p & 1];
        a.vals_out = vals[p & 1];
        a.shift = 8 * p;
        a.totals = totals + p * kRadix;
        TB_CUDA(launchDependent(p == 0 ? digitHistogramKernel<true> : digitHistogramKernel<false>, dim3((tiles + kHistTiles - 1) / kHistTiles), dim3(kSortThreads), 0,
                                stream, a));
        TB_CUDA(launchDependent(tableScanKernel, dim3(kRadix), dim3(1024), 0, stream, a.table, static_cast<const uint32_t*>(a.totals), tiles));
        TB_CUDA(launchDependent(p == 0 ? digitScatterKernel<true> : digitScatterKernel<false>, dim3(tiles), dim3(kSortThreads), 0, stream, a));
        countLaunch(3);
    }
    const uint32_t apply_blocks = static_cast<uint32_t>((n + static_cast<uint64_t>(kApplyThreads) * kApplyItems - 1) / (static_cast<uint64_t>(kApplyThreads) * kApplyItems));
    TB_CUDA(launchDependent(applyRunsKernel, dim3(apply_blocks), dim3(kApplyThreads), 0, stream, static_cast<const uint32_t*>(keys[(passes - 1) & 1]),
                            static_cast<const float*>(vals[(passes - 1) & 1]), static_cast<float*>(output), n, out_n));
    countLaunch();
    return THOR_B200_OK;
}

int thor_b200_scatter_add_launch_count(const thor_b200_scatter_add_desc* desc) {
    if (desc == nullptr || desc->num_updates == 0 || desc->output_numel == 0) return 0;
    if (desc->index_policy == THOR_B200_SCATTER_UNIQUE_VALID) return 1;
    return static_cast<int>(3 * tb::sortPasses(desc->output_numel) + 1);
}

}  // extern "C"

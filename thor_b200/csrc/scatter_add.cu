// Flat scatter-add without atomics: output[:] = 0, then output[index[i]] += update[i] for every valid i.
//
// Replaces prepareFlatScatterAdd / runFlatScatterAdd (Utilities/Expression/FlatScatterAddKernel.h:16-74;
// FlatScatterAddKernel.cu:46-64 materialise, :120-200 CUB sort + reduce-by-key, :330-376 cuSPARSE axpby), the step behind
// arg scans in min / max scan backward (StampedEquation.cpp:3134-3137).  The reference canonicalises duplicates with
// cub::DeviceRadixSort::SortPairs + cub::DeviceReduce::ReduceByKey and applies the unique updates with cusparseAxpby;
// here the same three steps are this library's own kernels and no vendor library is involved:
//
//   1. a stable least-significant-digit radix sort of (destination, update) pairs, 8 bits per pass, over only as many
//      bits as the output size needs (an output of 2^20 elements sorts in three passes, one of 200 in one).  The first
//      pass reads the caller's tensors directly and maps invalid destinations (the sentinel 0xFFFFFFFF or anything past
//      the output) to one key above every valid destination, so they sort to the end and no compaction pass exists.
//      Per pass: digit histogram per tile (shared-memory counters) -> one exclusive scan of the [digit][tile] table ->
//      stable scatter (each warp ranks its 32 consecutive elements per round with match.any; warps of a tile are ordered
//      by a per-digit prefix over the warps' counters).
//   2. one kernel that finds the head of every run of equal destinations in the sorted order and adds the run's updates
//      IN THEIR ORIGINAL ORDER (the sort is stable), starting from +0: the result equals the sequential loop of the
//      definition bit for bit, which a tree-shaped reduce-by-key does not promise.  Long runs are walked by a whole warp
//      that keeps that order: lanes load 32 consecutive updates at once, lane 0 adds them one after another.
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
    uint64_t n;
    uint64_t output_numel;
    uint32_t tiles;
    uint32_t shift;
};

__device__ __forceinline__ uint32_t loadKey(const PassArgs& a, uint64_t i) {
    if (a.keys_in != nullptr) return a.keys_in[i];
    const uint32_t dst = a.indices[i];
    // the sentinel and out-of-range destinations share the key just above the last valid destination
    return (dst == 0xFFFFFFFFu || static_cast<uint64_t>(dst) >= a.output_numel) ? static_cast<uint32_t>(a.output_numel) : dst;
}

__global__ void __launch_bounds__(kSortThreads) digitHistogramKernel(PassArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ uint32_t counts[kRadix];
    counts[threadIdx.x] = 0;
    __syncthreads();
    const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kTile;
#pragma unroll
    for (int r = 0; r < kItems; ++r) {
        const uint64_t i = base + static_cast<uint64_t>(r) * kSortThreads + threadIdx.x;
        if (i < a.n) atomicAdd(&counts[(loadKey(a, i) >> a.shift) & 0xFFu], 1u);  // integer counters: the order is irrelevant
    }
    __syncthreads();
    a.table[static_cast<uint64_t>(threadIdx.x) * a.tiles + blockIdx.x] = counts[threadIdx.x];
}

// Exclusive prefix sum of `count` 32-bit entries in place, one CTA: every thread owns a contiguous chunk.
__global__ void __launch_bounds__(1024) tableScanKernel(uint32_t* table, uint64_t count) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ uint32_t warp_sums[32];
    const uint64_t chunk = (count + 1023) / 1024;
    const uint64_t lo = min(count, static_cast<uint64_t>(threadIdx.x) * chunk), hi = min(count, lo + chunk);
    uint32_t sum = 0;
    for (uint64_t i = lo; i < hi; ++i) sum += table[i];
    uint32_t incl = sum;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= static_cast<uint32_t>(d)) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = warp_sums[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, w, d);
            if (lane >= static_cast<uint32_t>(d)) w += v;
        }
        warp_sums[lane] = w;
    }
    __syncthreads();
    uint32_t run = incl - sum + (warp ? warp_sums[warp - 1] : 0u);
    for (uint64_t i = lo; i < hi; ++i) {
        const uint32_t v = table[i];
        table[i] = run;
        run += v;
    }
}

// Stable scatter of one tile.  Warp w owns elements [w * 32 * kItems, (w + 1) * 32 * kItems) of the tile, in kItems rounds
// of 32 consecutive elements, so "earlier in the input" means (lower warp, lower round, lower lane).
__global__ void __launch_bounds__(kSortThreads) digitScatterKernel(PassArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ uint32_t warp_counts[kSortWarps][kRadix];
    for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&warp_counts[0][0])[i] = 0;
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint64_t base = static_cast<uint64_t>(blockIdx.x) * kTile + static_cast<uint64_t>(warp) * (32 * kItems);
    uint32_t key[kItems], rank[kItems];
    float val[kItems];
#pragma unroll
    for (int r = 0; r < kItems; ++r) {
        const uint64_t i = base + static_cast<uint64_t>(r) * 32 + lane;
        const bool live = i < a.n;
        key[r] = live ? loadKey(a, i) : 0xFFFFFFFFu;
        val[r] = live ? a.vals_in[i] : 0.0f;
        const uint32_t digit = (key[r] >> a.shift) & 0xFFu;
        // lanes past the end take no part; they sit at the end of the last tile so the ranks of live lanes are unaffected
        const uint32_t live_mask = __ballot_sync(0xFFFFFFFFu, live);
        uint32_t before = 0;
        if (live) {
            const uint32_t peers = __match_any_sync(live_mask, digit);
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
    {   // per digit: exclusive prefix over the warps, plus the tile's place in the whole array
        const uint32_t d = threadIdx.x;
        uint32_t run = a.table[static_cast<uint64_t>(d) * a.tiles + blockIdx.x];
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const uint32_t c = warp_counts[w][d];
            warp_counts[w][d] = run;
            run += c;
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kItems; ++r) {
        const uint64_t i = base + static_cast<uint64_t>(r) * 32 + lane;
        if (i < a.n) {
            const uint32_t pos = warp_counts[warp][(key[r] >> a.shift) & 0xFFu] + rank[r];
            a.keys_out[pos] = key[r];
            a.vals_out[pos] = val[r];
        }
    }
}

// Sorted pairs -> output.  One thread per sorted position; a position whose destination differs from its predecessor's
// is the head of a run and owns it.  Runs of up to kShortRun updates are added by the head's thread; longer runs are
// finished by the head's whole warp, 32 consecutive loads at a time, added by lane 0 in order.
constexpr uint32_t kShortRun = 32;

__global__ void __launch_bounds__(256) applyRunsKernel(const uint32_t* keys, const float* vals, float* output, uint64_t n, uint64_t output_numel) {
    gridDependencyWait();
    gridLaunchDependents();
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint32_t lane = threadIdx.x & 31u;
    bool head = false;
    uint32_t k = 0;
    if (i < n) {
        k = keys[i];
        head = static_cast<uint64_t>(k) < output_numel && (i == 0 || keys[i - 1] != k);
    }
    float sum = 0.0f;  // the zero-filled output cell the definition starts from
    uint64_t j = i;
    bool unfinished = false;
    if (head) {
        const uint64_t stop = min(n, i + kShortRun);
        for (; j < stop && keys[j] == k; ++j) sum += vals[j];
        unfinished = j == stop && j < n && keys[j] == k;
        if (!unfinished) output[k] = sum;
    }
    // long runs, one at a time, in lane order (any order would do: the runs are independent)
    uint32_t pending = __ballot_sync(0xFFFFFFFFu, unfinished);
    while (pending) {
        const uint32_t owner = __ffs(pending) - 1u;
        pending &= pending - 1u;
        const uint32_t rk = __shfl_sync(0xFFFFFFFFu, k, owner);
        uint64_t rj = __shfl_sync(0xFFFFFFFFu, j, owner);
        float rs = __shfl_sync(0xFFFFFFFFu, sum, owner);
        bool more = true;
        while (more) {
            const uint64_t p = rj + lane;
            const bool mine = p < n && keys[p] == rk;
            const float v = mine ? vals[p] : 0.0f;
            const uint32_t in_run = __ballot_sync(0xFFFFFFFFu, mine);
            // the run continues through the leading set bits only
            const uint32_t len = in_run == 0xFFFFFFFFu ? 32u : static_cast<uint32_t>(__ffs(~in_run) - 1);
            for (uint32_t t = 0; t < len; ++t) {
                const float vt = __shfl_sync(0xFFFFFFFFu, v, t);
                rs += vt;
            }
            rj += len;
            more = len == 32u;
        }
        if (lane == owner) output[rk] = rs;
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
    while (bits < 32 && (output_numel >> bits) != 0) ++bits;  // the invalid key equals output_numel, so it must fit too
    return (bits + 7) / 8 == 0 ? 1 : (bits + 7) / 8;
}

size_t alignUp(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

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
    *bytes = 4 * alignUp(n * 4) + alignUp(tiles * kRadix * 4);
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
    for (uint32_t p = 0; p < passes; ++p) {
        a.keys_in = p == 0 ? nullptr : keys[(p - 1) & 1];
        a.vals_in = p == 0 ? static_cast<const float*>(updates) : vals[(p - 1) & 1];
        a.keys_out = keys[p & 1];
        a.vals_out = vals[p & 1];
        a.shift = 8 * p;
        TB_CUDA(launchDependent(digitHistogramKernel, dim3(tiles), dim3(kSortThreads), 0, stream, a));
        TB_CUDA(launchDependent(tableScanKernel, dim3(1), dim3(1024), 0, stream, a.table, static_cast<uint64_t>(tiles) * kRadix));
        TB_CUDA(launchDependent(digitScatterKernel, dim3(tiles), dim3(kSortThreads), 0, stream, a));
        countLaunch(3);
    }
    TB_CUDA(launchDependent(applyRunsKernel, dim3(blocks), dim3(256), 0, stream, static_cast<const uint32_t*>(keys[(passes - 1) & 1]),
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

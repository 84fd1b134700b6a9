// Device-side graph preparation: ordering an edge list for the convolution kernels without leaving the GPU and
// without a host synchronisation.
//
//   group_by_key : edges grouped by one key (receiver or sender), inside a group ordered by a second key and then by
//                  edge id.  Counting sort (histogram, exclusive scan, scatter) followed by a rank-in-segment pass, so the
//                  result does not depend on the order in which the scatter's atomics were served.
//
// Two uses: (1) oeqb_prepare_graph = the reference's CoordGraph ordering (core/ConvolutionBase.py:57-82: edges sorted by
// (row, col), transpose_perm = positions, in that list, of the edges listed by (col, row)); (2) the convolution entry
// points group an *unsorted* edge list by receiver before they launch, so the atomic variant walks a receiver's edges
// together like the deterministic one does.
//
// These kernels do not depend on the problem: they are compiled with the library, not at run time.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace gprep {

constexpr int SCAN_THREADS = 1024;
constexpr int SCAN_ITEMS = 4;                       // elements per thread
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

constexpr int STATUS_BAD_INDEX = 41;   // code stored in the status word when an index lies outside [0, n_keys)

// counts[key[e]] += 1.  An index outside [0, n_keys) is skipped (here and in the scatter) and reported through the
// status word: the lists that come out are then incomplete, but nothing is read or written out of range.
template <typename IDX>
__global__ void count_keys(const IDX* __restrict__ key, long long n, long long n_keys, int* __restrict__ counts, int* status) {
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
        const long long k = (long long)key[e];
        if (k < 0 || k >= n_keys) { *(volatile int*)status = STATUS_BAD_INDEX; continue; }
        atomicAdd(&counts[k], 1);
    }
}

// Exclusive scan of counts[0, n) into ptr[0, n], three passes: tile totals, scan of the totals (one block), tile scans.
__device__ __forceinline__ long long block_exclusive_scan(long long v, long long* total) {
    __shared__ long long warp_tot[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const long long o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        long long w = (lane < (int)(blockDim.x >> 5)) ? warp_tot[lane] : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const long long o = __shfl_up_sync(0xffffffffu, w, d);
            if (lane >= d) w += o;
        }
        warp_tot[lane] = w;   // inclusive over warps
    }
    __syncthreads();
    const long long before = (warp == 0) ? 0 : warp_tot[warp - 1];
    if (total) *total = warp_tot[(blockDim.x >> 5) - 1];
    __syncthreads();
    return before + inc - v;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_tile_totals(const int* __restrict__ counts, long long n, long long* __restrict__ tile_tot) {
    const long long base = (long long)blockIdx.x * SCAN_TILE + (long long)threadIdx.x * SCAN_ITEMS;
    long long s = 0;
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; ++i) s += (base + i < n) ? counts[base + i] : 0;
    long long total;
    block_exclusive_scan(s, &total);
    if (threadIdx.x == 0) tile_tot[blockIdx.x] = total;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_of_totals(long long* tile_tot, long long n_tiles) {
    long long carry = 0;
    for (long long base = 0; base < n_tiles; base += SCAN_THREADS) {
        const long long i = base + threadIdx.x;
        const long long v = (i < n_tiles) ? tile_tot[i] : 0;
        long long total;
        const long long ex = block_exclusive_scan(v, &total);
        if (i < n_tiles) tile_tot[i] = carry + ex;
        carry += total;
    }
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_tiles(const int* __restrict__ counts, long long n, const long long* __restrict__ tile_tot,
                                                           long long* __restrict__ ptr) {
    const long long base = (long long)blockIdx.x * SCAN_TILE + (long long)threadIdx.x * SCAN_ITEMS;
    long long c[SCAN_ITEMS], s = 0;
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; ++i) { c[i] = (base + i < n) ? counts[base + i] : 0; s += c[i]; }
    long long run = tile_tot[blockIdx.x] + block_exclusive_scan(s, nullptr);
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; ++i) {
        if (base + i < n) ptr[base + i] = run;
        run += c[i];
        if (base + i == n - 1) ptr[n] = run;
    }
}

// slot[ptr[key[e]] + (arrival number of e among its key)] = e; arrival order is arbitrary, fixed by the next pass
template <typename IDX>
__global__ void scatter_ids(const IDX* __restrict__ key, long long n, long long n_keys, const long long* __restrict__ ptr,
                            int* __restrict__ cursor, long long* __restrict__ slot) {
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
        const long long k = (long long)key[e];
        if (k < 0 || k >= n_keys) continue;
        slot[ptr[k] + atomicAdd(&cursor[k], 1)] = e;
    }
}

// One warp per key: every element of the key's segment finds its rank by (second[id], id) among the segment's elements
// and is written at that rank.  Quadratic in the segment length, which is a node degree.
// out_id[p] = edge id at sorted position p; out_key / out_second (optional) = its two keys.
template <typename IDX>
__global__ void rank_segments(const long long* __restrict__ ptr, const long long* __restrict__ slot, const IDX* __restrict__ second,
                              long long n_keys, IDX* __restrict__ out_id, IDX* __restrict__ out_key, IDX* __restrict__ out_second) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long k = warp; k < n_keys; k += n_warps) {
        const long long a = ptr[k], b = ptr[k + 1];
        for (long long t = a + lane; t < b; t += 32) {
            const long long id = slot[t];
            const long long s2 = second ? (long long)second[id] : 0;
            long long rank = 0;
            for (long long u = a; u < b; ++u) {
                const long long idu = slot[u];
                const long long su = second ? (long long)second[idu] : 0;
                rank += (su < s2 || (su == s2 && idu < id)) ? 1 : 0;
            }
            out_id[a + rank] = (IDX)id;
            if (out_key) out_key[a + rank] = (IDX)k;
            if (out_second) out_second[a + rank] = (IDX)s2;
        }
    }
}

// Checks an edge list before any kernel turns its entries into addresses: rows in [0, n_nodes), cols in [0, n_senders), rows
// non-decreasing where the kernels rely on a receiver-sorted list, transpose_perm (optional) in [0, n_edges).
// Stores STATUS_BAD_INDEX in the status word on the first violation it sees; reads only [0, n_edges) of each array.
template <typename IDX>
__global__ void validate_edges(const IDX* __restrict__ rows, const IDX* __restrict__ cols, const IDX* __restrict__ perm,
                               long long n_edges, long long n_nodes, long long n_senders, int need_sorted, int* status) {
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n_edges; e += (long long)gridDim.x * blockDim.x) {
        const long long r = (long long)rows[e], c = (long long)cols[e];
        bool bad = r < 0 || r >= n_nodes || c < 0 || c >= n_senders;
        if (need_sorted && e > 0 && (long long)rows[e - 1] > r) bad = true;
        if (perm) { const long long q = (long long)perm[e]; bad = bad || q < 0 || q >= n_edges; }
        if (bad) *(volatile int*)status = STATUS_BAD_INDEX;
    }
}

inline size_t align_up(size_t v) { return (v + 255) / 256 * 256; }

// Scratch of one group_by_key call.
inline size_t group_workspace_bytes(long long n_keys, long long n) {
    const long long tiles = (n_keys + SCAN_TILE - 1) / SCAN_TILE + 1;
    return align_up((size_t)(n_keys + 1) * 4) * 2 + align_up((size_t)tiles * 8) + align_up((size_t)(n_keys + 1) * 8) +
           align_up((size_t)(n > 0 ? n : 1) * 8);
}

struct GroupResult { long long* ptr; };

// Launches the passes on `st`.  Returns false on a launch error (cudaGetLastError holds it).
template <typename IDX>
bool group_by_key(const IDX* key, const IDX* second, long long n, long long n_keys, IDX* out_id, IDX* out_key, IDX* out_second,
                  void* workspace, int* status, cudaStream_t st, GroupResult* res, long long* launches) {
    char* w = (char*)workspace;
    int* counts = (int*)w;            w += align_up((size_t)(n_keys + 1) * 4);
    int* cursor = (int*)w;            w += align_up((size_t)(n_keys + 1) * 4);
    const long long tiles = (n_keys + SCAN_TILE - 1) / SCAN_TILE;
    long long* tile_tot = (long long*)w;  w += align_up((size_t)(tiles + 1) * 8);
    long long* ptr = (long long*)w;   w += align_up((size_t)(n_keys + 1) * 8);
    long long* slot = (long long*)w;
    // counts and cursor are adjacent: one clear
    if (cudaMemsetAsync(counts, 0, (size_t)((char*)tile_tot - (char*)counts), st) != cudaSuccess) return false;
    const unsigned eb = (unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (n > 0) { count_keys<IDX><<<eb ? eb : 1, 256, 0, st>>>(key, n, n_keys, counts, status); ++*launches; }
    if (n_keys > 0) {
        scan_tile_totals<<<(unsigned)tiles, SCAN_THREADS, 0, st>>>(counts, n_keys, tile_tot);
        scan_of_totals<<<1, SCAN_THREADS, 0, st>>>(tile_tot, tiles);
        scan_tiles<<<(unsigned)tiles, SCAN_THREADS, 0, st>>>(counts, n_keys, tile_tot, ptr);
        *launches += 3;
    }
    if (n > 0) {
        scatter_ids<IDX><<<eb ? eb : 1, 256, 0, st>>>(key, n, n_keys, ptr, cursor, slot);
        const long long warps = n_keys < 148LL * 64 ? n_keys : 148LL * 64;
        rank_segments<IDX><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(ptr, slot, second, n_keys, out_id, out_key, out_second);
        *launches += 2;
    }
    if (res) res->ptr = ptr;
    return cudaGetLastError() == cudaSuccess;
}

}  // namespace gprep

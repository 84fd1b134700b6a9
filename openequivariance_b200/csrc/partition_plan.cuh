// Device-side planning for the partitioned and the streamed convolution drivers: what a rank (or a chunk of receivers)
// needs from a globally (row, col)-sorted edge list, built without host loops.
//
// For a receiver range [n0, n1) whose rows the caller also owns as senders ("owned" range [s0, s1), may be empty):
//   e0, e1        the range of edges into the receivers (the list is sorted by receiver)
//   halo ids      the senders of those edges outside the owned range, ascending and unique
//   recv_counts   how many of them each owner q holds (owner q = nodes [bounds[q], bounds[q+1]))
//   send lists    per owner q: the owned nodes that send into q's receivers, ascending (local numbering)
//   rows / cols   of the local edges in local numbering (owned senders first, halo senders after them, in halo order)
//   interior      the longest middle run of receivers [a, b) none of whose edges has a halo sender, and its edges [ea, eb)
// Two phases, because the sizes of the lists are data: `count` marks, scans and leaves every size in one small device
// array (the caller reads it back: the only host synchronisation); `fill` writes the lists into buffers of those sizes.
// The sender-major permutation of the local list is graph_prep.cuh's group_by_key on the local columns.
//
// Reference counterpart: none (the reference has no multi-GPU path); the host version these kernels replace scanned the
// edge list once per peer with library sorts and searches.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

#include "graph_prep.cuh"

namespace pplan {

constexpr int MAX_WORLD = 64;
struct Bounds { long long b[MAX_WORLD + 1]; int world; };
// counts array: [0] e0, [1] e1, [2] n_halo, [3] a, [4] b, [5] ea, [6] eb, [7] unused, [8 + q] recv_counts, [8 + world + q] send_counts
constexpr int COUNTS_HEAD = 8;

__device__ __forceinline__ int owner_of(const Bounds& B, long long n) {
    int q = 0;
    while (q + 1 < B.world && n >= B.b[q + 1]) ++q;
    return q;
}

__global__ void init_counts(long long* counts, int n, long long E) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) counts[i] = (i < 2) ? E : 0;
}

// One pass over all edges: edge range of the receivers, halo senders, boundary receivers, and what the peers need.
__global__ void mark_edges(const long long* __restrict__ rows, const long long* __restrict__ cols, long long E, long long n0, long long n1,
                           long long s0, long long s1, const __grid_constant__ Bounds B, int rank, int* __restrict__ halo_flag,
                           int* __restrict__ send_flag, int* __restrict__ boundary_flag, long long* __restrict__ counts) {
    const long long n_owned = s1 - s0;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < E; e += (long long)gridDim.x * blockDim.x) {
        const long long r = rows[e], c = cols[e];
        const long long rp = e > 0 ? rows[e - 1] : -1;
        if (r >= n0 && rp < n0) counts[0] = e;     // lower bounds of n0 and n1 in the sorted rows (E when there is none)
        if (r >= n1 && rp < n1) counts[1] = e;
        const bool rin = r >= n0 && r < n1, cin = c >= s0 && c < s1;
        if (rin && !cin) { halo_flag[c] = 1; boundary_flag[r - n0] = 1; }
        if (cin && !rin && B.world > 1) {
            const int q = owner_of(B, r);
            if (q != rank) send_flag[(long long)q * n_owned + (c - s0)] = 1;
        }
    }
}

// One block: sizes of the lists from the scanned flags, the interior run and its edges.
__global__ void __launch_bounds__(1024) finish_counts(const long long* __restrict__ rows, const long long* __restrict__ halo_pos,
                                                      const long long* __restrict__ send_pos, const int* __restrict__ boundary_flag,
                                                      long long n_nodes, long long n0, long long n1, long long s0, long long s1,
                                                      const __grid_constant__ Bounds B, long long* __restrict__ counts) {
    __shared__ long long lo_max[32], hi_min[32];
    const long long n_recv = n1 - n0, n_owned = s1 - s0, half = n_recv / 2;
    long long a = 0, b = n_recv;   // a = 1 + last boundary receiver left of the middle, b = first one right of it
    for (long long i = threadIdx.x; i < n_recv; i += blockDim.x)
        if (boundary_flag[i]) { if (i < half) a = i + 1 > a ? i + 1 : a; else b = i < b ? i : b; }
    for (int d = 16; d > 0; d >>= 1) {
        const long long oa = __shfl_xor_sync(0xffffffffu, a, d), ob = __shfl_xor_sync(0xffffffffu, b, d);
        a = oa > a ? oa : a; b = ob < b ? ob : b;
    }
    if ((threadIdx.x & 31) == 0) { lo_max[threadIdx.x >> 5] = a; hi_min[threadIdx.x >> 5] = b; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) { a = lo_max[w] > a ? lo_max[w] : a; b = hi_min[w] < b ? hi_min[w] : b; }
        counts[2] = halo_pos[n_nodes];
        counts[3] = a; counts[4] = b;
        // edges of the interior receivers: lower bounds of n0 + a and n0 + b inside [e0, e1)
        const long long e0 = counts[0], e1 = counts[1];
        for (int which = 0; which < 2; ++which) {
            const long long target = n0 + (which ? b : a);
            long long lo = e0, hi = e1;
            while (lo < hi) { const long long mid = (lo + hi) >> 1; if (rows[mid] < target) lo = mid + 1; else hi = mid; }
            counts[5 + which] = lo - e0;
        }
    }
    for (int q = threadIdx.x; q < B.world; q += blockDim.x) {
        counts[COUNTS_HEAD + q] = halo_pos[B.b[q + 1]] - halo_pos[B.b[q]];
        counts[COUNTS_HEAD + B.world + q] = (B.world > 1 && n_owned > 0) ? send_pos[(long long)(q + 1) * n_owned] - send_pos[(long long)q * n_owned] : 0;
    }
}

// out[pos[i]] = i % period + offset for every flagged i
__global__ void compact_ids(const int* __restrict__ flag, const long long* __restrict__ pos, long long n, long long period, long long offset,
                            long long* __restrict__ out) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        if (flag[i]) out[pos[i]] = (period > 0 ? i % period : i) + offset;
}

__global__ void localize_edges(const long long* __restrict__ rows, const long long* __restrict__ cols, long long e0, long long e1, long long n0,
                               long long s0, long long s1, const long long* __restrict__ halo_pos, long long* __restrict__ rows_local,
                               long long* __restrict__ cols_local) {
    for (long long e = e0 + blockIdx.x * (long long)blockDim.x + threadIdx.x; e < e1; e += (long long)gridDim.x * blockDim.x) {
        const long long c = cols[e];
        rows_local[e - e0] = rows[e] - n0;
        cols_local[e - e0] = (c >= s0 && c < s1) ? c - s0 : (s1 - s0) + halo_pos[c];
    }
}

inline size_t align_up(size_t v) { return (v + 255) / 256 * 256; }

struct Layout {
    size_t halo_flag, halo_pos, send_flag, send_pos, boundary_flag, tiles, group, total;
};
inline Layout layout(long long n_nodes, long long n_edges, long long n_recv, long long n_owned, int world) {
    Layout L;
    const long long n_send = (world > 1 ? (long long)world * n_owned : 0);
    const long long most = n_nodes > n_send ? n_nodes : n_send;
    size_t off = 0;
    L.halo_flag = off;     off += align_up((size_t)(n_nodes + 1) * 4);
    L.send_flag = off;     off += align_up((size_t)(n_send + 1) * 4);
    L.boundary_flag = off; off += align_up((size_t)(n_recv + 1) * 4);
    L.halo_pos = off;      off += align_up((size_t)(n_nodes + 2) * 8);
    L.send_pos = off;      off += align_up((size_t)(n_send + 2) * 8);
    L.tiles = off;         off += align_up((size_t)((most + gprep::SCAN_TILE - 1) / gprep::SCAN_TILE + 2) * 8);
    L.group = off;         off += gprep::group_workspace_bytes(n_nodes, n_edges);   // keys: local senders <= n_nodes
    L.total = off;
    return L;
}

inline void scan_flags(const int* flag, long long n, long long* tile_tot, long long* pos, cudaStream_t st, long long* launches) {
    if (n <= 0) return;
    const long long tiles = (n + gprep::SCAN_TILE - 1) / gprep::SCAN_TILE;
    gprep::scan_tile_totals<<<(unsigned)tiles, gprep::SCAN_THREADS, 0, st>>>(flag, n, tile_tot);
    gprep::scan_of_totals<<<1, gprep::SCAN_THREADS, 0, st>>>(tile_tot, tiles);
    gprep::scan_tiles<<<(unsigned)tiles, gprep::SCAN_THREADS, 0, st>>>(flag, n, tile_tot, pos);
    *launches += 3;
}

inline unsigned grid_for(long long n) { const long long g = (n + 255) / 256; return (unsigned)(g < 1 ? 1 : (g > 4096 ? 4096 : g)); }

// Phase 1.  Leaves the flags and their scans in the workspace for phase 2 and the sizes in counts_dev.
inline bool count(const long long* rows, const long long* cols, long long n_nodes, long long E, long long n0, long long n1, long long s0,
                  long long s1, const Bounds& B, int rank, void* workspace, long long* counts_dev, cudaStream_t st, long long* launches) {
    const Layout L = layout(n_nodes, E, n1 - n0, s1 - s0, B.world);
    char* w = (char*)workspace;
    const long long n_send = (B.world > 1 ? (long long)B.world * (s1 - s0) : 0);
    if (cudaMemsetAsync(w + L.halo_flag, 0, L.halo_pos - L.halo_flag, st) != cudaSuccess) return false;   // the three flag arrays
    init_counts<<<1, 256, 0, st>>>(counts_dev, COUNTS_HEAD + 2 * B.world, E);
    if (E > 0)
        mark_edges<<<grid_for(E), 256, 0, st>>>(rows, cols, E, n0, n1, s0, s1, B, rank, (int*)(w + L.halo_flag), (int*)(w + L.send_flag),
                                                (int*)(w + L.boundary_flag), counts_dev);
    *launches += 2;
    scan_flags((const int*)(w + L.halo_flag), n_nodes, (long long*)(w + L.tiles), (long long*)(w + L.halo_pos), st, launches);
    scan_flags((const int*)(w + L.send_flag), n_send, (long long*)(w + L.tiles), (long long*)(w + L.send_pos), st, launches);
    finish_counts<<<1, 1024, 0, st>>>(rows, (const long long*)(w + L.halo_pos), (const long long*)(w + L.send_pos),
                                      (const int*)(w + L.boundary_flag), n_nodes, n0, n1, s0, s1, B, counts_dev);
    ++*launches;
    return cudaGetLastError() == cudaSuccess;
}

// Phase 2, with the sizes read back by the caller.  halo_ids [n_halo]; send_ids [sum of send_counts], owner by owner;
// rows_local, cols_local, perm_local [e1 - e0].
inline bool fill(const long long* rows, const long long* cols, long long n_nodes, long long E, long long n0, long long n1, long long s0,
                 long long s1, const Bounds& B, long long e0, long long e1, long long n_halo, void* workspace, long long* halo_ids,
                 long long* send_ids, long long* rows_local, long long* cols_local, long long* perm_local, int* status, cudaStream_t st,
                 long long* launches) {
    const Layout L = layout(n_nodes, E, n1 - n0, s1 - s0, B.world);
    char* w = (char*)workspace;
    const long long n_send = (B.world > 1 ? (long long)B.world * (s1 - s0) : 0);
    if (n_halo > 0 && halo_ids) {
        compact_ids<<<grid_for(n_nodes), 256, 0, st>>>((const int*)(w + L.halo_flag), (const long long*)(w + L.halo_pos), n_nodes, 0, 0, halo_ids);
        ++*launches;
    }
    if (n_send > 0 && send_ids) {
        compact_ids<<<grid_for(n_send), 256, 0, st>>>((const int*)(w + L.send_flag), (const long long*)(w + L.send_pos), n_send, s1 - s0, 0, send_ids);
        ++*launches;
    }
    if (e1 > e0) {
        localize_edges<<<grid_for(e1 - e0), 256, 0, st>>>(rows, cols, e0, e1, n0, s0, s1, (const long long*)(w + L.halo_pos), rows_local, cols_local);
        ++*launches;
        if (!gprep::group_by_key<long long>(cols_local, rows_local, e1 - e0, (s1 - s0) + n_halo, perm_local, nullptr, nullptr, w + L.group,
                                            status, st, nullptr, launches))
            return false;
    }
    return cudaGetLastError() == cudaSuccess;
}

}  // namespace pplan

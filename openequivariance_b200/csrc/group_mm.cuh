// Ragged grouped matrix products for the symmetric contraction (the op that follows the convolution in MACE).
//
// Nodes are sorted by chemical element; group g owns the consecutive nodes [off[g], off[g+1]).  With F feature channels:
//   mode 0:  C[n, f, m]    = sum_k A[g(n), f, m, k] * B[n, f, k]          (weights x node vectors)
//   mode 1:  C[g, f, m, k] = sum_{n in group g} A[n, f, m] * B[n, f, k]    (the weight gradient of mode 0)
//   mode 2:  C[n, f, k]    = sum_m A[g(n), f, m, k] * B[n, f, m]          (the vector gradient of mode 0: the transposed
//                                                                          weights applied to the output cotangent)
// The reference issues one cuBLAS strided-batched GEMM per group from a host loop
// (extension/group_mm_cuda.hpp:33-126).  Here both modes are single launches: the products are tiny (K = number of
// spherical components, 16 for l <= 3) and the op is bound by writing C (mode 0) or reading A (mode 1) once, so a
// thread owns one row m, keeps its K weights (mode 0) or K accumulators (mode 1) in registers and streams over the
// group's nodes; the node vector B[n, f, :] is the same for all threads of a block and comes from shared memory.
// Sums over nodes run in node order: mode 1 is bitwise reproducible.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace gmm {

constexpr int MAX_GROUPS = 256;
constexpr int TM = 128;      // rows m per block
constexpr int NODE_TILE = 32;

struct Offsets { long long off[MAX_GROUPS + 1]; int n_groups; };

// block = (m-tile, f, g * node_chunks + chunk): rows m0 .. m0+TM of feature f for a slice of group g's nodes
template <typename T, int KT>
__global__ void __launch_bounds__(TM) group_mm_forward(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                                                       const __grid_constant__ Offsets offs, long long F, int M, int K,
                                                       int chunks_per_group) {
    __shared__ T bs[NODE_TILE][KT];
    const int g = blockIdx.z / chunks_per_group, chunk = blockIdx.z % chunks_per_group;
    const long long f = blockIdx.y;
    const int m = blockIdx.x * TM + threadIdx.x;
    const long long n_lo = offs.off[g], n_hi = offs.off[g + 1];
    const long long span = (n_hi - n_lo + chunks_per_group - 1) / chunks_per_group;
    const long long a = n_lo + chunk * span, b = (a + span < n_hi) ? a + span : n_hi;
    if (a >= b) return;
    T w[KT];
#pragma unroll
    for (int k = 0; k < KT; ++k) w[k] = (m < M && k < K) ? A[(((long long)g * F + f) * M + m) * K + k] : T(0);
    for (long long n0 = a; n0 < b; n0 += NODE_TILE) {
        const int cnt = (int)((b - n0 < NODE_TILE) ? b - n0 : NODE_TILE);
        __syncthreads();
        for (int q = threadIdx.x; q < cnt * KT; q += TM) {
            const int r = q / KT, k = q % KT;
            bs[r][k] = (k < K) ? B[((n0 + r) * F + f) * K + k] : T(0);
        }
        __syncthreads();
        if (m < M) {
            for (int r = 0; r < cnt; ++r) {
                T acc = T(0);
#pragma unroll
                for (int k = 0; k < KT; ++k) acc += w[k] * bs[r][k];
                C[((n0 + r) * F + f) * M + m] = acc;
            }
        }
    }
}

// block = (m-tile, f, g): C[g, f, m, :] for rows m0 .. m0+TM, summed over the group's nodes in node order
template <typename T, int KT>
__global__ void __launch_bounds__(TM) group_mm_reduce(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                                                      const __grid_constant__ Offsets offs, long long F, int M, int K) {
    __shared__ T bs[NODE_TILE][KT];
    const int g = blockIdx.z;
    const long long f = blockIdx.y;
    const int m = blockIdx.x * TM + threadIdx.x;
    const long long a = offs.off[g], b = offs.off[g + 1];
    T acc[KT];
#pragma unroll
    for (int k = 0; k < KT; ++k) acc[k] = T(0);
    for (long long n0 = a; n0 < b; n0 += NODE_TILE) {
        const int cnt = (int)((b - n0 < NODE_TILE) ? b - n0 : NODE_TILE);
        __syncthreads();
        for (int q = threadIdx.x; q < cnt * KT; q += TM) {
            const int r = q / KT, k = q % KT;
            bs[r][k] = (k < K) ? B[((n0 + r) * F + f) * K + k] : T(0);
        }
        __syncthreads();
        if (m < M) {
            for (int r = 0; r < cnt; ++r) {
                const T av = A[((n0 + r) * F + f) * M + m];
#pragma unroll
                for (int k = 0; k < KT; ++k) acc[k] += av * bs[r][k];
            }
        }
    }
    if (m < M) {
        T* dst = C + (((long long)g * F + f) * M + m) * K;
        for (int k = 0; k < K; ++k) dst[k] = acc[k];
    }
}

// block = (1, f, g * node_chunks + chunk): all K columns of feature f for a slice of group g's nodes; the sum over m runs
// in tiles of MT2 rows of A held in shared memory next to the matching pieces of the nodes' B rows
constexpr int MT2 = 32;
template <typename T, int KT>
__global__ void __launch_bounds__(TM) group_mm_transposed(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                                                          const __grid_constant__ Offsets offs, long long F, int M, int K,
                                                          int chunks_per_group) {
    __shared__ T as[MT2][KT];
    __shared__ T bs[NODE_TILE][MT2 + 1];
    constexpr int PAR = TM / KT;                 // nodes handled side by side
    constexpr int ACC = NODE_TILE / PAR;         // node slots per thread
    const int g = blockIdx.z / chunks_per_group, chunk = blockIdx.z % chunks_per_group;
    const long long f = blockIdx.y;
    const int k = threadIdx.x % KT, rsub = threadIdx.x / KT;
    const long long n_lo = offs.off[g], n_hi = offs.off[g + 1];
    const long long span = (n_hi - n_lo + chunks_per_group - 1) / chunks_per_group;
    const long long a = n_lo + chunk * span, b = (a + span < n_hi) ? a + span : n_hi;
    if (a >= b) return;
    const T* Ag = A + ((long long)g * F + f) * M * K;
    for (long long n0 = a; n0 < b; n0 += NODE_TILE) {
        const int cnt = (int)((b - n0 < NODE_TILE) ? b - n0 : NODE_TILE);
        T acc[ACC];
#pragma unroll
        for (int q = 0; q < ACC; ++q) acc[q] = T(0);
        for (int m0 = 0; m0 < M; m0 += MT2) {
            const int mc = (M - m0 < MT2) ? M - m0 : MT2;
            __syncthreads();
            for (int q = threadIdx.x; q < MT2 * KT; q += TM) {
                const int mm = q / KT, kk = q % KT;
                as[mm][kk] = (mm < mc && kk < K) ? Ag[(long long)(m0 + mm) * K + kk] : T(0);
            }
            for (int q = threadIdx.x; q < NODE_TILE * MT2; q += TM) {
                const int r = q / MT2, mm = q % MT2;
                bs[r][mm] = (r < cnt && mm < mc) ? B[((n0 + r) * F + f) * M + m0 + mm] : T(0);
            }
            __syncthreads();
#pragma unroll
            for (int q = 0; q < ACC; ++q) {
                const int r = rsub + q * PAR;
                T s = acc[q];
                for (int mm = 0; mm < MT2; ++mm) s += as[mm][k] * bs[r][mm];
                acc[q] = s;
            }
        }
        if (k < K) {
#pragma unroll
            for (int q = 0; q < ACC; ++q) {
                const int r = rsub + q * PAR;
                if (r < cnt) C[((n0 + r) * F + f) * K + k] = acc[q];
            }
        }
    }
}

template <typename T, int KT>
cudaError_t launch(int mode, const Offsets& offs, long long n_nodes, long long F, int M, int K, const T* A, const T* B, T* C,
                   cudaStream_t st) {
    const unsigned mt = (unsigned)((M + TM - 1) / TM);
    if (mode == 0 || mode == 2) {
        // enough blocks to fill the machine even when one element dominates: slice every group into chunks of nodes
        const unsigned bx = mode == 0 ? mt : 1u;
        long long chunks = (148LL * 16) / ((long long)bx * F * offs.n_groups) + 1;
        const long long avg = n_nodes / (offs.n_groups > 0 ? offs.n_groups : 1) / NODE_TILE + 1;
        if (chunks > avg) chunks = avg;
        if ((long long)offs.n_groups * chunks > 65535) chunks = 65535 / offs.n_groups;
        if (chunks < 1) chunks = 1;
        const dim3 grid(bx, (unsigned)F, (unsigned)(offs.n_groups * chunks));
        if (mode == 0) group_mm_forward<T, KT><<<grid, TM, 0, st>>>(A, B, C, offs, F, M, K, (int)chunks);
        else group_mm_transposed<T, KT><<<grid, TM, 0, st>>>(A, B, C, offs, F, M, K, (int)chunks);
    } else {
        group_mm_reduce<T, KT><<<dim3(mt, (unsigned)F, (unsigned)offs.n_groups), TM, 0, st>>>(A, B, C, offs, F, M, K);
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch(int mode, const Offsets& offs, long long n_nodes, long long F, int M, int K, const void* A, const void* B,
                     void* C, cudaStream_t st) {
    const T* a = (const T*)A; const T* b = (const T*)B; T* c = (T*)C;
    if (K <= 4) return launch<T, 4>(mode, offs, n_nodes, F, M, K, a, b, c, st);
    if (K <= 8) return launch<T, 8>(mode, offs, n_nodes, F, M, K, a, b, c, st);
    if (K <= 16) return launch<T, 16>(mode, offs, n_nodes, F, M, K, a, b, c, st);
    if (K <= 32) return launch<T, 32>(mode, offs, n_nodes, F, M, K, a, b, c, st);
    return launch<T, 64>(mode, offs, n_nodes, F, M, K, a, b, c, st);
}

}  // namespace gmm

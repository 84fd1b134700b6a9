/*
 * oeq_b200 -- C ABI of the B200 (sm_100a) tensor-product / fused-convolution kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; no torch or C++ types cross this
 * boundary.  All functions return 0 on success or one of the OEQB_E* codes; oeqb_last_error() then holds a
 * message for the calling thread.  Nothing here terminates the process (the reference's backend calls
 * exit(1) on driver / NVRTC failures: extension/backend/backend_cuda.hpp:14-44).
 *
 * A problem is identified by its descriptor text (see openequivariance_b200/core/descriptor.py for the
 * grammar) and a 64-bit key chosen by the caller; the library parses the descriptor once per key,
 * specialises its kernel templates for it with NVRTC (sm_100a) on first use and caches the result, under
 * one mutex -- the role of compile_tp_with_caching / compile_conv_with_caching in
 * extension/torch_core.hpp:180-270.
 *
 * Feature rows are contiguous: x [B|N, L1_dim], y [B|E, L2_dim], z [B|N, L3_dim]; weights are in kernel
 * ("OEQ") order, [weight_numel] when shared else [B|E, weight_numel]; indices are int64 (or int32 when
 * the descriptor says so).  Element type is the descriptor's dtype (float or double).
 */
#ifndef OEQ_B200_H
#define OEQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define OEQB_API __attribute__((visibility("default")))
#else
#define OEQB_API
#endif

#define OEQB_OK 0
#define OEQB_EINVAL 1      /* bad argument (null pointer, negative size, workspace too small, misalignment) */
#define OEQB_EPARSE 2      /* malformed descriptor */
#define OEQB_ECOMPILE 3    /* NVRTC / module load failure; message holds the compiler log */
#define OEQB_ECUDA 4       /* CUDA runtime error */
#define OEQB_EUNSUPPORTED 5
#define OEQB_EKERNEL 6     /* a kernel reported a bounded wait that ran out (device status word non-zero) */

/* Size of the scratch array built into the library for oeqb_conv_backward_noalloc (64 MiB). */
#define OEQB_NOALLOC_SCRATCH_BYTES (64u << 20)

/* Mirrors KernelProp of extension/torch_core.hpp:144-178 (sizes and dtype tags the op layer validates
 * tensors against), plus which kernel family will serve the problem. */
typedef struct oeqb_kernel_prop {
    int64_t L1_dim, L2_dim, L3_dim, weight_numel;
    int32_t shared_weights;
    int32_t irrep_dtype;   /* 1 = float32, 2 = float64 */
    int32_t weight_dtype;
    int32_t idx_dtype;     /* 3 = int32, 4 = int64 */
    int32_t is_conv, deterministic, kahan;
    int32_t is_uvw;
    int32_t fast_path;     /* 1: channel-parallel TMA-pipelined kernels; 2: tcgen05 'uvw' forward; 0: general kernels */
    int32_t reserved;
} oeqb_kernel_prop;

/* Parse (and cache) a descriptor; fills *out.  Replaces the kernel_prop JSON block parsed in
 * extension/torch_core.hpp:136-178. */
OEQB_API int oeqb_query(const void* desc, size_t desc_len, int64_t key, oeqb_kernel_prop* out);

/* z = TP(x, y, W).  Replaces JITTPImpl::exec_tensor_product (extension/tensorproducts.hpp:75-85) behind
 * jit_tp_forward (extension/torch_core.hpp:274-310).  Every element of z is written. */
OEQB_API int oeqb_tp_forward(const void* desc, size_t desc_len, int64_t key, int64_t batch,
                    const void* x, const void* y, const void* W, void* z, void* stream);

/* (dx, dy, dW) for cotangent g.  Replaces JITTPImpl::backward (tensorproducts.hpp:87-95) behind
 * jit_tp_backward (torch_core.hpp:312-352).  All outputs are fully written (shared dW is zeroed here). */
OEQB_API int oeqb_tp_backward(const void* desc, size_t desc_len, int64_t key, int64_t batch,
                     const void* x, const void* y, const void* W, const void* g,
                     void* dx, void* dy, void* dW, void* stream);

/* Second-order pass.  Inputs (x, y, W, g) and the cotangents (x2, y2, W2) of (dx, dy, dW); outputs the
 * gradients w.r.t. (x, y, W, g).  Replaces JITTPImpl::double_backward (tensorproducts.hpp:97-110) behind
 * jit_tp_double_backward (torch_core.hpp:354-418). */
OEQB_API int oeqb_tp_double_backward(const void* desc, size_t desc_len, int64_t key, int64_t batch,
                            const void* x, const void* y, const void* W, const void* g,
                            const void* x2, const void* y2, const void* W2,
                            void* dx, void* dy, void* dW, void* dg, void* stream);

/* Bytes of scratch the convolution entry points need for a graph of n_nodes / n_edges.
 * direction: 0 forward, 1 backward, 2 double backward.  The reference sizes its workspace at construction
 * from its launch geometry (core/LoopUnrollConv.py:142-185); here it depends on the graph size, so the
 * caller asks per call.  Returns a negative OEQB_E* code on error. */
OEQB_API int64_t oeqb_conv_workspace_bytes(const void* desc, size_t desc_len, int64_t key, int direction,
                                  int64_t n_nodes, int64_t n_edges);

/* Z[n] = sum over edges e with rows[e] == n of TP(X[cols[e]], Y[e], W[e]).
 * Atomic descriptors: any edge order, Z must be zero on entry.  Deterministic descriptors: edges sorted by
 * (row, col); every row of Z is written exactly once (no zeroing needed), results are bitwise reproducible
 * and independent of launch geometry.  Replaces JITConvImpl::exec_conv + fixup_forward
 * (extension/convolution.hpp:78-107) behind jit_conv_forward (torch_core.hpp:422-476). */
OEQB_API int oeqb_conv_forward(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                      const void* X, const void* Y, const void* W, void* Z,
                      const void* rows, const void* cols, const void* transpose_perm,
                      void* workspace, int64_t workspace_bytes, void* stream);

/* oeqb_conv_forward for callers whose X has another number of rows than Z (no counterpart in the reference, whose
 * X and Z always share the node count): n_nodes receivers = rows of Z, n_senders = rows of X.  The partitioned and
 * the streamed drivers of this library call it with a block of gathered sender rows.  The only difference is the
 * bound the index check applies to cols. */
OEQB_API int oeqb_conv_forward_rect(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_senders,
                           int64_t n_edges, const void* X, const void* Y, const void* W, void* Z,
                           const void* rows, const void* cols, const void* transpose_perm,
                           void* workspace, int64_t workspace_bytes, void* stream);

/* Gradients of the convolution.  G is dL/dZ [n_nodes, L3_dim].  dX [n_nodes, L1_dim], dY, dW like Y, W.
 * Deterministic descriptors need transpose_perm (position in the row-major edge list of the k-th edge in
 * column-major order) and a symmetric edge set is NOT required by this library.  All outputs are fully
 * written.  Replaces JITConvImpl::backward + fixup_backward (convolution.hpp:109-136) behind
 * jit_conv_backward (torch_core.hpp:478-540). */
OEQB_API int oeqb_conv_backward(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                       const void* X, const void* Y, const void* W, const void* G,
                       void* dX, void* dY, void* dW,
                       const void* rows, const void* cols, const void* transpose_perm,
                       void* workspace, int64_t workspace_bytes, void* stream);

/* oeqb_conv_backward for callers whose G has another number of rows than X (companion of oeqb_conv_forward_rect, no
 * counterpart in the reference): n_receivers = rows of G (bound of `rows`), n_nodes = rows of X and dX (bound of
 * `cols`). */
OEQB_API int oeqb_conv_backward_rect(const void* desc, size_t desc_len, int64_t key, int64_t n_receivers, int64_t n_nodes,
                            int64_t n_edges, const void* X, const void* Y, const void* W, const void* G,
                            void* dX, void* dY, void* dW,
                            const void* rows, const void* cols, const void* transpose_perm,
                            void* workspace, int64_t workspace_bytes, void* stream);

/* The deterministic backward pass in two steps, for callers that need some rows of dX before the others (no counterpart in
 * the reference): oeqb_conv_backward_edges runs the per-edge pass (dY, dW, and the per-edge dX rows into the workspace);
 * oeqb_conv_backward_rows then sums the workspace rows of the senders [row_begin, row_end) into dX, and may be called
 * several times with disjoint ranges, in any order, on the same stream or on streams ordered after the edge pass.  The
 * partitioned driver reduces the rows it sends back to other GPUs first and overlaps their transfer with the rest.
 * Together the calls give exactly oeqb_conv_backward_rect's result.  Only for deterministic descriptors that oeqb_query
 * reports as fast_path = 1 (others: OEQB_EUNSUPPORTED, use oeqb_conv_backward_rect); workspace as for that call. */
OEQB_API int oeqb_conv_backward_edges(const void* desc, size_t desc_len, int64_t key, int64_t n_receivers, int64_t n_nodes,
                             int64_t n_edges, const void* X, const void* Y, const void* W, const void* G,
                             void* dY, void* dW,
                             const void* rows, const void* cols, const void* transpose_perm,
                             void* workspace, int64_t workspace_bytes, void* stream);
OEQB_API int oeqb_conv_backward_rows(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                            int64_t row_begin, int64_t row_end, const void* transpose_perm,
                            void* workspace, int64_t workspace_bytes, void* dX, void* stream);

/* Allocation-free variant of oeqb_conv_backward for deterministic convolutions on the channel-parallel kernels.
 * It has no counterpart in the reference.
 *
 * Who needs it: hosts that may not allocate device memory at the point where they call us -- a solver or serving
 * runtime that has already handed all device memory to its own arena, or a step that must not provoke the implicit
 * device-wide synchronisation that cudaMalloc / cudaFree perform.  Such callers cannot give us a workspace, and we
 * must not create one.  The per-edge gradient rows and the sender offsets therefore live in a fixed array compiled
 * into the library (OEQB_NOALLOC_SCRATCH_BYTES, held by every GPU that loads the library until the process ends).
 *
 * Limits and rules:
 *   - n_edges * L1_dim * 4 (rounded up to 256) + (n_nodes + 1) * 8 (rounded up to 256) + 256 bytes must fit in
 *     OEQB_NOALLOC_SCRATCH_BYTES; larger graphs are refused with OEQB_EINVAL and a message giving both numbers.
 *   - Only descriptors with deterministic = 1 that oeqb_query reports as fast_path = 1; others get OEQB_EUNSUPPORTED.
 *   - The first call for a problem on a device does one-time set-up (looks up the array's device address, specialises
 *     and loads the kernels).  Make that call before entering any stream capture; later calls do no set-up.
 *   - No cudaMalloc / cudaFree / allocator call is made, on any call.  All calls share the one array, and it keeps the
 *     previous call's contents: the library re-zeroes the one word that must start at zero and overwrites the rest.
 *     Two calls whose kernels overlap on the GPU (different streams, or different host threads) race on the array.
 *   - Results are the same as oeqb_conv_backward's, bit for bit.  A kernel wait that runs out is recorded in the last
 *     word of the array; oeqb_noalloc_status (below) reads it. */
OEQB_API int oeqb_conv_backward_noalloc(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                               const void* X, const void* Y, const void* W, const void* G,
                               void* dX, void* dY, void* dW,
                               const void* rows, const void* cols, const void* transpose_perm, void* stream);

/* Companion of oeqb_conv_backward_noalloc (no counterpart in the reference either): reports whether a kernel of the
 * last allocation-free call on the current device abandoned a bounded wait.  Call it after synchronising with the
 * stream that call ran on.  It copies one 4-byte word out of the built-in array (a blocking copy; nothing is
 * allocated) and returns OEQB_OK or OEQB_EKERNEL; the word is cleared by the next oeqb_conv_backward_noalloc call. */
OEQB_API int oeqb_noalloc_status(void);

/* Second-order pass of the convolution; argument meaning as oeqb_tp_double_backward with node-level X, X2,
 * dX, G, dG.  Replaces JITConvImpl::double_backward (convolution.hpp:138-176) behind
 * jit_conv_double_backward (torch_core.hpp:542-622). */
OEQB_API int oeqb_conv_double_backward(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                              const void* X, const void* Y, const void* W, const void* G,
                              const void* X2, const void* Y2, const void* W2,
                              void* dX, void* dY, void* dW, void* dG,
                              const void* rows, const void* cols, const void* transpose_perm,
                              void* workspace, int64_t workspace_bytes, void* stream);

/* Orders an edge list for the convolution on the device, without a host synchronisation.  rows / cols [n_edges]
 * (idx_dtype 3 = int32, 4 = int64, values in [0, n_nodes)) in any order.  Outputs, same index type, [n_edges] each:
 * order (the permutation that sorts the edges by (row, col); apply it to per-edge tensors such as Y and W),
 * sorted_rows / sorted_cols (the sorted list) and transpose_perm (positions, in the sorted list, of the edges
 * listed by (col, row)): exactly the arrays of the reference's CoordGraph (core/ConvolutionBase.py:57-82, which
 * sorts a Python list on the host).  Duplicate edges keep their input order.  workspace: device scratch of at least
 * oeqb_graph_workspace_bytes(n_nodes, n_edges) bytes, 16-byte aligned.  An index out of range is skipped (nothing is
 * read or written out of bounds) and reported by the next call of this library or by oeqb_check_status. */
OEQB_API int64_t oeqb_graph_workspace_bytes(int64_t n_nodes, int64_t n_edges);
OEQB_API int oeqb_prepare_graph(int idx_dtype, int64_t n_nodes, int64_t n_edges, const void* rows, const void* cols,
                                void* sorted_rows, void* sorted_cols, void* order, void* transpose_perm,
                                void* workspace, int64_t workspace_bytes, void* stream);

/* Ragged grouped products of the symmetric contraction.  Nodes are sorted by group (chemical element); group g has
 * ragged_counts[g] consecutive nodes (a HOST array of num_groups entries, as in the reference, which takes the
 * bincount on the CPU).  dtype 1 = float32, 2 = float64; F = num_features.
 *   ragged_inner = 0:  C[n, f, m]    = sum_k A[g(n), f, m, k] * B[n, f, k]      A [G, F, M, K], B [N, F, K], C [N, F, M]
 *   ragged_inner = 1:  C[g, f, m, k] = sum_{n in g} A[n, f, m] * B[n, f, k]      A [N, F, M], B [N, F, K], C [G, F, M, K]
 *   ragged_inner = 2:  C[n, f, k]    = sum_m A[g(n), f, m, k] * B[n, f, m]      A [G, F, M, K], B [N, F, M], C [N, F, K]
 *                      (mode 0 with the weights transposed, without materialising the transpose: its vector gradient)
 * All row-major and contiguous; C is fully written (zeros for empty groups).  The sum over nodes runs in node order
 * (bitwise reproducible).  Limits: K <= 64, at most 256 groups.  Replaces GroupMMCUDA::group_gemm
 * (extension/group_mm_cuda.hpp:33-126: one cuBLAS strided-batched GEMM per group from a host loop). */
OEQB_API int oeqb_group_mm(int dtype, int ragged_inner, int64_t num_groups, int64_t num_features, int64_t M, int64_t K,
                           const int64_t* ragged_counts, const void* A, const void* B, void* C, void* stream);

/* Kernels of this library report run-time failures (a bounded wait that ran out, an index out of range) through a
 * host-visible word per device that the next entry-point call inspects.  This call inspects it now: after the
 * caller has synchronised with the stream, it tells whether the work issued so far on the current device failed.
 * Returns OEQB_OK, OEQB_EKERNEL or OEQB_EINVAL and clears the word.  The reference exits the process on a device
 * error instead (extension/backend/backend_cuda.hpp:30-46). */
OEQB_API int oeqb_check_status(void);

/* How many calls so far took a slower route than the problem's specialised kernels (operands that are not 16-byte
 * aligned, no workspace for grouping an unsorted edge list).  With the "log" option each one is also printed. */
OEQB_API int64_t oeqb_slow_path_count(void);

/* Writes the CUDA source the library would hand to NVRTC for `kind` (a kernel-family name such as
 * "generic_forward") into buf (NUL-terminated, truncated to cap); *needed receives the full length
 * including the NUL.  Lets the specialised source be inspected or compiled offline with nvcc.  Plays the
 * part of the kernel string the reference exposes as TensorProduct.jit_kernel (core/LoopUnrollTP.py:93-99). */
OEQB_API int oeqb_emit_source(const void* desc, size_t desc_len, const char* kind, char* buf, size_t cap, size_t* needed);

/* Compile every kernel family of a descriptor now (works without a GPU) and keep the cubins in the on-disk
 * cache directory, so later processes skip NVRTC.  Returns the number of programs compiled, or a negative
 * OEQB_E* code.  Equivalent in purpose to the reference's eager JIT in the JITTPImpl / JITConvImpl
 * constructors (tensorproducts.hpp:32-46, convolution.hpp:36-56). */
OEQB_API int oeqb_precompile(const void* desc, size_t desc_len, int64_t key);

/* Planning for the partitioned / streamed convolution drivers, on the device (csrc/partition_plan.cuh).  From a globally
 * (row, col)-sorted int64 edge list: what the holder of receivers [recv_begin, recv_end), who owns the rows
 * [own_begin, own_end) as senders (may be empty), needs.  `bounds` [world + 1] are the owners' node ranges (NULL = one
 * owner).  No reference counterpart: the reference has no multi-GPU path.
 *
 * oeqb_plan_count leaves in `counts` (device, int64 [8 + 2 world]): [0] e0, [1] e1 (edges into the receivers), [2] number
 * of halo senders (senders of those edges outside the owned range), [3] a, [4] b (longest middle run of receivers without a
 * halo sender, relative to recv_begin), [5] ea, [6] eb (its edges, relative to e0), [8 + q] halo senders owned by q,
 * [8 + world + q] owned nodes that owner q's receivers read.  The caller reads them back (the one synchronisation),
 * allocates, and calls oeqb_plan_fill with the same arguments and workspace: halo_ids [n_halo] ascending, send_ids
 * (concatenated by owner, local numbering, ascending), rows_local / cols_local [e1 - e0] (owned senders first, halo senders
 * after them in halo order) and perm_local (the sender-major order of the local list).  Any output pointer may be NULL
 * when its size is zero. */
OEQB_API int64_t oeqb_plan_workspace_bytes(int64_t n_nodes, int64_t n_edges, int64_t n_receivers, int64_t n_owned, int32_t world);
OEQB_API int oeqb_plan_count(int64_t n_nodes, int64_t n_edges, const void* rows, const void* cols, int64_t recv_begin,
                             int64_t recv_end, int64_t own_begin, int64_t own_end, int32_t world, int32_t rank,
                             const int64_t* bounds, void* workspace, int64_t workspace_bytes, int64_t* counts, void* stream);
OEQB_API int oeqb_plan_fill(int64_t n_nodes, int64_t n_edges, const void* rows, const void* cols, int64_t recv_begin,
                            int64_t recv_end, int64_t own_begin, int64_t own_end, int32_t world, const int64_t* bounds,
                            int64_t e0, int64_t e1, int64_t n_halo, void* workspace, int64_t workspace_bytes, void* halo_ids,
                            void* send_ids, void* rows_local, void* cols_local, void* perm_local, void* stream);

/* Self-test of the kernels' bounded waits (every spin on a barrier in the pipelined kernels gives up after ~2 s, raises its
 * CTA's abort flag and stores a code in a host-mapped status word): launches one small CTA that waits for a barrier nobody
 * arrives at and checks that it returns by itself, that all threads leave and that the code arrives.  Takes ~2 s.  The
 * descriptor must be one the channel-parallel kernels serve (fast_path = 1).  Returns OEQB_OK when the mechanism works and
 * leaves the status word clear. */
OEQB_API int oeqb_selftest_bounded_wait(const void* desc, size_t desc_len, int64_t key, void* stream);

/* String options: "cache_dir" (cubin cache directory), "log" ("0"/"1"), "validate" ("0"/"1"/"2": index checks), and the
 * tuning aids "force_generic", "single_group", "single_producer", "no_tc", "tc_backward" ("0".."7"), "streams",
 * "streams_forward".  Unknown names are refused with OEQB_EINVAL. */
OEQB_API int oeqb_set_option(const char* name, const char* value);

/* Number of kernel launches issued by this library since load (all threads). */
OEQB_API int64_t oeqb_launch_count(void);

/* Message of the last failure on the calling thread ("" if none). */
OEQB_API const char* oeqb_last_error(void);

/* Library version string. */
OEQB_API const char* oeqb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* OEQ_B200_H */

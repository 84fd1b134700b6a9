// 'uvw' forward on the 5th-generation tensor cores (tcgen05) for shared weights, 32-wide multiplicities, fp32.
//
//   z[b, o][w, k] = sum over paths p into output block o, channels u:   W_p[u, w] * T_p[b][u, k]
//   T_p[b][u, k]  = sum_{i,j} C_p[i, j, k] x[b, a(p)][u, i] y[b][j]           (Clebsch-Gordan stage, CUDA cores)
//
// For a tile of 128 batch items and one output component (o, k) the u -> w contraction of all paths into o is a
// GEMM  D[128 items, 32 w] += A_p,k[128 items, 32 u] * B_p[32 u, 32 w]  accumulated over the paths p: A is produced by
// the CG stage straight into shared memory in the tensor core's canonical K-major layout, B is the path's weight
// block, D lives in tensor memory (TMEM).  fp32 accuracy comes from the 3xTF32 split: every operand is written as
// hi = tf32(v), lo = tf32(v - hi) and each product is issued as hi*hi + lo*hi + hi*lo, accumulated in fp32.
// Reference counterpart: the scalar-FMA warp matmul of templates/wmm.cuh:1-87 driven from loop_unroll_tp.cuh:55-61.
//
// Thread roles in a CTA of 256 threads (one CTA per SM, all 512 TMEM columns):
//   all threads : stage the path's input block in shared memory; CG stage + hi/lo split of one A chunk (16 elements
//                 each) per step; weight block at a path's start
//   thread 0    : issues the 12 tcgen05.mma of a step (4 k-steps x 3 split terms), commits to an mbarrier
//   all warps   : epilogue of an output block: tcgen05.ld of the accumulators, stores to z
// A and B chunks are double buffered; the accumulators of consecutive output blocks alternate between two TMEM halves.
// Every mbarrier wait is bounded; on time-out the CTA leaves after releasing its TMEM.
#pragma once
#if OEQ_TC

// TC_MODE (with the tables): 0 forward, 1 gradient of x, 2 gradient of y, 3 gradient of the weights.
struct TcParams {
    const float* x; const float* y; const float* W; float* z;
    const float* g;     // mode 2 only: the output cotangent (x is then the first input, z the gradient of y)
    long long batch;
    int accum;          // add to what z holds instead of overwriting it
    int* status;
};

OEQ_DEV unsigned tc_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
OEQ_DEV void tc_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem_u32(bar)), "r"(count) : "memory");
}
OEQ_DEV bool tc_mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(tc_smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
OEQ_DEV unsigned long long tc_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
OEQ_DEV bool tc_mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int* status, int code) {
    if (tc_mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = tc_global_ns();
    for (unsigned spin = 0;; ++spin) {
        if (tc_mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u) {
            if (*abort_flag) return false;
            if (tc_global_ns() - t0 > 2000000000ull) { *abort_flag = 1; *(volatile int*)status = code; return false; }
        }
    }
}
// Asynchronous copies global -> shared (16 or 4 bytes; nothing is read and zeros are written when !live): a staging
// loop issues all of its copies back to back and waits once, so their latencies overlap.
OEQ_DEV void tc_cp16(void* dst_smem, const void* src, bool live) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tc_smem_u32(dst_smem)), "l"(src), "r"(live ? 16u : 0u) : "memory");
}
OEQ_DEV void tc_cp4(void* dst_smem, const void* src, bool live) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(tc_smem_u32(dst_smem)), "l"(src), "r"(live ? 4u : 0u) : "memory");
}
OEQ_DEV void tc_cp_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// One row by a bulk copy (TMA, untiled): 16-byte aligned addresses, a multiple of 16 bytes; completion is counted in
// bytes on the mbarrier.
OEQ_DEV void tc_bulk_row(void* dst_smem, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc_smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(tc_smem_u32(bar)) : "memory");
}
OEQ_DEV void tc_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(tc_smem_u32(bar)), "r"(bytes) : "memory");
}
OEQ_DEV float tc_tf32(float v) {   // round to tf32 (10-bit mantissa), result is a valid fp32 bit pattern
    unsigned r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; LBO = distance between core
// matrices adjacent in K, SBO = distance between 8-row groups.  Bits: [0,14) address>>4, [16,30) LBO>>4,
// [32,46) SBO>>4, [46,48) descriptor version 1, [61,64) swizzle mode 0.
OEQ_DEV unsigned long long tc_desc(const void* smem, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((tc_smem_u32(smem) & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    return d;
}
// Instruction descriptor for kind::tf32, fp32 accumulate, both operands K-major, M = 128, N = 32:
// [4,6) D format 1 = f32, [7,10) A format 2 = tf32, [10,13) B format 2 = tf32, [17,23) N>>3, [24,29) M>>4.
constexpr unsigned TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);

OEQ_DEV void tc_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p; }"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(TC_IDESC), "r"(accumulate) : "memory");
}
OEQ_DEV void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem_u32(bar)) : "memory");
}
OEQ_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
OEQ_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
OEQ_DEV void tc_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// A / B chunk geometry: 32 K-columns = 8 core matrices of 128 bytes per 8-row group
constexpr unsigned TC_LBO = 128, TC_SBO = 1024;
constexpr int TC_A_FLOATS = 128 * 32, TC_B_FLOATS = 32 * 32;
// padded row of the staged input block: conflict-free for the column reads of the Clebsch-Gordan stage (modes 0, 1) or
// for one thread per row (mode 2)
constexpr int TC_XSTRIDE = 32 * TC_MAXD1 + (TC_MODE == 2 ? 1 : 4);
constexpr int TC_XSTRIDE2 = 32 * TC_XS2_D1 + 4;  // row of the second staging buffer (blocks of up to TC_XS2_D1 components)
constexpr int TC_DYS = L2_DIM | 1;              // mode 2: row of a thread's partial sums of dy
constexpr int TC_YSTRIDE = (L2_DIM + 3) & ~3;
constexpr int TC_CW = 16;                       // compute warps
constexpr int TC_CT = 32 * TC_CW;               // compute threads
constexpr int TC_THREADS = TC_CT + 32;          // ... and the warp that issues the MMAs
constexpr int TC_EC = 128 / TC_CW;              // channels (accumulator columns) of one thread in an epilogue

struct __align__(128) TcShared {
    float a[2][2][TC_A_FLOATS];       // [buffer][hi, lo]
    float b[2][2][TC_B_FLOATS];
    float xs[128 * TC_XSTRIDE];       // input block a(p) of the 128 items of the tile
    float xs2[TC_XS2_D1 > 0 ? 128 * TC_XSTRIDE2 : 4];   // second staging buffer: the next block arrives while this one is read
    float ys[TC_MODE == 2 ? 4 : 128 * TC_YSTRIDE];   // harmonics of the 128 items (mode 2 does not read them)
    float dys[TC_MODE == 2 ? TC_CT * TC_DYS : 4];   // mode 2: per-thread partial sums of dy (TC_CW / 4 threads per item)
    unsigned long long a_full[2];     // the operands of a step are in place (every compute warp arrives once)
    unsigned long long mma_done[2];   // a buffer may be rewritten
    unsigned long long acc_done[2];   // accumulators of an output block are complete
    unsigned long long xs_full[2];    // a staged input block has arrived (bytes of the bulk copies), per staging buffer
    unsigned tmem_base;
    int abort_flag;
};
// One CTA per SM is assumed (it owns all of TMEM): the host asks for more than half of the shared memory even when the
// buffers need less.
static_assert(sizeof(TcShared) <= 232448, "the buffers exceed shared memory");

// offset (in floats) of element (row, kcol) in a chunk
OEQ_DEV int tc_elem(int row, int kcol) { return (row >> 3) * (TC_SBO / 4) + (kcol >> 2) * (TC_LBO / 4) + (row & 7) * 4 + (kcol & 3); }
OEQ_DEV void tc_mbar_arrive(unsigned long long* bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(tc_smem_u32(bar)) : "memory");
}
OEQ_DEV void tc_compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(TC_CT) : "memory"); }   // the compute warps only
// eight consecutive accumulator columns of this thread's TMEM lane
OEQ_DEV void tc_ld8(unsigned taddr, unsigned (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Epilogue of one output block for one thread: its item's TC_EC output channels x D3 components are TC_EC * D3 consecutive
// floats of the z row.  All components are pulled out of tensor memory first (column 32 k + c holds channel c of
// component k), then written as 16-byte stores, so every 32-byte sector of z is written whole.
template <int D3>
OEQ_DEV void tc_epilogue(unsigned tbase, float* zdst, bool live, bool accum) {
    float v[TC_EC * D3];   // v[c * D3 + k]
#pragma unroll
    for (int k = 0; k < D3; ++k) {
        unsigned r[8];
        tc_ld8(tbase + 32u * (unsigned)k, r);
#pragma unroll
        for (int c = 0; c < TC_EC; ++c) v[c * D3 + k] = __uint_as_float(r[c]);
    }
    if (live) {
        float4* dst = reinterpret_cast<float4*>(zdst);   // 32 * D3 bytes from a 16-byte boundary
        if (accum) {
#pragma unroll
            for (int q = 0; q < 2 * D3; ++q) {
                const float4 old = dst[q];
                v[4 * q] += old.x; v[4 * q + 1] += old.y; v[4 * q + 2] += old.z; v[4 * q + 3] += old.w;
            }
        }
#pragma unroll
        for (int q = 0; q < 2 * D3; ++q) __stcs(dst + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
    }
}
static_assert(TC_EC == 8, "the epilogues read eight accumulator columns per thread");

#if TC_MODE != 3
// Clebsch-Gordan stage of one step for one thread: its 8 channels are 4 * D1 floats apart in the staged row (D1 at
// compile time makes those offsets immediates).
template <int D1>
OEQ_DEV void tc_cg(const float* xrow, const float* yrow, int t0, int t1, float (&acc)[8]) {
    for (int t = t0; t < t1; ++t) {
        const float cy = TC_TC[t] * yrow[TC_TJ[t]];
        const float* px = xrow + TC_TI[t];
#pragma unroll
        for (int uu = 0; uu < 8; ++uu) acc[uu] = fmaf(cy, px[uu * 4 * D1], acc[uu]);
    }
}

// The loops over paths, output components and Clebsch-Gordan terms are run-time loops over the TC_* tables of the
// problem header (not unrolled): the whole kernel is a few KB of code and stays in the instruction cache.
// The same kernel computes the gradient of the first input when it is compiled with the transposed tables (TC_WT = 1:
// x is then the output cotangent, z the gradient, and the weight block is applied transposed), and the gradient of the
// second input (mode 2); TC_KERNEL_NAME, TC_IN_DIM and TC_OUT_DIM (row lengths of x and z) come with the tables.
//
// Sixteen compute warps and one warp that issues the MMAs.  The compute warps never meet the issuing warp at a CTA-wide
// barrier: a step's operands are handed over through the a_full mbarrier (every compute thread arrives after its
// stores), buffers come back through mma_done, finished accumulators through acc_done (tcgen05.commit).  The compute
// warps meet among themselves (named barrier) only where the staged input block changes hands.  A thread that gave up
// keeps walking the loops and joining those barriers without doing work, so nobody waits for it.
extern "C" __global__ void __launch_bounds__(TC_THREADS, 1) TC_KERNEL_NAME(const TcParams p) {
    extern __shared__ __align__(128) unsigned char tc_smem_raw[];
    TcShared& sh = *reinterpret_cast<TcShared*>(tc_smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    volatile int* abortf = &sh.abort_flag;
    if (tid == 0) {
        tc_mbar_init(&sh.a_full[0], TC_CW); tc_mbar_init(&sh.a_full[1], TC_CW);   // one arrival per compute warp
        tc_mbar_init(&sh.mma_done[0], 1); tc_mbar_init(&sh.mma_done[1], 1);
        tc_mbar_init(&sh.acc_done[0], 1); tc_mbar_init(&sh.acc_done[1], 1);
        tc_mbar_init(&sh.xs_full[0], 1); tc_mbar_init(&sh.xs_full[1], 1);
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(tc_smem_u32(&sh.tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = sh.tmem_base;
    const long long ntiles = (p.batch + 127) / 128;
    unsigned step = 0;     // chunk steps so far: operand buffer = step & 1
    unsigned npath = 0;    // paths started so far: weight buffer = npath & 1
    unsigned nblock = 0;   // output blocks finished so far: accumulator half = nblock & 1
    bool dead = false;

    if (warp == TC_CW) {
        // ---- the issuing warp: for every step, wait for its operands, issue 12 MMAs (4 k-steps x 3 split terms), commit.
        // The operand descriptors are built once; a k-step further along K is 256 bytes (16 in the address field) on.
        const unsigned long long da0h = tc_desc(&sh.a[0][0][0], TC_LBO, TC_SBO), da0l = tc_desc(&sh.a[0][1][0], TC_LBO, TC_SBO);
        const unsigned long long da1h = tc_desc(&sh.a[1][0][0], TC_LBO, TC_SBO), da1l = tc_desc(&sh.a[1][1][0], TC_LBO, TC_SBO);
        const unsigned long long db0h = tc_desc(&sh.b[0][0][0], TC_LBO, TC_SBO), db0l = tc_desc(&sh.b[0][1][0], TC_LBO, TC_SBO);
        const unsigned long long db1h = tc_desc(&sh.b[1][0][0], TC_LBO, TC_SBO), db1l = tc_desc(&sh.b[1][1][0], TC_LBO, TC_SBO);
        for (long long tile = blockIdx.x; tile < ntiles && !dead; tile += gridDim.x) {
            for (int q = 0; q < TC_NPATH && !dead; ++q) {
                const int d3 = TC_D3[q], first = TC_FIRST[q], last = TC_LAST[q];
                for (int k = 0; k < d3 && !dead; ++k) {
                    const unsigned buf = step & 1u;
                    if (!tc_mbar_wait(&sh.a_full[buf], (step >> 1) & 1u, abortf, p.status, 35)) { dead = true; break; }
                    tc_fence_after();
                    if (lane == 0) {
                        const unsigned bbuf = npath & 1u;
                        const unsigned dcol = tmem + (nblock & 1u) * 256u + 32u * (unsigned)k;
                        const unsigned long long ah0 = buf ? da1h : da0h, al0 = buf ? da1l : da0l;
                        const unsigned long long bh0 = bbuf ? db1h : db0h, bl0 = bbuf ? db1l : db0l;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const unsigned long long ah = ah0 + 16ull * ks, al = al0 + 16ull * ks;
                            const unsigned long long bh = bh0 + 16ull * ks, bl = bl0 + 16ull * ks;
                            tc_mma(dcol, ah, bh, (first && ks == 0) ? 0u : 1u);
                            tc_mma(dcol, al, bh, 1u);
                            tc_mma(dcol, ah, bl, 1u);
                        }
                        tc_commit(&sh.mma_done[buf]);
                        if (last && k == d3 - 1) tc_commit(&sh.acc_done[nblock & 1u]);
                    }
                    __syncwarp();
                    ++step;
                }
                if (last) ++nblock;
                ++npath;
            }
        }
    } else {
        // ---- compute warps.  This thread's 8 elements of every A chunk: item brow, channels ucol + 4 * uu, uu < 8
        const int brow = warp * 8 + (lane >> 2);
        const int ucol = lane & 3;
        unsigned nfill[2] = {0u, 0u};   // blocks that have arrived in each staging buffer so far (phases of xs_full)
        int cur = 0;                    // staging buffer that holds the block of the path at hand
        float gnext[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // mode 2: the next step's cotangent values
        float wnext[1024 / TC_CT];                                    // this thread's entries of the next path's weight block
#pragma unroll
        for (int r = 0; r < 1024 / TC_CT; ++r) wnext[r] = __ldg(p.W + TC_WOFF[0] + tid + TC_CT * r);
        for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const long long item0 = tile * 128;
            int pre_q = -1;      // path whose block has been requested ahead (none across tiles)
            tc_compute_sync();   // previous tile's readers of xs / ys / dys are done
            if (TC_MODE != 2) {
                for (int r = warp; r < 128; r += TC_CW)          // one warp per row: no index division
                    for (int j = lane; j < L2_DIM; j += 32)
                        sh.ys[r * TC_YSTRIDE + j] = (item0 + r < p.batch) ? __ldg(p.y + (item0 + r) * L2_DIM + j) : 0.f;
            } else {
                for (int j = 0; j < TC_DYS; ++j) sh.dys[tid * TC_DYS + j] = 0.f;   // read and written by this thread only
            }
            for (int q = 0; q < TC_NPATH; ++q) {
                const int d1 = TC_D1[q], d3 = TC_D3[q], xoff = TC_XOFF[q], zoff = TC_ZOFF[q], woff = TC_WOFF[q];
                const int tq = TC_INS[q] * 8;   // this path's instruction: start of its term ranges
                const int last = TC_LAST[q];
                // stage the path's input block by asynchronous row copies; the block stays when the previous path of this
                // tile read the same one
                const bool restage = q == 0 || TC_XOFF[q - 1] != xoff;
                tc_compute_sync();   // readers of the previous path's block are done
                if (TC_MODE != 2) {
                    // One bulk copy per row, issued by the first 128 threads; everybody waits for the bytes to arrive.  Rows past
                    // the end of the batch read row 0: their results are never stored.  While this block is read, the next
                    // different one of the tile's schedule is already requested into the other staging buffer when that
                    // buffer can hold it (its readers left before the barrier above).
                    auto request = [&](int buf, int qq) {
                        const int dd = TC_D1[qq];
                        if (tid == 0) tc_mbar_expect_tx(&sh.xs_full[buf], 128u * 128u * (unsigned)dd);
                        if (tid < 128) {
                            const long long b = item0 + tid;
                            float* dst = buf ? sh.xs2 + tid * TC_XSTRIDE2 : sh.xs + tid * TC_XSTRIDE;
                            tc_bulk_row(dst, p.x + (b < p.batch ? b : 0) * TC_IN_DIM + TC_XOFF[qq], 128u * (unsigned)dd, &sh.xs_full[buf]);
                        }
                    };
                    if (restage && !dead) {
                        if (pre_q == q) cur ^= 1;
                        else { cur = 0; request(0, q); }
                        if (!tc_mbar_wait(&sh.xs_full[cur], nfill[cur] & 1u, abortf, p.status, 37)) dead = true;
                        ++nfill[cur];
                        const int qn = TC_NEXTX[q];   // first later path of the schedule that stages another block, or -1
                        if (!dead && qn >= 0 && TC_D1[qn] <= (cur ? TC_MAXD1 : TC_XS2_D1)) { request(cur ^ 1, qn); pre_q = qn; }
                    }
                } else {
                    if (restage && !dead) {   // warp w copies rows w, w + 16, ... (odd row stride: 4-byte pieces)
                        for (int r = warp; r < 128; r += TC_CW) {
                            const long long b = item0 + r;
                            const bool live = b < p.batch;
                            const float* src = p.x + (live ? b : 0) * TC_IN_DIM + xoff;
                            float* dst = sh.xs + r * TC_XSTRIDE;
                            for (int c = lane; c < 32 * d1; c += 32) tc_cp4(dst + c, src + c, live);
                        }
                        tc_cp_wait_all();
                    }
                    tc_compute_sync();
                }
                const float* xrow = (cur ? sh.xs2 + brow * TC_XSTRIDE2 : sh.xs + brow * TC_XSTRIDE) + ucol * d1;
                const int ustride = 4 * d1;                 // distance between this thread's consecutive channels
                const float* yrow = sh.ys + brow * TC_YSTRIDE;
                for (int k = 0; k < d3; ++k) {
                    const unsigned buf = step & 1u;
                    float acc[8];
#pragma unroll
                    for (int uu = 0; uu < 8; ++uu) acc[uu] = 0.f;
                    if (TC_MODE != 2) {
                        // Clebsch-Gordan stage for component k, term by term
                        const int t0 = TC_KBEG[tq + k], t1 = TC_KBEG[tq + k + 1];
                        if (d1 == 1) tc_cg<1>(xrow, yrow, t0, t1, acc);
                        else if (d1 == 3) tc_cg<3>(xrow, yrow, t0, t1, acc);
                        else if (d1 == 5) tc_cg<5>(xrow, yrow, t0, t1, acc);
                        else tc_cg<7>(xrow, yrow, t0, t1, acc);
                    } else {
                        // mode 2: the A operand is component k of the cotangent's block itself, A[b][w] = g[b, o][w, k].  The values
                        // were requested one step ahead (gnext); now request those of the next step: the next component of this
                        // path, or component 0 of the next path.
                        const long long b0 = item0 + brow;
                        const bool live = b0 < p.batch;
                        const float* grow = p.g + (live ? b0 : 0) * L3_DIM;
                        if (q == 0 && k == 0) {
#pragma unroll
                            for (int uu = 0; uu < 8; ++uu) gnext[uu] = live ? __ldg(grow + zoff + (ucol + 4 * uu) * d3) : 0.f;
                        }
#pragma unroll
                        for (int uu = 0; uu < 8; ++uu) acc[uu] = gnext[uu];
                        const bool more = k + 1 < d3;
                        if (more || q + 1 < TC_NPATH) {
                            const int nd3 = more ? d3 : TC_D3[q + 1];
                            const float* gn = grow + (more ? zoff + k + 1 : TC_ZOFF[q + 1]) + ucol * nd3;
#pragma unroll
                            for (int uu = 0; uu < 8; ++uu) gnext[uu] = live ? __ldg(gn + uu * 4 * nd3) : 0.f;
                        }
                    }
                    // the operand buffer was last read by the MMAs of step - 2 (a commit covers every MMA issued before it)
                    if (!dead && step >= 2 && !tc_mbar_wait(&sh.mma_done[buf], ((step >> 1) - 1) & 1u, abortf, p.status, 31)) dead = true;
                    dead = __any_sync(0xffffffffu, dead);   // a warp gives up as one: its arrival below is a single one
                    if (!dead) {
                        if (k == 0) {   // weight block of the path: B[n, kk] = W_p[kk, n] (forward: n = w, kk = u) or
                                        // W_p[n, kk] (gradients: n = u, kk = w); its buffer was last read two paths ago
#pragma unroll
                            for (int r = 0; r < 1024 / TC_CT; ++r) {
                                const int e = tid + TC_CT * r;          // e = u * 32 + w
                                const int u = e >> 5, w = e & 31;
                                const float v = wnext[r];               // requested one path ahead
                                const float hi = tc_tf32(v);
                                const int off = TC_WT ? tc_elem(u, w) : tc_elem(w, u);
                                sh.b[npath & 1u][0][off] = hi;
                                sh.b[npath & 1u][1][off] = tc_tf32(v - hi);
                            }
                            const int wq = (q + 1 < TC_NPATH) ? TC_WOFF[q + 1] : TC_WOFF[0];   // the next path's (or next tile's first)
#pragma unroll
                            for (int r = 0; r < 1024 / TC_CT; ++r) wnext[r] = __ldg(p.W + wq + tid + TC_CT * r);
                        }
#pragma unroll
                        for (int uu = 0; uu < 8; ++uu) {
                            const int off = tc_elem(brow, ucol + 4 * uu);
                            const float h = tc_tf32(acc[uu]);
                            sh.a[buf][0][off] = h;
                            sh.a[buf][1][off] = acc[uu] - h;   // the tensor core reads the top 19 bits: truncation of the low part is below 2^-21
                        }
                        tc_fence_async_smem();
                        tc_fence_before();
                        __syncwarp();                                   // every lane's stores and fences precede ...
                        if (lane == 0) tc_mbar_arrive(&sh.a_full[buf]);   // ... the warp's one arrival
                    }
                    ++step;
                }
                if (last) {
                    // epilogue of the output block: accumulators -> z
                    if (!dead && !tc_mbar_wait(&sh.acc_done[nblock & 1u], (nblock >> 1) & 1u, abortf, p.status, 32)) dead = true;
                    if (!dead) {
                        tc_fence_after();
                        const int qd = warp & 3, part = warp >> 2;          // TMEM lane quarter, column part
                        const long long b = item0 + qd * 32 + lane;
                        const unsigned tbase = tmem + ((unsigned)(qd * 32) << 16) + (nblock & 1u) * 256u + (unsigned)(TC_EC * part);
                        if (TC_MODE != 2) {
                            float* zdst = p.z + (b < p.batch ? b : 0) * TC_OUT_DIM + zoff + TC_EC * part * d3;
                            const bool live = b < p.batch;
                            if (d3 == 1) tc_epilogue<1>(tbase, zdst, live, p.accum != 0);
                            else if (d3 == 3) tc_epilogue<3>(tbase, zdst, live, p.accum != 0);
                            else if (d3 == 5) tc_epilogue<5>(tbase, zdst, live, p.accum != 0);
                            else tc_epilogue<7>(tbase, zdst, live, p.accum != 0);
                        } else {
                            // mode 2: the accumulators are g'[b][u, k] = sum_w W_p[u, w] g[b, o][w, k]; this thread folds its
                            // item's TC_EC channels into dy[b][j] += c * sum_u x[b][u, i] g'[b][u, k], term by term
                            float* dyp = sh.dys + tid * TC_DYS;
                            const float* xb = sh.xs + (qd * 32 + lane) * TC_XSTRIDE + TC_EC * part * d1;
                            for (int k = 0; k < d3; ++k) {
                                unsigned r[8];
                                tc_ld8(tbase + 32u * (unsigned)k, r);
                                const int t0 = TC_KBEG[tq + k], t1 = TC_KBEG[tq + k + 1];
                                for (int t = t0; t < t1; ++t) {
                                    const float* px = xb + TC_TI[t];
                                    float dot = 0.f;
#pragma unroll
                                    for (int u = 0; u < TC_EC; ++u) dot = fmaf(px[u * d1], __uint_as_float(r[u]), dot);
                                    dyp[TC_TJ[t]] = fmaf(TC_TC[t], dot, dyp[TC_TJ[t]]);
                                }
                            }
                        }
                        tc_fence_before();
                    }
                    ++nblock;
                }
                ++npath;
            }
            if (TC_MODE == 2) {
                // dy of the tile: threads t, t + 128, ... hold the channel parts of item t
                tc_compute_sync();
                const long long b = item0 + tid;
                if (tid < 128 && b < p.batch && !sh.abort_flag)
                    for (int j = 0; j < L2_DIM; ++j) {
                        float v = 0.f;
#pragma unroll
                        for (int part = 0; part < TC_CW / 4; ++part) v += sh.dys[(tid + 128 * part) * TC_DYS + j];
                        p.z[b * L2_DIM + j] = p.accum ? p.z[b * L2_DIM + j] + v : v;
                    }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}
#endif  // TC_MODE != 3

#if TC_MODE == 3
// ---- gradient of the shared weights ---------------------------------------------------------------------------
//   dW_p[u, w] = sum_b sum_k T_p[b][u, k] * g[b, o][w, k],     T_p as in the forward (Clebsch-Gordan stage, CUDA cores)
// A GEMM whose reduction runs over the batch.  Up to four paths into the same output block o are stacked on M (they share
// the B operand): per step (group of paths, component k, 32 items)
//   D[(slot, u), w] += A[(slot, u), b] * B[w, b],   A = T (128 x 32), B = component k of the cotangent block (32 x 32),
// both K-major with the items on K (4 tcgen05.mma of K = 8, three split terms each; the chunk geometry of the forward).
// The accumulators of every group live in tensor memory (32 columns per group) for one tile of 64 items; after the tile
// the CTA stores them as row `tile` of a partials matrix that a second kernel sums in row order (bitwise reproducible,
// and in fp32 with rounding: the tensor cores' own accumulation truncates, so its sums are kept short).
// The input blocks of a group's slots are staged in shared memory once per (tile of 64 items, group) by asynchronous row
// copies and serve all components k and both halves of the tile.
// Sixteen compute warps and one issuing warp, coupled through mbarriers like the forward.  Compute warp w works on slot
// w % 4 and items 8 (w / 4) ... + 8 of the step's 32; a lane covers channels lane / 4 + 8 uu (uu < 4) and items lane % 4 + 4 bb
// (bb < 2): with staged rows of 32 d1 + 8 floats its reads, and in the canonical operand layout its writes, fall into 32
// different banks.
struct TcDwParams {
    const float* x; const float* y; const float* g; float* part;
    long long batch;
    int grp_begin, grp_end;   // this launch's groups (at most 16: one 32-column accumulator each)
    int* status;
};
constexpr int TCW_TILE = 64;
constexpr int TCW_YS = L2_DIM | 1;
struct __align__(128) TcDwShared {
    float a[2][2][TC_A_FLOATS];       // [buffer][hi, lo]
    float b[2][2][TC_B_FLOATS];
    float xs[TCW_XS_FLOATS];          // the input blocks of the group's slots for the tile's items (TCW_XSOFF)
    float ys[TCW_TILE * TCW_YS];      // harmonics of the tile's items
    unsigned long long a_full[2];
    unsigned long long mma_done[2];
    unsigned long long xs_full;       // the staged input blocks have arrived (bytes of the bulk copies)
    unsigned tmem_base;
    int abort_flag;
};
// Clebsch-Gordan stage of one step for one thread (two items, four channels each); D1 at compile time makes the offsets
// in the staged rows immediates.
template <int D1>
OEQ_DEV void tcw_cg(const float* xt, const float* yb, int t0, int t1, float (&acc)[4][2]) {
    constexpr int XS = 32 * D1 + 8;
    for (int t = t0; t < t1; ++t) {
        const float c = TCW_TC[t];
        const float* py = yb + TCW_TJ[t];
        const float* px = xt + TCW_TI[t];
        const float cy0 = c * py[0], cy1 = c * py[4 * TCW_YS];
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
            acc[uu][0] = fmaf(cy0, px[8 * uu * D1], acc[uu][0]);
            acc[uu][1] = fmaf(cy1, px[4 * XS + 8 * uu * D1], acc[uu][1]);
        }
    }
}
static_assert(sizeof(TcDwShared) <= 232448, "the buffers exceed shared memory");   // (one CTA per SM: see TcShared)

extern "C" __global__ void __launch_bounds__(TC_THREADS, 1) oeq_uvw_tc_backward_dw(const TcDwParams p) {
    extern __shared__ __align__(128) unsigned char tc_smem_raw[];
    TcDwShared& sh = *reinterpret_cast<TcDwShared*>(tc_smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    volatile int* abortf = &sh.abort_flag;
    if (tid == 0) {
        tc_mbar_init(&sh.a_full[0], TC_CW); tc_mbar_init(&sh.a_full[1], TC_CW);   // one arrival per compute warp
        tc_mbar_init(&sh.mma_done[0], 1); tc_mbar_init(&sh.mma_done[1], 1);
        tc_mbar_init(&sh.xs_full, 1);
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(tc_smem_u32(&sh.tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = sh.tmem_base;
    const long long ntiles = (p.batch + TCW_TILE - 1) / TCW_TILE;
    unsigned step = 0;     // steps so far: operand buffer = step & 1
    bool dead = false;

    if (warp == TC_CW) {
        // ---- the issuing warp (operand descriptors built once, see the forward)
        const unsigned long long da0h = tc_desc(&sh.a[0][0][0], TC_LBO, TC_SBO), da0l = tc_desc(&sh.a[0][1][0], TC_LBO, TC_SBO);
        const unsigned long long da1h = tc_desc(&sh.a[1][0][0], TC_LBO, TC_SBO), da1l = tc_desc(&sh.a[1][1][0], TC_LBO, TC_SBO);
        const unsigned long long db0h = tc_desc(&sh.b[0][0][0], TC_LBO, TC_SBO), db0l = tc_desc(&sh.b[0][1][0], TC_LBO, TC_SBO);
        const unsigned long long db1h = tc_desc(&sh.b[1][0][0], TC_LBO, TC_SBO), db1l = tc_desc(&sh.b[1][1][0], TC_LBO, TC_SBO);
        for (long long tile = blockIdx.x; tile < ntiles && !dead; tile += gridDim.x) {
            for (int grp = p.grp_begin; grp < p.grp_end && !dead; ++grp) {
                const int d3 = TCW_D3[grp];
                for (int kh = 0; kh < 2 * d3 && !dead; ++kh) {   // (component k, half of the tile)
                    const unsigned buf = step & 1u;
                    if (!tc_mbar_wait(&sh.a_full[buf], (step >> 1) & 1u, abortf, p.status, 36)) { dead = true; break; }
                    tc_fence_after();
                    if (lane == 0) {
                        const unsigned dcol = tmem + 32u * (unsigned)(grp - p.grp_begin);
                        const unsigned long long ah0 = buf ? da1h : da0h, al0 = buf ? da1l : da0l;
                        const unsigned long long bh0 = buf ? db1h : db0h, bl0 = buf ? db1l : db0l;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const unsigned long long ah = ah0 + 16ull * ks, al = al0 + 16ull * ks;
                            const unsigned long long bh = bh0 + 16ull * ks, bl = bl0 + 16ull * ks;
                            tc_mma(dcol, ah, bh, (kh == 0 && ks == 0) ? 0u : 1u);   // every tile starts its sums afresh
                            tc_mma(dcol, al, bh, 1u);
                            tc_mma(dcol, ah, bl, 1u);
                        }
                        tc_commit(&sh.mma_done[buf]);
                    }
                    __syncwarp();
                    ++step;
                }
            }
        }
    } else {
        const int slot = warp & 3, sub = warp >> 2, r8 = lane >> 2, b4 = lane & 3;
        unsigned nstage = 0;   // staged groups so far (phase of xs_full)
        for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const long long item0 = tile * TCW_TILE;
            const long long nlive = p.batch - item0;         // items of the tile that exist
            tc_compute_sync();   // the previous tile's readers of ys are done
            for (int r = warp; r < TCW_TILE; r += TC_CW)
                for (int j = lane; j < L2_DIM; j += 32)
                    sh.ys[r * TCW_YS + j] = (r < nlive) ? __ldg(p.y + (item0 + r) * L2_DIM + j) : 0.f;
            for (int grp = p.grp_begin; grp < p.grp_end; ++grp) {
                const int d3 = TCW_D3[grp], zoff = TCW_ZOFF[grp], ns = TCW_NS[grp];
                // stage the slots' input blocks: one bulk copy per (slot, row), issued by the first 64 * ns threads; everybody
                // waits for the bytes.  Rows past the end of the batch read row 0 and meet y = 0.
                tc_compute_sync();   // readers of the previous group's blocks are done
                if (!dead) {
                    if (tid == 0) {
                        int sumd1 = 0;
                        for (int sl = 0; sl < ns; ++sl) sumd1 += TCW_D1[grp * 4 + sl];
                        tc_mbar_expect_tx(&sh.xs_full, 64u * 128u * (unsigned)sumd1);
                    }
                    if (tid < 64 * ns) {
                        const int sl = tid >> 6, r = tid & 63, qs = grp * 4 + sl, ds = TCW_D1[qs];
                        tc_bulk_row(sh.xs + TCW_XSOFF[qs] + r * (32 * ds + 8),
                                    p.x + (r < nlive ? item0 + r : 0) * L1_DIM + TCW_XOFF[qs], 128u * (unsigned)ds, &sh.xs_full);
                    }
                    if (!tc_mbar_wait(&sh.xs_full, nstage & 1u, abortf, p.status, 38)) dead = true;
                    ++nstage;
                }
                const int q = grp * 4 + slot;
                const int d1 = TCW_D1[q], xs_stride = 32 * d1 + 8;
                for (int kh = 0; kh < 2 * d3; ++kh) {
                    const int k = kh >> 1, half = kh & 1;
                    const unsigned buf = step & 1u;
                    const int ic = 8 * sub + b4;                     // this thread's first column (item of the step's 32)
                    const int ib = 32 * half + ic;                   // ... and its item of the tile; the second is 4 further
                    // Clebsch-Gordan stage: acc[uu][bb] = T[item ib + 4 bb][channel r8 + 8 uu] of this warp's slot
                    float acc[4][2];
#pragma unroll
                    for (int uu = 0; uu < 4; ++uu) { acc[uu][0] = 0.f; acc[uu][1] = 0.f; }
                    const float* xt = sh.xs + TCW_XSOFF[q] + ib * xs_stride + r8 * d1;
                    const int tq = TCW_INS[q] < 0 ? 0 : TCW_INS[q] * 8;
                    const int t0 = TCW_KBEG[tq + k], t1 = TCW_INS[q] < 0 ? t0 : TCW_KBEG[tq + k + 1];
                    const float* yb = sh.ys + ib * TCW_YS;
                    if (d1 == 1) tcw_cg<1>(xt, yb, t0, t1, acc);
                    else if (d1 == 3) tcw_cg<3>(xt, yb, t0, t1, acc);
                    else if (d1 == 5) tcw_cg<5>(xt, yb, t0, t1, acc);
                    else tcw_cg<7>(xt, yb, t0, t1, acc);
                    // this thread's 2 entries of B: row w = r8 + 8 * slot, the same two items
                    float gv[2];
#pragma unroll
                    for (int bb = 0; bb < 2; ++bb) {
                        const int bi = ib + 4 * bb;
                        gv[bb] = (bi < nlive) ? __ldg(p.g + (item0 + bi) * L3_DIM + zoff + (r8 + 8 * slot) * d3 + k) : 0.f;
                    }
                    if (!dead && step >= 2 && !tc_mbar_wait(&sh.mma_done[buf], ((step >> 1) - 1) & 1u, abortf, p.status, 33)) dead = true;
                    dead = __any_sync(0xffffffffu, dead);   // a warp gives up as one: its arrival below is a single one
                    if (!dead) {
#pragma unroll
                        for (int uu = 0; uu < 4; ++uu)
#pragma unroll
                            for (int bb = 0; bb < 2; ++bb) {
                                const int off = tc_elem(slot * 32 + r8 + 8 * uu, ic + 4 * bb);
                                const float v = acc[uu][bb], hi = tc_tf32(v);
                                sh.a[buf][0][off] = hi;
                                sh.a[buf][1][off] = v - hi;   // truncated by the tensor core: below 2^-21
                            }
#pragma unroll
                        for (int bb = 0; bb < 2; ++bb) {
                            const int off = tc_elem(r8 + 8 * slot, ic + 4 * bb);
                            const float hi = tc_tf32(gv[bb]);
                            sh.b[buf][0][off] = hi;
                            sh.b[buf][1][off] = tc_tf32(gv[bb] - hi);
                        }
                        tc_fence_async_smem();
                        tc_fence_before();
                        __syncwarp();                                   // every lane's stores and fences precede ...
                        if (lane == 0) tc_mbar_arrive(&sh.a_full[buf]);   // ... the warp's one arrival
                    }
                    ++step;
                }
            }
            // The tile's sums: row `tile` of the partials matrix (TMEM lane = (slot, u), column = 32 * group + w).  The
            // accumulators are emptied after every tile because the tensor cores add into them with truncation: the error of
            // a sum grows with its length, and a sum over the whole batch would leave the fp32 bound (measured: 1e-5 at
            // 50,000 items, 8e-5 at 400,000); the rows are added in fp32 with rounding by the ordered reduce.
            if (!dead && step >= 1 && !tc_mbar_wait(&sh.mma_done[(step - 1) & 1u], ((step - 1) >> 1) & 1u, abortf, p.status, 34)) dead = true;
            dead = __any_sync(0xffffffffu, dead);
            if (!dead && step >= 1) {
                tc_fence_after();
                float* prow = p.part + tile * WN;
                for (int grp = p.grp_begin; grp < p.grp_end; ++grp) {
                    if (slot >= TCW_NS[grp]) continue;   // uniform in the warp
                    unsigned r[8];
                    tc_ld8(tmem + ((unsigned)(slot * 32) << 16) + 32u * (unsigned)(grp - p.grp_begin) + (unsigned)(TC_EC * sub), r);
                    float4* dst = reinterpret_cast<float4*>(prow + TCW_WOFF[grp * 4 + slot] + lane * 32 + TC_EC * sub);
                    dst[0] = make_float4(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]), __uint_as_float(r[3]));
                    dst[1] = make_float4(__uint_as_float(r[4]), __uint_as_float(r[5]), __uint_as_float(r[6]), __uint_as_float(r[7]));
                }
                tc_fence_before();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}
#endif  // TC_MODE == 3

#endif  // OEQ_TC

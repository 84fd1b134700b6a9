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

struct TcParams {
    const float* x; const float* y; const float* W; float* z;
    long long batch;
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
constexpr int TC_XSTRIDE = 32 * TC_MAXD1 + 4;   // padded row of the staged input block (conflict-free column reads)
constexpr int TC_YSTRIDE = (L2_DIM + 3) & ~3;

struct __align__(128) TcShared {
    float a[2][2][TC_A_FLOATS];       // [buffer][hi, lo]
    float b[2][2][TC_B_FLOATS];
    float xs[128 * TC_XSTRIDE];       // input block a(p) of the 128 items of the tile
    float ys[128 * TC_YSTRIDE];       // harmonics of the 128 items
    unsigned long long mma_done[2];   // a buffer may be rewritten
    unsigned long long acc_done[2];   // accumulators of an output block are complete
    unsigned tmem_base;
    int abort_flag;
};
static_assert(sizeof(TcShared) > 116 * 1024 && sizeof(TcShared) <= 232448, "one CTA per SM is assumed (it owns all of TMEM)");

// offset (in floats) of element (row, kcol) in a chunk
OEQ_DEV int tc_elem(int row, int kcol) { return (row >> 3) * (TC_SBO / 4) + (kcol >> 2) * (TC_LBO / 4) + (row & 7) * 4 + (kcol & 3); }

// Epilogue of one output block for one thread: its item's 16 output channels x D3 components are 16 * D3 consecutive
// floats of the z row.  All components are pulled out of tensor memory first (column 32 k + c holds channel c of
// component k), then written as 16-byte stores, so every 32-byte sector of z is written whole.
template <int D3>
OEQ_DEV void tc_epilogue(unsigned tbase, float* zdst, bool live) {
    float v[16 * D3];   // v[c * D3 + k]
#pragma unroll
    for (int k = 0; k < D3; ++k) {
        unsigned r[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(tbase + 32u * (unsigned)k) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c * D3 + k] = __uint_as_float(r[c]);
    }
    if (live) {
        float4* dst = reinterpret_cast<float4*>(zdst);   // 64 * D3 bytes from a 16-byte boundary
#pragma unroll
        for (int q = 0; q < 4 * D3; ++q) __stcs(dst + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
    }
}

// The loops over paths, output components and Clebsch-Gordan terms are run-time loops over the TC_* tables of the
// problem header (not unrolled): the whole kernel is a few KB of code and stays in the instruction cache.
extern "C" __global__ void __launch_bounds__(256, 1) oeq_uvw_tc_forward(const TcParams p) {
    extern __shared__ __align__(128) unsigned char tc_smem_raw[];
    TcShared& sh = *reinterpret_cast<TcShared*>(tc_smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    volatile int* abortf = &sh.abort_flag;
    if (tid == 0) {
        tc_mbar_init(&sh.mma_done[0], 1); tc_mbar_init(&sh.mma_done[1], 1);
        tc_mbar_init(&sh.acc_done[0], 1); tc_mbar_init(&sh.acc_done[1], 1);
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

    // this thread's 16 elements of every A chunk: items brow, brow + 8 and channels ucol + 4 * uu, uu < 8
    const int brow = warp * 16 + (lane >> 2);
    const int ucol = lane & 3;
    unsigned step = 0;     // chunk steps issued so far: A buffer = step & 1
    unsigned npath = 0;    // paths started so far: weight buffer = npath & 1
    unsigned nblock = 0;   // output blocks finished so far: accumulator half = nblock & 1
    const long long ntiles = (p.batch + 127) / 128;
    bool dead = false;

    for (long long tile = blockIdx.x; tile < ntiles && !dead; tile += gridDim.x) {
        const long long item0 = tile * 128;
        __syncthreads();   // previous tile's readers of xs / ys are done
        for (int r = warp; r < 128; r += 8)          // one warp per row: no index division
            for (int j = lane; j < L2_DIM; j += 32)
                sh.ys[r * TC_YSTRIDE + j] = (item0 + r < p.batch) ? __ldg(p.y + (item0 + r) * L2_DIM + j) : 0.f;
        for (int q = 0; q < NINS && !dead; ++q) {
            const int d1 = TC_D1[q], d3 = TC_D3[q], xoff = TC_XOFF[q], zoff = TC_ZOFF[q], woff = TC_WOFF[q];
            const int first = TC_FIRST[q], last = TC_LAST[q];
            // stage the path's input block: rows of 32 * d1 contiguous floats, coalesced; the block stays when the previous
            // path of this tile read the same one
            const bool restage = q == 0 || TC_XOFF[q - 1] != xoff;
            __syncthreads();   // readers of the previous path's block are done
            const int rowlen = restage ? 32 * d1 : 0;
            for (int c = lane; c < rowlen; c += 32) {   // warp w copies rows w, w + 8, ...: 16 independent loads in flight
                float v[16];
#pragma unroll
                for (int rr = 0; rr < 16; ++rr) {
                    const long long b = item0 + warp + 8 * rr;
                    v[rr] = (b < p.batch) ? __ldg(p.x + b * L1_DIM + xoff + c) : 0.f;
                }
#pragma unroll
                for (int rr = 0; rr < 16; ++rr) sh.xs[(warp + 8 * rr) * TC_XSTRIDE + c] = v[rr];
            }
            __syncthreads();
            const float* xrow0 = sh.xs + brow * TC_XSTRIDE + ucol * d1;
            const float* xrow1 = xrow0 + 8 * TC_XSTRIDE;
            const int ustride = 4 * d1;                 // distance between this thread's consecutive channels
            const float* yrow0 = sh.ys + brow * TC_YSTRIDE;
            const float* yrow1 = yrow0 + 8 * TC_YSTRIDE;
            for (int k = 0; k < d3 && !dead; ++k) {
                const unsigned buf = step & 1u;
                // Clebsch-Gordan stage for output component k: 16 elements per thread, term by term
                float acc0[8], acc1[8];
#pragma unroll
                for (int uu = 0; uu < 8; ++uu) { acc0[uu] = 0.f; acc1[uu] = 0.f; }
                const int t0 = TC_KBEG[q * 8 + k], t1 = TC_KBEG[q * 8 + k + 1];
                for (int t = t0; t < t1; ++t) {
                    const int ti = TC_TI[t], tj = TC_TJ[t];
                    const float c = TC_TC[t];
                    const float cy0 = c * yrow0[tj], cy1 = c * yrow1[tj];
                    const float* px0 = xrow0 + ti;
                    const float* px1 = xrow1 + ti;
#pragma unroll
                    for (int uu = 0; uu < 8; ++uu) {
                        acc0[uu] = fmaf(cy0, px0[uu * ustride], acc0[uu]);
                        acc1[uu] = fmaf(cy1, px1[uu * ustride], acc1[uu]);
                    }
                }
                // the A buffer was last read by the MMAs of step - 2 (a commit covers every MMA issued before it)
                if (step >= 2 && !tc_mbar_wait(&sh.mma_done[buf], ((step >> 1) - 1) & 1u, abortf, p.status, 31)) dead = true;
                if (!dead) {
                    if (k == 0) {   // weight block of the path: B[w, u] = W_p[u, w]; its buffer was last read two paths ago
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int e = tid + 256 * r;          // e = u * 32 + w
                            const int u = e >> 5, w = e & 31;
                            const float v = __ldg(p.W + woff + e);
                            const float hi = tc_tf32(v);
                            sh.b[npath & 1u][0][tc_elem(w, u)] = hi;
                            sh.b[npath & 1u][1][tc_elem(w, u)] = tc_tf32(v - hi);
                        }
                    }
#pragma unroll
                    for (int uu = 0; uu < 8; ++uu) {
                        const int off0 = tc_elem(brow, ucol + 4 * uu), off1 = tc_elem(brow + 8, ucol + 4 * uu);
                        const float h0 = tc_tf32(acc0[uu]), h1 = tc_tf32(acc1[uu]);
                        sh.a[buf][0][off0] = h0;
                        sh.a[buf][1][off0] = tc_tf32(acc0[uu] - h0);
                        sh.a[buf][0][off1] = h1;
                        sh.a[buf][1][off1] = tc_tf32(acc1[uu] - h1);
                    }
                    tc_fence_async_smem();
                }
                tc_fence_before();
                __syncthreads();
                tc_fence_after();
                if (sh.abort_flag) dead = true;
                if (!dead && tid == 0) {
                    const unsigned bbuf = npath & 1u;
                    const unsigned dcol = tmem + (nblock & 1u) * 256u + 32u * (unsigned)k;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const unsigned long long ah = tc_desc(&sh.a[buf][0][ks * 2 * (TC_LBO / 4)], TC_LBO, TC_SBO);
                        const unsigned long long al = tc_desc(&sh.a[buf][1][ks * 2 * (TC_LBO / 4)], TC_LBO, TC_SBO);
                        const unsigned long long bh = tc_desc(&sh.b[bbuf][0][ks * 2 * (TC_LBO / 4)], TC_LBO, TC_SBO);
                        const unsigned long long bl = tc_desc(&sh.b[bbuf][1][ks * 2 * (TC_LBO / 4)], TC_LBO, TC_SBO);
                        tc_mma(dcol, ah, bh, (first && ks == 0) ? 0u : 1u);
                        tc_mma(dcol, al, bh, 1u);
                        tc_mma(dcol, ah, bl, 1u);
                    }
                    tc_commit(&sh.mma_done[buf]);
                    if (last && k == d3 - 1) tc_commit(&sh.acc_done[nblock & 1u]);
                }
                ++step;
            }
            if (last) {
                // epilogue of the output block: accumulators -> z
                if (!dead && !tc_mbar_wait(&sh.acc_done[nblock & 1u], (nblock >> 1) & 1u, abortf, p.status, 32)) dead = true;
                if (!dead) {
                    tc_fence_after();
                    const int qd = warp & 3, half = warp >> 2;          // TMEM lane quarter, column half
                    const long long b = item0 + qd * 32 + lane;
                    const unsigned tbase = tmem + ((unsigned)(qd * 32) << 16) + (nblock & 1u) * 256u + 16u * half;
                    float* zdst = p.z + (b < p.batch ? b : 0) * L3_DIM + zoff + 16 * half * d3;
                    const bool live = b < p.batch;
                    if (d3 == 1) tc_epilogue<1>(tbase, zdst, live);
                    else if (d3 == 3) tc_epilogue<3>(tbase, zdst, live);
                    else if (d3 == 5) tc_epilogue<5>(tbase, zdst, live);
                    else tc_epilogue<7>(tbase, zdst, live);
                    tc_fence_before();
                }
                ++nblock;
                __syncthreads();                      // keeps the give-up decision uniform across the CTA
                if (sh.abort_flag) dead = true;
            }
            ++npath;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

#endif  // OEQ_TC

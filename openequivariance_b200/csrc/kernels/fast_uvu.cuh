// Channel-parallel, TMA-pipelined kernels for 'uvu' problems whose second operand has multiplicity 1 everywhere
// and whose first operand uses one common multiplicity FU (the MACE-style channelwise product), fp32 or fp64 (T).
//
// Work decomposition
//   * one consumer thread per channel u (FU threads) handles every path of its channel, so all of an edge's
//     arithmetic for one channel stays in registers and nothing is exchanged between threads except the
//     16-number dY reduction;
//   * one producer warp per CTA streams edges: it issues 1-D TMA bulk copies (cp.async.bulk) of the sender's
//     feature row X[col] and the edge's weight row W[e] into a ring of shared-memory stages guarded by
//     mbarriers, fetches Y[e] with cp.async and turns it into the edge's folded coefficients
//     cy[i,k] = sum_j C[i,j,k] y[j] (they do not depend on the channel), and -- in the backward pass -- drains each finished stage: dX row
//     by TMA bulk store / bulk reduce-add, dY by a fixed-order sum of per-warp partials;
//   * receiver-sorted edges: a CTA owns a contiguous receiver range, keeps the receiver's output row (forward) or
//     its gradient row (backward) in registers across the receiver's edges; the summation order per receiver
//     is the edge order, whatever the grid size, hence bitwise reproducible results.
//
// Math per channel u and path (l1,l2,l3) with folded coefficients (reference formulas: templates/loop_unroll_tp.cuh:46-96
// forward, :202-291 backward):
//   forward   z[k]  += w * sum_i cy[i,k] x[i]
//   backward  s[i]   = sum_k cy[i,k] g[k];  dx[i] += w s[i];  dW = sum_i x[i] s[i];  dy[j] += C[i,j,k] x[i] (w g[k])
//
// Every wait on an mbarrier is bounded: when the limit is hit the thread records a code in *status, raises a
// CTA-wide abort flag and leaves; the host reports OEQB_EKERNEL.
#pragma once
#if OEQ_FAST

#define FAST_TP 0       // batch tensor product: edge e reads X[e], writes row e
#define FAST_DET 1      // convolution, receiver-sorted edges, plain stores
#define FAST_ATOMIC 2   // convolution, any edge order, atomic / bulk-reduce scatter

struct FastParams {
    const T* X; const T* Y; const T* W; const T* G;
    T* Z; T* dX; T* dY; T* dW; T* scratch;
    const IDX* rows; const IDX* cols;
    long long N; long long E;
    int* status;
    int accum;          // forward kernels: add to the output rows instead of overwriting them
    int pad;
    const T* X2; const T* Y2; const T* W2;   // second-order kernels: the cotangents of (dX, dY, dW)
    const IDX* eorder;  // convolutions over an unsorted edge list: position -> edge id, grouped by receiver (or null:
                        // position = edge id).  rows / cols / Y / W / dY / dW are indexed by edge id.
};
// Second-order kernels (FAST_DBL), one pass each:
//   forward   z = F(X2, Y, W) + F(X, Y, W2) + F(X, Y2, W)
//   backward  (dX, dY, dW) = Bwd(X2, Y, W | g) with dX scaled by W2  +  Bwd(X, Y2, W2 | g) with dX scaled by W
// X and W are staged as usual; the rows of X2 and W2 are read by the consumers straight from global memory (the
// producer brings them into the L2 ahead), Y2 is folded into a second coefficient table.
#define FAST_FWD3 (FAST_DBL && FAST_KERNEL <= 2)

// ---- PTX wrappers -----------------------------------------------------------------------------------------
OEQ_DEV unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
OEQ_DEV void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
OEQ_DEV void mbar_arrive(unsigned long long* bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
OEQ_DEV void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
OEQ_DEV bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
OEQ_DEV unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait (about two seconds of wall time).  Returns false when it gave up or another thread did.
OEQ_DEV bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > 2000000000ull) {
                *abort_flag = 1;
                *(volatile int*)status = code;   // host-mapped word: a plain store, no atomics across the bus
                return false;
            }
        }
    }
}
// L2 eviction policies for the bulk copies: rows that are touched once (weights, per-edge outputs) should leave the L2
// first, so that the sender rows, which neighbouring receivers read again, stay.
OEQ_DEV unsigned long long l2_evict_first() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
OEQ_DEV void tma_load(void* dst_smem, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
OEQ_DEV void tma_load_hint(void* dst_smem, const void* src, unsigned bytes, unsigned long long* bar, unsigned long long pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol) : "memory");
}
OEQ_DEV void tma_store(void* dst, const void* src_smem, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)), "r"(bytes) : "memory");
}
OEQ_DEV void tma_store_hint(void* dst, const void* src_smem, unsigned bytes, unsigned long long pol) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(dst), "r"(smem_u32(src_smem)), "r"(bytes), "l"(pol) : "memory");
}
OEQ_DEV void tma_reduce_add(void* dst, const void* src_smem, unsigned bytes) {
    if (sizeof(T) == 8)
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f64 [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)),
                     "r"(bytes) : "memory");
    else
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)),
                     "r"(bytes) : "memory");
}
OEQ_DEV void l2_prefetch(const void* src, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
OEQ_DEV void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> OEQ_DEV void tma_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> OEQ_DEV void tma_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
OEQ_DEV void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
OEQ_DEV void ldgsts4(void* dst_smem, const void* src) {   // one element of T
    if (sizeof(T) == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
OEQ_DEV void ldgsts_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> OEQ_DEV void ldgsts_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- shared-memory stage ----------------------------------------------------------------------------------
constexpr int FAST_GT = FU / FAST_CH;                      // threads per group: each carries FAST_CH channels
constexpr int FAST_NT = FAST_NG * FAST_GT;                // consumer threads (of one edge stream)
constexpr int FAST_NCW = FAST_NT / 32;                    // consumer warps (of one edge stream)
// Producer warps per CTA.  With two, they take the CTA's edges in turn: with 4 + 2 warps per CTA and
// two CTAs per SM every scheduler hosts two consumer warps and one (half-loaded) producer; with a single producer warp two
// of the four schedulers carried 40 % more instructions than the others and set the pace.
// FAST_NP (problem header): 2 from four stages on (the look-ahead is then a multiple of two), else 1.
// Edge streams per CTA (FAST_V, problem header).  With FAST_V > 1 one CTA per SM hosts FAST_V independent sets of
// FAST_NT consumer threads, each with its own ring of stages, range of edges and producer warp (the sets share nothing but
// the SM), followed by one warpgroup of producer warps.  The point is the register file: producer warps need few
// registers but a launch gives every thread the same number, so right after the role split the producer warpgroup hands
// its surplus to the consumer warpgroups (setmaxnreg); that pays for a third consumer set per SM (12 consumer warps
// instead of 8) where two CTAs of 4 + 2 warps filled the register file.  The register numbers below only add up when the
// launch gave every thread exactly FAST_REG_LAUNCH registers (the host checks the compiled kernel before using it).
constexpr int FAST_PW = (FAST_V == 1) ? FAST_NP : 4;                 // producer warps in the CTA
constexpr int FAST_THREADS = FAST_V * FAST_NT + 32 * FAST_PW;
constexpr int FAST_REG_LAUNCH = 65536 / (FAST_V * 128 + 128) / 8 * 8;   // FAST_V > 1: registers per thread at launch
constexpr int FAST_REG_PRODUCER = 56;
constexpr int FAST_REG_CONSUMER = (FAST_REG_LAUNCH + (FAST_REG_LAUNCH - FAST_REG_PRODUCER) / FAST_V) / 8 * 8;
static_assert(FAST_V == 1 || (FAST_NT == 128 && FAST_NP == 1), "edge streams are warpgroups with one producer warp each");
static_assert(FAST_V <= 4, "one producer warp per stream out of a single warpgroup");
// With several streams the single producer warp of a stream is the scarce resource (it serves every edge, where two warps
// take turns otherwise), so the folding of Y[e] into the coefficients moves to the stream's consumer threads: each folds
// up to three of the NCY entries from a table in shared memory, then all meet at a per-stage mbarrier.
constexpr bool FAST_CFOLD = FAST_V > 1;
constexpr int FAST_TAB_ENTRIES = FAST_CFOLD ? NCY * FAST_CYT : 1;
constexpr int FAST_NYP = (L2_DIM <= 1) ? 1 : (L2_DIM <= 2) ? 2 : (L2_DIM <= 4) ? 4 : (L2_DIM <= 8) ? 8 : (L2_DIM <= 16) ? 16 : 32;
constexpr int FAST_YPAD = (L2_DIM + 3) & ~3;
struct __align__(16) FastStage {
    T x[L1_DIM];                 // sender row; the backward pass overwrites it in place with the edge's dX row
    T w[WN];
    T cy[NCY];                   // folded coefficients of this edge: cy[q] = sum_j C[i_q][j][k_q] * y[j], one per (i, k) pair
    T y[FAST_YPAD];
    T cy2[FAST_DBL ? NCY : 4];   // second-order kernels: coefficients folded with Y2
    T y2[FAST_DBL ? FAST_YPAD : 4];
    T dyp[FAST_NCW][FAST_NYP];   // per-warp partial sums of dY
    long long edge, row, col;
    int first, last, pad0, pad1;
};
constexpr int FAST_ZBUF = (FAST_KERNEL == 2) ? L3_DIM : 4;   // atomic forward stages a receiver row for a bulk reduce
struct __align__(16) FastShared {
    FastStage st[FAST_S];
    T zbuf[FAST_ZBUF];
    unsigned long long full[FAST_S];
    unsigned long long empty[FAST_S];
    unsigned long long drained[FAST_S];   // backward with two producers: the stage's dX row has left shared memory
    unsigned long long folded[FAST_CFOLD ? FAST_S : 1];   // consumer-side folding: every consumer has written its coefficients
    unsigned long long zfull, zfree;
    long long range[4];              // e0, e1, n0, n1
    int abort_flag;
    int pad[3];
};
// coefficient table for consumer-side folding, behind the streams' FastShared blocks: (coefficient, index into y) pairs
struct FastTabEntry { T c; int j; };
constexpr size_t FAST_SMEM_NEED = FAST_V * sizeof(FastShared) + (FAST_CFOLD ? FAST_TAB_ENTRIES * sizeof(FastTabEntry) : 0);
static_assert(FAST_SMEM_NEED <= 232448, "stages exceed shared memory");
static_assert(FAST_KERNEL == 6 || FAST_SMEM_NEED <= FAST_SMEM_BYTES, "the host sized the dynamic shared memory too small");
OEQ_DEV FastTabEntry* fast_tab(unsigned char* smem_raw) { return reinterpret_cast<FastTabEntry*>(smem_raw + FAST_V * sizeof(FastShared)); }
// All threads of the CTA: copy the table into shared memory (before the CTA-wide barrier that follows the set-up).
OEQ_DEV void fast_tab_fill(unsigned char* smem_raw) {
    if (FAST_CFOLD) {
        FastTabEntry* tab = fast_tab(smem_raw);
        for (int q = threadIdx.x; q < FAST_TAB_ENTRIES; q += blockDim.x) { tab[q].c = FAST_CYC[q]; tab[q].j = FAST_CYJ[q]; }
    }
}
// Consumer thread ltid of a stream: fold its share of the edge's coefficients, then wait until all have.
OEQ_DEV bool fast_consumer_fold(FastShared& sh, FastStage& st, const FastTabEntry* tab, int s, unsigned par, int ltid,
                                volatile int* abortf, int* status) {
    if (!FAST_CFOLD) return true;
#pragma unroll
    for (int q = ltid; q < NCY; q += FAST_NT) {
        T v = tab[q * FAST_CYT].c * st.y[tab[q * FAST_CYT].j];
#pragma unroll
        for (int m = 1; m < FAST_CYT; ++m) v = oeq_fma(tab[q * FAST_CYT + m].c, st.y[tab[q * FAST_CYT + m].j], v);
        st.cy[q] = v;
    }
    mbar_arrive(&sh.folded[FAST_CFOLD ? s : 0]);
    return mbar_wait(&sh.folded[FAST_CFOLD ? s : 0], par, abortf, status, 25);
}
// TMA look-ahead in edges.  One stage stays in hand: in the backward pass for the dX row that is still leaving shared
// memory (FAST_S >= FAST_D + 2); the forward pass measured fastest two edges ahead (7.07 ms against 7.23 / 7.36 ms at 3 / 4).
constexpr int FAST_D = (FAST_KERNEL <= 2) ? ((FAST_S >= 4) ? 2 : 1)
                       : (FAST_NP == 2)   ? ((FAST_S - 2) & ~1)
                                          : ((FAST_S >= 4) ? FAST_S - 2 : 1);
// FAST_XPC / FAST_GPC (problem header): registers per channel for an X / dX row and for a Z / G row

// Transposed butterfly over a warp: on return v[0] of lane L holds the sum over all 32 lanes of element L / (32 / N)
// (N a power of two <= 32; the 32 / N lanes of a group hold the same total).  Each halving step exchanges half of the
// values a lane still carries, starting with the most distant partner, so 16 values cost 8 + 4 + 2 + 1 shuffles plus one
// for the last lane bit; the order of the additions is fixed, hence reproducible.
template <int N>
OEQ_DEV void warp_reduce_transpose(T (&v)[N], int lane) {
    int d = 16;
#pragma unroll
    for (int h = N / 2; h >= 1; h >>= 1, d >>= 1) {
        const bool up = (lane & d) != 0;
#pragma unroll
        for (int t = 0; t < h; ++t) {
            const T send = up ? v[t] : v[t + h];
            const T keep = up ? v[t + h] : v[t];
            v[t] = keep + __shfl_xor_sync(0xffffffffu, send, d);
        }
    }
#pragma unroll
    for (; d >= 1; d >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], d);
}

// ---- work split -------------------------------------------------------------------------------------------
// Edge / receiver range of a CTA.  Deterministic forward: ranges are snapped to receiver boundaries (a receiver's
// edges never straddle two CTAs) and together cover every receiver, including those without edges.
template <int KIND, bool SNAP>
OEQ_DEV void cta_range(const FastParams& p, long long* out, const int stream) {
    const long long G = (long long)gridDim.x * FAST_V, b = (long long)blockIdx.x * FAST_V + stream;
    long long e0 = (p.E * b) / G, e1 = (p.E * (b + 1)) / G, n0 = 0, n1 = 0;
    if (KIND == FAST_DET && SNAP) {
        auto row_at = [&](long long k) { return (long long)p.rows[p.eorder ? (long long)p.eorder[k] : k]; };
        n0 = (e0 == 0) ? 0 : row_at(e0 - 1) + 1;
        n1 = (b == G - 1) ? p.N : ((e1 == 0) ? 0 : row_at(e1 - 1) + 1);
        e0 = lower_bound_ll(p.E, n0, row_at);
        e1 = lower_bound_ll(p.E, n1, row_at);
    }
    out[0] = e0; out[1] = e1; out[2] = n0; out[3] = n1;
}

// ---- producer ---------------------------------------------------------------------------------------------
template <int KIND, bool BWD>
OEQ_DEV void fast_producer(const FastParams& p, FastShared& sh, int lane, const int pid) {
    static_assert(FAST_D % FAST_NP == 0 && FAST_NP < FAST_S, "a producer looks ahead in units of its own edges");
    const long long e0 = sh.range[0], n = sh.range[1] - sh.range[0];
    volatile int* abortf = &sh.abort_flag;
    const unsigned long long pol_stream = l2_evict_first();
    IDX colv = 0, rowv = 0, rown = 0, eidv = 0;
    // this lane's share of the coefficient table stays in registers for the whole kernel
    // (with several edge streams per CTA the producer warps run on a small register budget and read the table from
    // memory, where it stays in the L1, every time)
    constexpr int CY_PER_LANE = (NCY + 31) / 32;
    constexpr bool TAB_IN_REGS = FAST_V == 1;
    T tab_c[TAB_IN_REGS ? CY_PER_LANE : 1][FAST_CYT];
    int tab_j[TAB_IN_REGS ? CY_PER_LANE : 1][FAST_CYT];
    if (TAB_IN_REGS) {
#pragma unroll
        for (int t = 0; t < CY_PER_LANE; ++t) {
            const int q = lane + 32 * t;
#pragma unroll
            for (int m = 0; m < FAST_CYT; ++m) {
                tab_c[TAB_IN_REGS ? t : 0][m] = (q < NCY) ? FAST_CYC[q * FAST_CYT + m] : T(0);
                tab_j[TAB_IN_REGS ? t : 0][m] = (q < NCY) ? FAST_CYJ[q * FAST_CYT + m] : 0;
            }
        }
    }

    // Ring positions of the three phases (stage and use parity of the edge each will handle next): walked with counters,
    // the producer shares its scheduler with consumer warps and should not spend issue slots on 64-bit divisions.
    struct RingPos {
        int s; unsigned par;
        OEQ_DEV void next() { s += FAST_NP; if (s >= FAST_S) { s -= FAST_S; par ^= 1u; } }
    };
    RingPos pos_a{pid, 0u}, pos_b{pid, 0u}, pos_c{pid, 0u};   // this producer's edges are pid, pid + FAST_NP, ...
    long long cur_blk = -1, prefetched_row = -1;

    auto phase_a = [&](long long ia) -> bool {   // claim a stage for edge ia and start its copies
        const int s = pos_a.s;
        const unsigned par_prev = pos_a.par ^ 1u;   // parity of the stage's previous use
        pos_a.next();
        FastStage& st = sh.st[s];
        long long e = e0 + ia;                           // position in the list; below: the edge's id
        if ((ia >> 5) != cur_blk && KIND != FAST_TP) {   // indices of 32 consecutive edges, one per lane
            cur_blk = ia >> 5;
            const long long me = e0 + (cur_blk << 5) + lane;
            if (p.eorder) {
                const IDX id = (me < p.E) ? p.eorder[me] : (IDX)0;
                const IDX idn = (me + 1 < p.E) ? p.eorder[me + 1] : (IDX)0;
                eidv = id;
                colv = (me < p.E) ? p.cols[id] : (IDX)0;
                rowv = (me < p.E) ? p.rows[id] : (IDX)0;
                rown = (me + 1 < p.E) ? p.rows[idn] : (IDX)-1;
            } else {
                colv = (me < p.E) ? p.cols[me] : (IDX)0;
                rowv = (me < p.E) ? p.rows[me] : (IDX)0;
                rown = (me + 1 < p.E) ? p.rows[me + 1] : (IDX)-1;
            }
        }
        long long col = e, row = e, nxt = -1;
        if (KIND != FAST_TP) {
            col = (long long)__shfl_sync(0xffffffffu, colv, (int)(ia & 31));
            row = (long long)__shfl_sync(0xffffffffu, rowv, (int)(ia & 31));
            nxt = (long long)__shfl_sync(0xffffffffu, rown, (int)(ia & 31));
            if (p.eorder) e = (long long)__shfl_sync(0xffffffffu, eidv, (int)(ia & 31));
        }
        if (ia >= FAST_S) {
            if (!BWD) {
                if (!mbar_wait(&sh.empty[s], par_prev, abortf, p.status, 11)) return false;
            } else if (FAST_NP == 1) {
                tma_wait_read<FAST_S - FAST_D - 1>();   // the stage's previous dX row has left shared memory
            } else {
                // FAST_S is odd or even, so the stage's previous edge may have been drained by the other producer warp
                if (!mbar_wait(&sh.drained[s], par_prev, abortf, p.status, 13)) return false;
            }
        }
        if (lane == 0) {
            if (BWD && KIND != FAST_TP && row != prefetched_row) {
                // a receiver the consumers will reach in a few edges: bring its gradient row into the L2 now
                l2_prefetch(p.G + row * L3_DIM, (unsigned)(L3_DIM * sizeof(T)));
                prefetched_row = row;
            }
            st.edge = e; st.row = row; st.col = col;
            st.first = (ia == 0) || (KIND == FAST_TP);   // consumers also compare rows; see fast_backward
            st.last = (ia == n - 1) || (row != nxt) || (KIND == FAST_TP);
            mbar_arrive_expect_tx(&sh.full[s], (unsigned)((L1_DIM + WN) * sizeof(T)));
            // weight rows are read once: they should leave the L2 before the sender rows, which neighbouring receivers reuse
            if (KIND == FAST_TP) tma_load_hint(st.x, p.X + col * L1_DIM, (unsigned)(L1_DIM * sizeof(T)), &sh.full[s], pol_stream);
            else tma_load(st.x, p.X + col * L1_DIM, (unsigned)(L1_DIM * sizeof(T)), &sh.full[s]);
            tma_load_hint(st.w, p.W + e * WN, (unsigned)(WN * sizeof(T)), &sh.full[s], pol_stream);
            // second-order kernels: the rows of X2 and W2 are read by the consumers straight from global memory (staging
            // them too would leave room for two stages only); bring them into the L2 ahead of the consumers
            if (FAST_DBL) {
                l2_prefetch(p.W2 + e * WN, (unsigned)(WN * sizeof(T)));
                l2_prefetch(p.X2 + col * L1_DIM, (unsigned)(L1_DIM * sizeof(T)));
            }
        }
        for (int j = lane; j < L2_DIM; j += 32) ldgsts4(&st.y[j], p.Y + e * L2_DIM + j);
        if (FAST_DBL)
            for (int j = lane; j < L2_DIM; j += 32) ldgsts4(&st.y2[j], p.Y2 + e * L2_DIM + j);
        ldgsts_commit();
        return true;
    };
    auto phase_b = [&](long long i) {            // Y[e] has landed: fold it into the coefficients, publish the stage
        const int sb = pos_b.s;
        pos_b.next();
        FastStage& st = sh.st[sb];
        // copies are committed one group per edge, FAST_D edges ahead; near the end of the range fewer are in flight
        if (i + FAST_D - FAST_NP < n) ldgsts_wait<FAST_D / FAST_NP - 1>(); else ldgsts_wait<0>();
        __syncwarp();
#pragma unroll
        for (int t = 0; t < (FAST_CFOLD ? 0 : CY_PER_LANE); ++t) {
            const int q = lane + 32 * t;
            if (q < NCY) {
                T tc[FAST_CYT];
                int tj[FAST_CYT];
#pragma unroll
                for (int m = 0; m < FAST_CYT; ++m) {
                    tc[m] = TAB_IN_REGS ? tab_c[TAB_IN_REGS ? t : 0][m] : __ldg(&FAST_CYC[q * FAST_CYT + m]);
                    tj[m] = TAB_IN_REGS ? tab_j[TAB_IN_REGS ? t : 0][m] : __ldg(&FAST_CYJ[q * FAST_CYT + m]);
                }
                T v = tc[0] * st.y[tj[0]];
#pragma unroll
                for (int m = 1; m < FAST_CYT; ++m) v = oeq_fma(tc[m], st.y[tj[m]], v);
                st.cy[q] = v;
                if (FAST_DBL) {
                    T v2 = tc[0] * st.y2[tj[0]];
#pragma unroll
                    for (int m = 1; m < FAST_CYT; ++m) v2 = oeq_fma(tc[m], st.y2[tj[m]], v2);
                    st.cy2[FAST_DBL ? q : 0] = v2;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.full[sb]);
    };
    auto phase_c = [&](long long j) -> bool {    // backward only: drain the outputs of a finished edge
        const int s = pos_c.s;
        const unsigned par = pos_c.par;
        pos_c.next();
        FastStage& st = sh.st[s];
        if (!mbar_wait(&sh.empty[s], par, abortf, p.status, 12)) return false;
        if (lane < L2_DIM) {
            T tot = T(0);
#pragma unroll
            for (int w = 0; w < FAST_NCW; ++w) tot += st.dyp[w][lane];
            T* dst = p.dY + st.edge * L2_DIM + lane;
            *dst = tot;
        }
        if (lane == 0) {
            T* row = (KIND == FAST_TP) ? p.dX + st.edge * L1_DIM : (KIND == FAST_DET) ? p.scratch + st.edge * L1_DIM
                                                                                        : p.dX + st.col * L1_DIM;
            if (KIND == FAST_ATOMIC) tma_reduce_add(row, st.x, (unsigned)(L1_DIM * sizeof(T)));
            else tma_store_hint(row, st.x, (unsigned)(L1_DIM * sizeof(T)), pol_stream);
        }
        tma_commit();
        if (FAST_NP == 2) {   // tell whichever producer reuses the stage that the row has been read out
            tma_wait_read<0>();
            if (lane == 0) mbar_arrive(&sh.drained[s]);
        }
        return true;
    };

    bool ok = true;
    long long i = pid - (long long)FAST_D;
    for (; i < n && ok; i += FAST_NP) {
        if (i >= 0) phase_b(i);
        if (BWD && i >= FAST_NP) ok = phase_c(i - FAST_NP);
        if (ok && i + FAST_D < n) ok = phase_a(i + FAST_D);
    }
    if (BWD) {
        if (ok && i - FAST_NP >= 0) ok = phase_c(i - FAST_NP);   // this producer's last edge
        tma_wait_all<0>();
    }
    ldgsts_wait<0>();
}


// ---- a thread's slice of a row -----------------------------------------------------------------------------
// Thread u carries channels u + ch * FAST_GT; a block's values are kept as v[ch * D + i].  (Giving a thread two
// neighbouring channels and moving them with 8-byte accesses was measured: no faster.)
OEQ_DEV int chan(int u, int ch) { return u + ch * FAST_GT; }
template <class BLK>
OEQ_DEV void block_load(const T* row, int u, T* v) {
#pragma unroll
    for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
        for (int i = 0; i < BLK::D; ++i) v[ch * BLK::D + i] = row[feat_idx<BLK::OFF, BLK::MUL, BLK::D>(chan(u, ch), i)];
}
// the reverse; ADD: add to what the row holds; STREAM: global row that is not read again soon (evict-first stores).
// a(ch, i) yields the value of channel ch, component i.
template <class BLK, bool ADD, bool STREAM, class F>
OEQ_DEV void block_store(T* row, int u, F&& a) {
#pragma unroll
    for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
        for (int i = 0; i < BLK::D; ++i) {
            T* dst = row + feat_idx<BLK::OFF, BLK::MUL, BLK::D>(chan(u, ch), i);
            const T t = ADD ? *dst + a(ch, i) : a(ch, i);
            if (STREAM) __stcs(dst, t); else *dst = t;
        }
}
template <int WOFF>
OEQ_DEV void weight_load(const T* w, int u, T* wv) {
#pragma unroll
    for (int ch = 0; ch < FAST_CH; ++ch) wv[ch] = w[WOFF + chan(u, ch)];
}

// ---- forward ----------------------------------------------------------------------------------------------
// Consumer thread t: group t / FAST_GT, channels chan(u, ch) (u = t % FAST_GT, ch < FAST_CH).  The folded
// coefficients are the same for every channel, so a thread that carries two channels reads them from shared memory
// once for both: that halves the load on the shared-memory pipe, which is what limits these kernels.  A group owns a
// subset of the output blocks (forward) or of the input blocks (backward) and runs only the paths that touch its
// blocks, which keeps the per-thread row registers at the single-channel level.
template <int KIND, int GRP>
OEQ_DEV void fast_forward_group(const FastParams& p, FastShared& sh, const int tid, const FastTabEntry* tab) {
    const int u = tid % FAST_GT;   // channel ch of this thread is chan(u, ch)
    const long long n = sh.range[1] - sh.range[0];
    volatile int* abortf = &sh.abort_flag;
    T acc[FAST_CH * FAST_GPC];
#pragma unroll
    for (int k = 0; k < FAST_CH * FAST_GPC; ++k) acc[k] = T(0);
#if OEQ_KAHAN
    // Compensated summation over a receiver's edges (the reference's Kahan option of the deterministic convolution:
    // templates/loop_unroll_conv_det.cuh): the edge's message for one output block at a time is formed in msg and added
    // to (acc, comp).  One channel per thread (the wide configuration), so sum and compensation fit the registers.
    static_assert(FAST_CH == 1 && !FAST_FWD3, "compensated summation runs on the one-channel first-order kernels");
    T comp[FAST_GPC];
#pragma unroll
    for (int k = 0; k < FAST_GPC; ++k) comp[k] = T(0);
#endif
    long long next_row = sh.range[2];
    long long nseg = 0;                                // receiver rows this CTA has handed to the bulk reduce
    auto zero_rows = [&](long long a, long long b) {   // receivers without edges
        for (long long r = a; r < b; ++r)
            for (int q = tid; q < L3_DIM; q += FAST_NT) p.Z[r * L3_DIM + q] = T(0);
    };
    int s = -1;          // stage of edge i and the parity of its use: the ring is walked with counters, not divisions
    unsigned par = 1;
    for (long long i = 0; i < n; ++i) {
        if (++s == FAST_S) s = 0;
        par ^= (s == 0);
        FastStage& st = sh.st[s];
        if (!mbar_wait(&sh.full[s], par, abortf, p.status, 21)) return;
        if (!fast_consumer_fold(sh, st, tab, s, par, tid, abortf, p.status)) return;
        const long long row = st.row;
        const int last = st.last;
        const T4* cy4 = reinterpret_cast<const T4*>(st.cy);
#if OEQ_KAHAN
        // Paths are taken output block by output block: the block's message of this edge is complete before it is added.
        static_for<0, NB3>([&](auto oc) {
            constexpr int O = decltype(oc)::value;
            using B3 = Blk3<O>;
            if constexpr (FP_Z_OWNER[O] == GRP) {
                T msg[B3::D];
#pragma unroll
                for (int k = 0; k < B3::D; ++k) msg[k] = T(0);
                static_for<0, NINS>([&](auto ic) {
                    constexpr int I = decltype(ic)::value;
                    using F = FIns<I>;
                    if constexpr (F::OB == O) {
                        using B1 = Blk1<F::A>;
                        T xb[B1::D], wv[1];
                        block_load<B1>(st.x, u, xb);
                        weight_load<F::WOFF>(st.w, u, wv);
                        F::fwd(xb, cy4, wv, msg);
                    }
                });
#pragma unroll
                for (int k = 0; k < B3::D; ++k) {
                    T& a = acc[B3::OFF / FU + k];
                    T& c = comp[B3::OFF / FU + k];
                    const T yk = msg[k] - c;
                    const T tk = a + yk;
                    c = (tk - a) - yk;
                    a = tk;
                }
            }
        });
#else
        // Paths are taken input block by input block, so that only one block of the sender row is in registers at a time.
        static_for<0, NB1>([&](auto bc) {
            constexpr int B = decltype(bc)::value;
            using B1 = Blk1<B>;
            if constexpr ((GRP == 0 ? FP_FWD_NEEDS_X0[B] : FP_FWD_NEEDS_X1[B]) != 0) {
                T xb[FAST_CH * B1::D];
                block_load<B1>(st.x, u, xb);
#if FAST_FWD3
                T x2b[FAST_CH * B1::D];
                {
                    const T* x2row = p.X2 + st.col * L1_DIM;
#pragma unroll
                    for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
                        for (int i1 = 0; i1 < B1::D; ++i1)
                            x2b[ch * B1::D + i1] = __ldg(x2row + feat_idx<B1::OFF, B1::MUL, B1::D>(chan(u, ch), i1));
                }
                const T4* cy4b = reinterpret_cast<const T4*>(st.cy2);
                const T* w2row = p.W2 + st.edge * WN;
#endif
                static_for<0, NINS>([&](auto ic) {
                    constexpr int I = decltype(ic)::value;
                    using F = FIns<I>;
                    if constexpr (F::A == B && FP_INS_GF[I] == GRP) {
                        T wv[FAST_CH];
                        weight_load<F::WOFF>(st.w, u, wv);
#if FAST_FWD3
                        T w2v[FAST_CH];
#pragma unroll
                        for (int ch = 0; ch < FAST_CH; ++ch) w2v[ch] = __ldg(w2row + F::WOFF + chan(u, ch));
                        F::fwd3(xb, x2b, cy4, cy4b, wv, w2v, acc + F::GO);
#else
                        F::fwd(xb, cy4, wv, acc + F::GO);
#endif
                    }
                });
            }
        });
#endif
        mbar_arrive(&sh.empty[s]);
        if (last && KIND == FAST_ATOMIC) {
            // The row is added to Z[row] by one bulk reduce (cp.reduce.async.bulk) out of shared memory: far fewer
            // L2 atomic transactions than one red per element.  zfree/zfull hand the staging row back and forth
            // between the consumer threads and the thread that issues the copy.
            if (nseg > 0 && !mbar_wait(&sh.zfree, (unsigned)((nseg - 1) & 1), abortf, p.status, 23)) return;
            static_for<0, NB3>([&](auto oc) {
                constexpr int O = decltype(oc)::value;
                using B3 = Blk3<O>;
                if constexpr (FP_Z_OWNER[O] == GRP) {
                    block_store<B3, false, false>(sh.zbuf, u, [&](int ch, int k) { return acc[ch * FAST_GPC + B3::OFF / FU + k]; });
#pragma unroll
                    for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
                        for (int k = 0; k < B3::D; ++k) acc[ch * FAST_GPC + B3::OFF / FU + k] = T(0);
                }
            });
            fence_async_smem();
            mbar_arrive(&sh.zfull);
            if (tid == 0) {
                if (!mbar_wait(&sh.zfull, (unsigned)(nseg & 1), abortf, p.status, 24)) return;
                tma_reduce_add(p.Z + row * L3_DIM, sh.zbuf, (unsigned)(L3_DIM * sizeof(T)));
                tma_commit();
                tma_wait_read<0>();
                mbar_arrive(&sh.zfree);
            }
            ++nseg;
        } else if (last) {
            if (KIND == FAST_DET && !p.accum) { zero_rows(next_row, row); next_row = row + 1; }
            T* zrow = p.Z + row * L3_DIM;
            static_for<0, NB3>([&](auto oc) {
                constexpr int O = decltype(oc)::value;
                using B3 = Blk3<O>;
                if constexpr (FP_Z_OWNER[O] == GRP) {
                    auto val = [&](int ch, int k) { return acc[ch * FAST_GPC + B3::OFF / FU + k]; };
                    if (KIND == FAST_ATOMIC) {
#pragma unroll
                        for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
                            for (int k = 0; k < B3::D; ++k)
                                atomicAdd(zrow + feat_idx<B3::OFF, B3::MUL, B3::D>(chan(u, ch), k), val(ch, k));
                    } else if (p.accum) {
                        block_store<B3, true, false>(zrow, u, val);
                    } else {
                        block_store<B3, false, true>(zrow, u, val);
                    }
#pragma unroll
                    for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
                        for (int k = 0; k < B3::D; ++k) acc[ch * FAST_GPC + B3::OFF / FU + k] = T(0);
#if OEQ_KAHAN
#pragma unroll
                    for (int k = 0; k < B3::D; ++k) comp[B3::OFF / FU + k] = T(0);
#endif
                }
            });
        }
    }
    if (KIND == FAST_DET && !p.accum) zero_rows(next_row, sh.range[3]);
    if (KIND == FAST_ATOMIC && tid == 0) tma_wait_all<0>();
}

// Role split of a CTA: threads [0, FAST_V * FAST_NT) are the consumers of stream tid / FAST_NT, the warps behind them the
// producers (FAST_V == 1: FAST_NP of them for the one stream; else one per stream out of a warpgroup of four).
OEQ_DEV void fast_regs_producer() {
    if (FAST_V > 1) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FAST_REG_PRODUCER));
}
OEQ_DEV void fast_regs_consumer() {
    if (FAST_V > 1) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FAST_REG_CONSUMER));
}

template <int KIND>
OEQ_DEV void fast_forward_body(const FastParams& p) {
    extern __shared__ __align__(16) unsigned char fast_smem_raw[];
    FastShared* shs = reinterpret_cast<FastShared*>(fast_smem_raw);
    const int tid = threadIdx.x, lane = tid & 31;
    if (tid < FAST_V) {   // thread v sets up stream v
        FastShared& sh = shs[tid];
        for (int s = 0; s < FAST_S; ++s) { mbar_init(&sh.full[s], 2); mbar_init(&sh.empty[s], FAST_NT); }
        for (int s = 0; s < (FAST_CFOLD ? FAST_S : 0); ++s) mbar_init(&sh.folded[s], FAST_NT);
        mbar_init(&sh.zfull, FAST_NT);
        mbar_init(&sh.zfree, 1);
        sh.abort_flag = 0;
        cta_range<KIND, true>(p, sh.range, tid);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fast_tab_fill(fast_smem_raw);
    __syncthreads();
    if (tid >= FAST_V * FAST_NT) {
        fast_regs_producer();
        const int pw = (tid - FAST_V * FAST_NT) >> 5;
        if (pw < FAST_V * FAST_NP) fast_producer<KIND, false>(p, shs[pw / FAST_NP], lane, pw % FAST_NP);
        return;
    }
    fast_regs_consumer();
    FastShared& sh = shs[tid / FAST_NT];
    const int ltid = tid % FAST_NT;
    const FastTabEntry* tab = fast_tab(fast_smem_raw);
    if (FAST_NG == 1 || ltid < FAST_GT) fast_forward_group<KIND, 0>(p, sh, ltid, tab); else fast_forward_group<KIND, 1>(p, sh, ltid, tab);
}

// ---- backward ---------------------------------------------------------------------------------------------
template <int KIND, int GRP>
OEQ_DEV void fast_backward_group(const FastParams& p, FastShared& sh, const int tid, const FastTabEntry* tab) {
    const int u = tid % FAST_GT, lane = tid & 31, warp = tid >> 5;
    const long long n = sh.range[1] - sh.range[0];
    volatile int* abortf = &sh.abort_flag;
    T g[FAST_CH * FAST_GPC];
    long long cur_row = -1;
    int s = -1;
    unsigned par = 1;
    for (long long i = 0; i < n; ++i) {
        if (++s == FAST_S) s = 0;
        par ^= (s == 0);
        FastStage& st = sh.st[s];
        if (!mbar_wait(&sh.full[s], par, abortf, p.status, 22)) return;
        if (!fast_consumer_fold(sh, st, tab, s, par, tid, abortf, p.status)) return;
        const long long row = st.row, e = st.edge;
        if (row != cur_row) {   // new receiver: its gradient row goes to registers for all of its edges
            const T* grow = p.G + row * L3_DIM;
            static_for<0, NB3>([&](auto oc) {
                constexpr int O = decltype(oc)::value;
                using B3 = Blk3<O>;
                if constexpr ((GRP == 0 ? FP_BWD_NEEDS_G0[O] : FP_BWD_NEEDS_G1[O]) != 0) {
#pragma unroll
                    for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
                        for (int k = 0; k < B3::D; ++k)
                            g[ch * FAST_GPC + B3::OFF / FU + k] = __ldcs(grow + feat_idx<B3::OFF, B3::MUL, B3::D>(chan(u, ch), k));
                }
            });
            cur_row = row;
        }
        T dyr[FAST_NYP];
#pragma unroll
        for (int j = 0; j < FAST_NYP; ++j) dyr[j] = T(0);
        const T4* cy4 = reinterpret_cast<const T4*>(st.cy);
        T* dwrow = p.dW + e * WN;
        // second-order backward: this thread's entries of the W2 row, all requested now and used path by path
        T wdxv[FAST_DBL ? FAST_CH * NINS : 1];
        const T4* cy4b = reinterpret_cast<const T4*>(st.cy2);
        if (FAST_DBL) {
            const T* wdxrow = p.W2 + e * WN;
            static_for<0, NINS>([&](auto ic) {
                constexpr int I = decltype(ic)::value;
                if constexpr (FP_INS_GB[I] == GRP) {
#pragma unroll
                    for (int ch = 0; ch < FAST_CH; ++ch) wdxv[FAST_DBL ? ch * NINS + I : 0] = __ldg(wdxrow + FIns<I>::WOFF + chan(u, ch));
                }
            });
        }
        // Paths are taken input block by input block: one block of x and of dx is in registers at a time, and the
        // block's dx overwrites its x in the stage as soon as its paths are done.
        static_for<0, NB1>([&](auto bc) {
            constexpr int B = decltype(bc)::value;
            using B1 = Blk1<B>;
            if constexpr (FP_X_OWNER[B] == GRP) {
                T xb[FAST_CH * B1::D], dxb[FAST_CH * B1::D];
                block_load<B1>(st.x, u, xb);
#pragma unroll
                for (int q = 0; q < FAST_CH * B1::D; ++q) dxb[q] = T(0);
#if FAST_DBL
                T x2b[FAST_CH * B1::D];
                {
                    const T* x2row = p.X2 + st.col * L1_DIM;
#pragma unroll
                    for (int ch = 0; ch < FAST_CH; ++ch)
#pragma unroll
                        for (int i1 = 0; i1 < B1::D; ++i1)
                            x2b[ch * B1::D + i1] = __ldg(x2row + feat_idx<B1::OFF, B1::MUL, B1::D>(chan(u, ch), i1));
                }
#endif
                static_for<0, NINS>([&](auto ic) {
                    constexpr int I = decltype(ic)::value;
                    using F = FIns<I>;
                    if constexpr (F::A == B && FP_INS_GB[I] == GRP) {
                        T wv[FAST_CH], wx[FAST_CH], dw[FAST_CH];
#pragma unroll
                        for (int ch = 0; ch < FAST_CH; ++ch) {
                            wv[ch] = st.w[F::WOFF + chan(u, ch)];
                            wx[ch] = FAST_DBL ? wdxv[FAST_DBL ? ch * NINS + I : 0] : wv[ch];
                        }
#if FAST_DBL
                        F::bwd3(xb, x2b, g + F::GO, cy4, cy4b, wv, wx, dxb, dyr + F::Y0, dw);
#else
                        F::bwd(xb, g + F::GO, cy4, wv, wx, dxb, dyr + F::Y0, dw);
#endif
#pragma unroll
                        for (int ch = 0; ch < FAST_CH; ++ch) __stcs(dwrow + F::WOFF + chan(u, ch), dw[ch]);   // written once, not read again here
                    }
                });
                block_store<B1, false, false>(st.x, u, [&](int ch, int i1) { return dxb[ch * B1::D + i1]; });
            }
        });
        warp_reduce_transpose<FAST_NYP>(dyr, lane);
        if ((lane & (32 / FAST_NYP - 1)) == 0) st.dyp[warp][lane / (32 / FAST_NYP)] = dyr[0];
        fence_async_smem();          // the dX row is read from shared memory by the async proxy (TMA)
        mbar_arrive(&sh.empty[s]);
    }
}

template <int KIND>
OEQ_DEV void fast_backward_body(const FastParams& p) {
    extern __shared__ __align__(16) unsigned char fast_smem_raw[];
    FastShared* shs = reinterpret_cast<FastShared*>(fast_smem_raw);
    const int tid = threadIdx.x, lane = tid & 31;
    if (tid < FAST_V) {   // thread v sets up stream v
        FastShared& sh = shs[tid];
        for (int s = 0; s < FAST_S; ++s) { mbar_init(&sh.full[s], 2); mbar_init(&sh.empty[s], FAST_NT); mbar_init(&sh.drained[s], 1); }
        for (int s = 0; s < (FAST_CFOLD ? FAST_S : 0); ++s) mbar_init(&sh.folded[s], FAST_NT);
        sh.abort_flag = 0;
        cta_range<KIND, false>(p, sh.range, tid);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fast_tab_fill(fast_smem_raw);
    __syncthreads();
    if (tid >= FAST_V * FAST_NT) {
        fast_regs_producer();
        const int pw = (tid - FAST_V * FAST_NT) >> 5;
        if (pw < FAST_V * FAST_NP) fast_producer<KIND, true>(p, shs[pw / FAST_NP], lane, pw % FAST_NP);
        return;
    }
    fast_regs_consumer();
    FastShared& sh = shs[tid / FAST_NT];
    const int ltid = tid % FAST_NT;
    const FastTabEntry* tab = fast_tab(fast_smem_raw);
    if (FAST_NG == 1 || ltid < FAST_GT) fast_backward_group<KIND, 0>(p, sh, ltid, tab); else fast_backward_group<KIND, 1>(p, sh, ltid, tab);
}

// ---- entry points (one per program: FAST_KERNEL selects which) ----------------------------------------------
// Kernel names carry "forward" / "backward" / "double_backward" like the reference's (its profiling helpers and stream
// tests select kernels by those substrings: core/utils.py:174-203, tests/stream_test.py:97-319).  The second-order
// programs (FAST_DBL) are the fused passes A (the three terms of dG) and B (both terms of dX, dY, dW).
#define FAST_ENTRY(NAME, BODY) \
    extern "C" __global__ void __launch_bounds__(FAST_THREADS, FAST_CTAS) NAME(const FastParams p) { BODY(p); }
#if FAST_KERNEL == 0 && !FAST_DBL
FAST_ENTRY(oeq_fast_forward_tp, fast_forward_body<FAST_TP>)
#elif FAST_KERNEL == 1 && !FAST_DBL
FAST_ENTRY(oeq_fast_forward_det, fast_forward_body<FAST_DET>)
#elif FAST_KERNEL == 2 && !FAST_DBL
FAST_ENTRY(oeq_fast_forward_atomic, fast_forward_body<FAST_ATOMIC>)
#elif FAST_KERNEL == 3 && !FAST_DBL
FAST_ENTRY(oeq_fast_backward_tp, fast_backward_body<FAST_TP>)
#elif FAST_KERNEL == 4 && !FAST_DBL
FAST_ENTRY(oeq_fast_backward_det, fast_backward_body<FAST_DET>)
#elif FAST_KERNEL == 5 && !FAST_DBL
FAST_ENTRY(oeq_fast_backward_atomic, fast_backward_body<FAST_ATOMIC>)
#elif FAST_KERNEL == 0
FAST_ENTRY(oeq_fast_double_backward_A_tp, fast_forward_body<FAST_TP>)
#elif FAST_KERNEL == 1
FAST_ENTRY(oeq_fast_double_backward_A_det, fast_forward_body<FAST_DET>)
#elif FAST_KERNEL == 3
FAST_ENTRY(oeq_fast_double_backward_B_tp, fast_backward_body<FAST_TP>)
#elif FAST_KERNEL == 4
FAST_ENTRY(oeq_fast_double_backward_B_det, fast_backward_body<FAST_DET>)
#elif FAST_KERNEL == 5
FAST_ENTRY(oeq_fast_double_backward_B_atomic, fast_backward_body<FAST_ATOMIC>)
#elif FAST_KERNEL == 6
// Self-test of the bounded wait that every pipeline stage of this file relies on: a CTA waits on a barrier that nobody
// arrives at.  The wait has to give up by itself, raise the CTA's abort flag and leave its code in the status word; the
// threads that did not run out themselves leave through the flag.  *left counts the threads that came back.
extern "C" __global__ void oeq_selftest_starved_wait(int* status, int* left) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (!mbar_wait(&bar, 0u, &abort_flag, status, 99)) atomicAdd(left, 1);
}
// Deterministic scatter of the per-edge dX rows: colptr[c] = first position k (in sender-major order) whose sender >= c
extern "C" __global__ void oeq_fixup_backward_offsets(const IDX* cols, const IDX* perm, long long E, long long N, long long* colptr) {
    const long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (k > E) return;
    const long long prev = (k == 0) ? -1 : (long long)cols[perm[k - 1]];
    const long long cur = (k == E) ? N : (long long)cols[perm[k]];
    for (long long c = prev + 1; c <= cur; ++c) colptr[c] = k;
}
// dX[c] = sum over the sender's edges, in sender-major list order, of the per-edge rows in scratch
// (senders [c_begin, c_end): a partitioned caller reduces the rows it has to send away first)
extern "C" __global__ void __launch_bounds__(256) oeq_fixup_backward_reduce(const T* scratch, const IDX* perm, const long long* colptr,
                                                                     long long c_begin, long long c_end, T* dX) {
    constexpr int VE = 16 / sizeof(T);          // elements per 16-byte piece
    constexpr int NQ = L1_DIM / VE;
    struct __align__(16) Piece { T v[VE]; };
    auto load = [&](long long e, int q) { return __ldcs(reinterpret_cast<const float4*>(scratch + e * L1_DIM) + q); };
    for (long long c = c_begin + blockIdx.x; c < c_end; c += gridDim.x) {
        const long long k0 = colptr[c], k1 = colptr[c + 1];
        for (int q = threadIdx.x; q < NQ; q += 256) {
            Piece acc;
#pragma unroll
            for (int t = 0; t < VE; ++t) acc.v[t] = T(0);
#if OEQ_KAHAN
            Piece comp;   // compensated summation over the sender's edges
#pragma unroll
            for (int t = 0; t < VE; ++t) comp.v[t] = T(0);
#endif
            auto add = [&](const float4& raw) {
                const Piece& pc = reinterpret_cast<const Piece&>(raw);
#pragma unroll
                for (int t = 0; t < VE; ++t) {
#if OEQ_KAHAN
                    const T yk = pc.v[t] - comp.v[t];
                    const T tk = acc.v[t] + yk;
                    comp.v[t] = (tk - acc.v[t]) - yk;
                    acc.v[t] = tk;
#else
                    acc.v[t] += pc.v[t];
#endif
                }
            };
            long long k = k0;
            for (; k + 4 <= k1; k += 4) {
                const long long ea = perm[k], eb = perm[k + 1], ec = perm[k + 2], ed = perm[k + 3];
                const float4 a = load(ea, q), b = load(eb, q), cc = load(ec, q), d = load(ed, q);
                add(a); add(b); add(cc); add(d);
            }
            for (; k < k1; ++k) add(load((long long)perm[k], q));
            reinterpret_cast<Piece*>(dX + c * L1_DIM)[q] = acc;
        }
    }
}
#endif

#endif  // OEQ_FAST
